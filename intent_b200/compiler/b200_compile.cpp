// b200-compile: the native compile step of the "b200" provider.
//
// It honours the command line and exit codes of the reference's
// `intent-compile` driver (tools/intent-compile/intent-compile.cpp:37-178,
// include/Intent/Compiler/Compiler.h:17-21) so the reference's Python driver
// (python/intent/compiler/toolchain.py:97-242) can run it unchanged:
//
//   b200-compile --compiler-info
//   b200-compile --target=b200 --target-options=JSON [--numerics=.. --optimization-remarks=..
//                --optimization=NAME=BOOL ..] [--input-stage=kir|shared]
//                --ir-output=F --source-output=F --metadata-output=F  -
//
// Kernel IR arrives as generic-form MLIR text on stdin.  There is no tile
// compiler behind this step: the module is classified STRUCTURALLY (operation
// multiset, operator kinds, element types, parameter shapes — never the
// kernel's name, doc/getting-started/configuration.en.md:7) into one of the
// operator families, each of which has a hand-written sm_100a kernel in
// libintent_b200.so.  Anything else is refused with the provider_pipeline exit
// code; there is no fallback.  Outputs: the IR echoed back, a small launch
// descriptor as "source", and artifact.json in the NativeABI flavour
// (python/intent/runtime/native.py:77-130, lib/Serialization/NativeABI.cpp:14-118).
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

namespace {

enum ExitCode { kInvocation = 1, kKernelIR = 2, kConstruction = 3, kSharedPipeline = 4,
                kUnavailableProvider = 5, kProviderPipeline = 6, kTranslation = 7, kOutput = 8 };

const char *kFailureStages =
    "{\"1\": \"compiler_invocation\", \"2\": \"kernel_ir\", \"3\": \"physical_program\", "
    "\"4\": \"shared_pipeline\", \"5\": \"provider_program\", \"6\": \"provider_pipeline\", "
    "\"7\": \"terminal_translation\", \"8\": \"compiler_output\"}";

struct Failure {
  int code;
  std::string message;
};

[[noreturn]] void fail(int code, const std::string &message) { throw Failure{code, message}; }

// ---------------------------------------------------------------- parameters
struct Stride {
  enum Kind { kFree, kFixed, kSymbol } kind = kFree;
  long long value = 0;
  std::string symbol;
};

struct Parameter {
  enum Kind { kView, kScalar, kConstexpr } kind = kScalar;
  std::string name, dtype, ssa;
  int declared_position = 0;
  std::vector<long long> shape;       // -1 = dynamic
  std::vector<long long> dimensions;  // logical dimension identities
  std::vector<Stride> strides;
  int access = 0;
  std::string alias;
  bool noalias = false;
};

std::string trim(const std::string &text) {
  size_t begin = text.find_first_not_of(" \t\r\n");
  if (begin == std::string::npos) return "";
  size_t end = text.find_last_not_of(" \t\r\n");
  return text.substr(begin, end - begin + 1);
}

// Splits on `separator` at bracket depth zero; quotes are opaque.
std::vector<std::string> split_top(const std::string &text, char separator) {
  std::vector<std::string> parts;
  int depth = 0;
  bool quoted = false;
  std::string current;
  for (size_t i = 0; i < text.size(); ++i) {
    const char c = text[i];
    if (quoted) {
      current += c;
      if (c == '\\' && i + 1 < text.size()) current += text[++i];
      else if (c == '"') quoted = false;
      continue;
    }
    if (c == '"') quoted = true;
    if (c == '<' || c == '(' || c == '[' || c == '{') ++depth;
    if (c == '>' || c == ')' || c == ']' || c == '}') --depth;
    if (c == separator && depth == 0) {
      parts.push_back(current);
      current.clear();
    } else {
      current += c;
    }
  }
  if (!trim(current).empty() || !parts.empty()) parts.push_back(current);
  return parts;
}

// Returns the text between the bracket that opens at `open` and its match.
std::string bracketed(const std::string &text, size_t open) {
  const char opener = text[open];
  const char closer = opener == '<' ? '>' : opener == '(' ? ')' : opener == '[' ? ']' : '}';
  int depth = 0;
  bool quoted = false;
  for (size_t i = open; i < text.size(); ++i) {
    const char c = text[i];
    if (quoted) {
      if (c == '\\') ++i;
      else if (c == '"') quoted = false;
      continue;
    }
    if (c == '"') { quoted = true; continue; }
    if (c == opener) ++depth;
    else if (c == closer && --depth == 0) return text.substr(open + 1, i - open - 1);
  }
  fail(kKernelIR, "unbalanced brackets in kernel IR");
}

std::string after(const std::string &text, const std::string &marker, const char *what) {
  size_t at = text.find(marker);
  if (at == std::string::npos) fail(kKernelIR, std::string("kernel IR lacks ") + what);
  return text.substr(at + marker.size());
}

std::string unquote(const std::string &text) {
  std::string t = trim(text);
  if (t.size() < 2 || t.front() != '"' || t.back() != '"') fail(kKernelIR, "expected a quoted string: " + t);
  return t.substr(1, t.size() - 2);
}

void parse_view(const std::string &type, Parameter *p) {
  // !intent.view<tensor<DxDxT, #intent.tensor_shape<[ids]>>, ACCESS, #intent.view_constraints<HAS, [..], "ALIAS", NOALIAS>>
  const std::string body = bracketed(type, type.find('<'));
  std::vector<std::string> fields = split_top(body, ',');
  if (fields.size() != 3) fail(kKernelIR, "malformed view type: " + type);
  const std::string tensor = bracketed(fields[0], fields[0].find('<'));
  std::vector<std::string> tensor_fields = split_top(tensor, ',');
  if (tensor_fields.size() != 2) fail(kKernelIR, "view tensor type needs a shape encoding: " + tensor);
  std::string spec = trim(tensor_fields[0]);
  size_t cursor = 0;
  while (cursor < spec.size()) {
    size_t end = cursor;
    if (spec[end] == '?') ++end;
    else while (end < spec.size() && isdigit((unsigned char)spec[end])) ++end;
    if (end == cursor || end >= spec.size() || spec[end] != 'x') break;
    p->shape.push_back(spec[cursor] == '?' ? -1 : atoll(spec.substr(cursor, end - cursor).c_str()));
    cursor = end + 1;
  }
  p->dtype = spec.substr(cursor);
  const std::string ids = bracketed(tensor_fields[1], tensor_fields[1].find('['));
  for (const std::string &id : split_top(ids, ',')) p->dimensions.push_back(atoll(trim(id).c_str()));
  if (p->dimensions.size() != p->shape.size()) fail(kKernelIR, "dimension identities disagree with view rank");
  p->access = atoi(trim(fields[1]).c_str());
  const std::string constraints = bracketed(fields[2], fields[2].find('<'));
  std::vector<std::string> cf = split_top(constraints, ',');
  if (cf.size() != 4) fail(kKernelIR, "malformed view constraints: " + constraints);
  p->strides.assign(p->shape.size(), Stride{});
  if (trim(cf[0]) == "true") {
    std::vector<std::string> entries = split_top(bracketed(cf[1], cf[1].find('[')), ',');
    if (entries.size() != p->shape.size()) fail(kKernelIR, "stride constraints disagree with view rank");
    for (size_t axis = 0; axis < entries.size(); ++axis) {
      const std::string entry = trim(entries[axis]);
      if (entry == "unit") continue;
      if (entry[0] == '"') {
        p->strides[axis].kind = Stride::kSymbol;
        p->strides[axis].symbol = unquote(entry);
      } else {
        p->strides[axis].kind = Stride::kFixed;
        p->strides[axis].value = atoll(entry.c_str());
      }
    }
  }
  p->alias = unquote(cf[2]);
  p->noalias = trim(cf[3]) == "true";
}

std::vector<Parameter> parse_signature(const std::string &ir, std::string *function) {
  size_t at = ir.find("func.func @");
  if (at == std::string::npos) fail(kKernelIR, "kernel IR has no func.func");
  size_t name_begin = at + strlen("func.func @");
  size_t open = ir.find('(', name_begin);
  if (open == std::string::npos) fail(kKernelIR, "func.func has no parameter list");
  *function = ir.substr(name_begin, open - name_begin);
  if (ir.find("func.func @", open) != std::string::npos)
    fail(kProviderPipeline, "b200 compiles single-kernel modules only");
  std::vector<Parameter> parameters;
  for (const std::string &raw : split_top(bracketed(ir, open), ',')) {
    const std::string text = trim(raw);
    if (text.empty()) continue;
    Parameter p;
    size_t colon = text.find(':');
    if (colon == std::string::npos) fail(kKernelIR, "malformed parameter: " + text);
    p.ssa = trim(text.substr(0, colon));
    size_t attributes = text.rfind("{intent.parameter");
    if (attributes == std::string::npos) fail(kKernelIR, "parameter lacks intent.parameter: " + text);
    const std::string type = trim(text.substr(colon + 1, attributes - colon - 1));
    const std::string marker = after(text.substr(attributes), "#intent.parameter", "a parameter attribute");
    std::vector<std::string> np = split_top(bracketed(marker, marker.find('<')), ',');
    if (np.size() != 2) fail(kKernelIR, "malformed intent.parameter");
    p.name = unquote(np[0]);
    p.declared_position = atoi(trim(np[1]).c_str());
    if (type.rfind("!intent.view<", 0) == 0) {
      p.kind = Parameter::kView;
      parse_view(type, &p);
    } else if (type.rfind("!intent.constexpr<", 0) == 0) {
      p.kind = Parameter::kConstexpr;
    } else {
      p.kind = Parameter::kScalar;
      p.dtype = type;
    }
    parameters.push_back(p);
  }
  return parameters;
}

// ---------------------------------------------------------------- operations
struct Operation {
  std::string name;      // without the "intent." prefix
  std::string kind;      // operator_kind / predicate, if any
  std::string result;    // first result SSA name
  std::vector<std::string> operands;
  bool approximate = false, flush_to_zero = false;
  std::string line;
};

std::vector<Operation> parse_operations(const std::string &ir) {
  std::vector<Operation> operations;
  std::istringstream stream(ir);
  std::string line;
  while (std::getline(stream, line)) {
    size_t at = line.find("\"intent.");
    if (at == std::string::npos) continue;
    size_t end = line.find('"', at + 1);
    if (end == std::string::npos) continue;
    // an operation name is followed by its operand list
    if (end + 1 >= line.size() || line[end + 1] != '(') continue;
    Operation op;
    op.name = line.substr(at + 8, end - at - 8);
    op.line = line;
    const std::string head = trim(line.substr(0, at));
    if (!head.empty() && head[0] == '%') op.result = trim(head.substr(0, head.find_first_of(" =,:")));
    for (const std::string &operand : split_top(bracketed(line, end + 1), ','))
      if (!trim(operand).empty()) op.operands.push_back(trim(operand));
    for (const char *key : {"operator_kind = #intent.binary_operator<", "operator_kind = #intent.unary_operator<",
                            "predicate = #intent.compare_predicate<", "operator_kind = #intent.compare_operator<"}) {
      size_t k = line.find(key);
      if (k != std::string::npos) {
        size_t b = k + strlen(key);
        op.kind = line.substr(b, line.find('>', b) - b);
      }
    }
    op.approximate = line.find("approximate = true") != std::string::npos;
    op.flush_to_zero = line.find("flush_to_zero = true") != std::string::npos;
    operations.push_back(op);
  }
  return operations;
}

struct Census {
  std::map<std::string, int> count;
  int of(const std::string &key) const {
    auto found = count.find(key);
    return found == count.end() ? 0 : found->second;
  }
};

Census take_census(const std::vector<Operation> &operations) {
  Census census;
  for (const Operation &op : operations) {
    census.count[op.name]++;
    if (!op.kind.empty()) census.count[op.name + "<" + op.kind + ">"]++;
  }
  return census;
}

long long integer_constant(const std::vector<Operation> &operations, const std::string &ssa) {
  for (const Operation &op : operations)
    if (op.name == "constant" && op.result == ssa) {
      size_t at = op.line.find("value = ");
      if (at == std::string::npos) break;
      return atoll(op.line.c_str() + at + 8);
    }
  fail(kProviderPipeline, "expected " + ssa + " to be an integer constant");
}

// ---------------------------------------------------------------- structure
// The census below shortlists a family from operation counts; counts alone would also accept
// programs that merely look alike (a maximum with a non-zero constant where ReLU has zero,
// swapped operands of a subtract or divide, dy * (p - sum) for p * (dy - sum)).  So the whole
// operation graph is compared as well: the IR text is reduced to a canonical form that keeps
// every operation, attribute, constant, type and operand order but drops what an author may
// change without changing the computation (source locations, function, parameter and value
// names, static extents, the HEAD_GROUP divisor), and its hash must be one of the structures
// this provider has a kernel for (structures.inc, generated from the packaged kernel IR).
std::string strip_locations(const std::string &ir) {
  std::string out;
  out.reserve(ir.size());
  for (size_t i = 0; i < ir.size();) {
    if (ir.compare(i, 4, "loc(") == 0 && (i == 0 || !(isalnum((unsigned char)ir[i - 1]) || ir[i - 1] == '_'))) {
      int depth = 0;
      bool in_string = false;
      size_t j = i + 3;
      for (; j < ir.size(); ++j) {
        const char c = ir[j];
        if (in_string) { if (c == '\\') ++j; else if (c == '"') in_string = false; continue; }
        if (c == '"') in_string = true;
        else if (c == '(') ++depth;
        else if (c == ')' && --depth == 0) { ++j; break; }
      }
      i = j;
      continue;
    }
    out.push_back(ir[i++]);
  }
  return out;
}

std::string canonical_structure(const std::string &ir, const std::vector<Operation> &operations) {
  std::string text = strip_locations(ir);
  // the HEAD_GROUP divisor: the integer constant that is the second operand of floor_divide
  std::string divisor;
  for (const Operation &op : operations)
    if (op.name == "binary" && op.kind == "floor_divide" && op.operands.size() == 2) divisor = op.operands[1];
  auto erase_quoted_attribute = [&](const std::string &key) {
    for (size_t at = text.find(key); at != std::string::npos; at = text.find(key, at)) {
      size_t open = text.find('"', at + key.size());
      size_t close = open == std::string::npos ? open : text.find('"', open + 1);
      if (close == std::string::npos) break;
      text.erase(at, close + 1 - at);
    }
  };
  erase_quoted_attribute("intent.source_module = ");
  erase_quoted_attribute("intent.source = ");
  // local variable names the author chose: intent.result_names = ["start", ...]
  for (size_t at = text.find("intent.result_names = ["); at != std::string::npos;
       at = text.find("intent.result_names = [", at + 1)) {
    size_t open = at + strlen("intent.result_names = ");
    size_t close = text.find(']', open);
    if (close == std::string::npos) break;
    text.erase(open + 1, close - open - 1);
  }
  // static extents of the views; an integer constant equal to one of them is a loop bound or a
  // shape of the same instance and is reduced to "E" with them
  std::vector<std::string> extents;
  for (size_t at = text.find("tensor<"); at != std::string::npos; at = text.find("tensor<", at + 1)) {
    size_t j = at + 7;
    while (j < text.size()) {
      size_t k = j;
      while (k < text.size() && isdigit((unsigned char)text[k])) ++k;
      if (k > j && k < text.size() && text[k] == 'x') { extents.push_back(text.substr(j, k - j)); j = k + 1; }
      else if (text[j] == '?' && j + 1 < text.size() && text[j + 1] == 'x') j += 2;
      else break;
    }
  }
  auto is_extent = [&](const std::string &digits) {
    if (digits == "0" || digits == "1") return false;
    for (const std::string &extent : extents)
      if (extent == digits) return true;
    return false;
  };
  std::string out;
  std::map<std::string, int> names;
  for (size_t i = 0; i < text.size();) {
    const char c = text[i];
    if (c == '%') {                                         // value names, numbered by first appearance
      size_t j = i + 1;
      while (j < text.size() && (isalnum((unsigned char)text[j]) || text[j] == '_')) ++j;
      const std::string name = text.substr(i, j - i);
      auto found = names.emplace(name, (int)names.size());
      out += "%" + std::to_string(found.first->second);
      if (!divisor.empty() && name == divisor && text.compare(j, 21, " = \"intent.constant\"(") == 0) {
        size_t value = text.find("value = ", j);            // this line defines the divisor
        size_t line_end = text.find('\n', j);
        if (value != std::string::npos && value < line_end) {
          size_t digits = value + 8;
          while (digits < text.size() && isdigit((unsigned char)text[digits])) ++digits;
          out += text.substr(j, value + 8 - j) + "G";
          j = digits;
        }
      }
      i = j;
    } else if (text.compare(i, 11, "func.func @") == 0) {   // function name
      size_t j = i + 11;
      while (j < text.size() && text[j] != '(') ++j;
      out += "func.func @f";
      i = j;
    } else if (text.compare(i, 18, "#intent.parameter<") == 0) {   // parameter name, position kept
      size_t close = text.find('>', i);
      size_t comma = text.rfind(',', close);
      out += "#intent.parameter<" + trim(text.substr(comma + 1, close - comma - 1)) + ">";
      i = close + 1;
    } else if (text.compare(i, 7, "tensor<") == 0) {        // static extents -> N, dynamic stay ?
      size_t j = i + 7;
      out += "tensor<";
      while (j < text.size()) {
        size_t k = j;
        while (k < text.size() && isdigit((unsigned char)text[k])) ++k;
        if (k > j && k < text.size() && text[k] == 'x') { out += "Nx"; j = k + 1; }
        else if (text[j] == '?' && j + 1 < text.size() && text[j + 1] == 'x') { out += "?x"; j += 2; }
        else break;
      }
      i = j;
    } else if (text.compare(i, 8, "value = ") == 0 && i + 8 < text.size() && isdigit((unsigned char)text[i + 8])) {
      size_t j = i + 8;
      while (j < text.size() && isdigit((unsigned char)text[j])) ++j;
      const std::string digits = text.substr(i + 8, j - i - 8);
      out += (text.compare(j, 6, " : i64") == 0 && is_extent(digits)) ? std::string("value = E") : "value = " + digits;
      i = j;
    } else if (isspace((unsigned char)c)) {                 // runs of white space -> one blank
      if (!out.empty() && out.back() != ' ') out.push_back(' ');
      ++i;
    } else {
      out.push_back(c);
      ++i;
    }
  }
  return out;
}

unsigned long long structure_hash(const std::string &canonical) {
  unsigned long long hash = 1469598103934665603ull;         // FNV-1a
  for (unsigned char c : canonical) { hash ^= c; hash *= 1099511628211ull; }
  return hash;
}

struct KnownStructure {
  const char *family;
  unsigned long long hash;
  const char *origin;
};
const KnownStructure kKnownStructures[] = {
#include "structures.inc"
    {nullptr, 0, nullptr}};

void require_known_structure(const std::string &family, unsigned long long hash) {
  for (const KnownStructure *known = kKnownStructures; known->family; ++known)
    if (family == known->family && hash == known->hash) return;
  std::ostringstream message;
  message << "b200 has no kernel for this program: its operation counts are those of the " << family
          << " family, but its operations, constants or operand order differ from every " << family
          << " kernel this provider implements (structure " << std::hex << hash << ")";
  fail(kProviderPipeline, message.str());
}

// ---------------------------------------------------------------- the plan
struct TailConstant {
  std::string name;
  long long value;
};

struct Plan {
  std::string family, entry;
  std::vector<TailConstant> tail;  // int32 constants after the public slots
  bool workspace = false;
  int alignment = 0;               // required pointer alignment in bytes (0 = element size)
  std::vector<int> contiguous;     // interface positions that must be canonical contiguous
};

int dtype_code(const std::string &dtype) {
  if (dtype == "f32") return 0;
  if (dtype == "f16") return 1;
  if (dtype == "bf16") return 2;
  return -1;
}
int dtype_bytes(const std::string &dtype) {
  if (dtype == "f32" || dtype == "i32") return 4;
  if (dtype == "f16" || dtype == "bf16") return 2;
  if (dtype == "f64" || dtype == "i64") return 8;
  return 1;
}

void require(bool condition, const std::string &message) {
  if (!condition) fail(kProviderPipeline, "b200 has no kernel for this program: " + message);
}

bool view_is(const Parameter &p, size_t rank, int access, const std::string &dtype) {
  return p.kind == Parameter::kView && p.shape.size() == rank && p.access == access && p.dtype == dtype;
}

Plan classify(const std::vector<Parameter> &all, const std::vector<Operation> &operations) {
  const Census c = take_census(operations);
  std::vector<Parameter> p;  // runtime parameters only
  for (const Parameter &parameter : all)
    if (parameter.kind != Parameter::kConstexpr) p.push_back(parameter);
  Plan plan;
  const bool heavy = c.of("contract") || c.of("region_fold") || c.of("for") || c.of("scan") || c.of("region_scan");

  if (c.of("region_fold") == 1 && c.of("view_load") == 6 && c.of("unary<exp2>") == 1 && c.of("binary<true_divide>") == 0) {
    // ---- attention backward: dK/dV (two outputs, a record summary) or dQ (one output) ----------
    const bool key_value = c.of("view_store") == 2;
    const bool causal = c.of("compare") == 1;
    require(c.of("parallel") == 2 && c.of("unary") == 1 && c.of("transpose") == 2 && c.of("for") == 0 &&
                c.of("compare") <= 1 && (key_value ? c.of("make_record") == 4 : c.of("view_store") == 1 && c.of("make_record") == 0),
            "region_fold program is not an attention gradient summary");
    // causal programs replace the second pair of contractions by masked products with a reduction
    if (key_value) require(causal ? c.of("contract") == 2 && c.of("mask") == 3 && c.of("reduce") == 2
                                  : c.of("contract") == 4 && c.of("mask") == 0 && c.of("reduce") == 0,
                           "dK/dV summary is not K.Q^T, V.dO^T and the two gradient products");
    else require(causal ? c.of("contract") == 2 && c.of("mask") == 2 && c.of("reduce") == 1
                        : c.of("contract") == 3 && c.of("mask") == 0 && c.of("reduce") == 0,
                 "dQ summary is not Q.K^T, dO.V^T and the gradient product");
    for (const Operation &op : operations) {
      if (op.name == "unary" && op.kind == "exp2") require(op.approximate && op.flush_to_zero, "exp2 must be approximate with flush_to_zero");
      if (op.name == "compare") require(op.kind == (key_value ? "le" : "ge"), "causal mask must be key <= query");
    }
    const size_t outputs = key_value ? 2 : 1;
    require(p.size() == 7 + outputs && p.back().kind == Parameter::kScalar && p.back().dtype == "f32",
            "attention gradients take q, k, v, grad_output, lse, delta, outputs, scale");
    const std::string dtype = p[0].dtype;
    require(dtype == "f16" || dtype == "bf16", "attention gradient element type must be f16 or bf16");
    require(view_is(p[0], 4, 0, dtype) && view_is(p[1], 4, 0, dtype) && view_is(p[2], 4, 0, dtype) && view_is(p[3], 4, 0, dtype) &&
                view_is(p[4], 3, 0, "f32") && view_is(p[5], 3, 0, "f32") && view_is(p[6], 4, 1, dtype) &&
                (!key_value || view_is(p[7], 4, 1, dtype)),
            "attention gradient views must be four rank-4 inputs, lse and delta rank-3 f32, rank-4 outputs");
    long long head_group = -1;
    for (const Operation &op : operations) {
      if (key_value) {
        // group_query_count = HEAD_GROUP * Q: the first index product whose left operand is a constant
        if (head_group < 0 && op.name == "binary" && op.kind == "multiply" && op.operands.size() == 2)
          for (const Operation &other : operations)
            if (other.name == "constant" && other.result == op.operands[0]) head_group = integer_constant(operations, op.operands[0]);
      } else if (op.name == "binary" && op.kind == "floor_divide") {
        require(op.operands.size() == 2, "floor_divide arity");
        head_group = integer_constant(operations, op.operands[1]);
      }
    }
    require(head_group >= 1, "HEAD_GROUP must be a positive constant");
    plan.family = key_value ? "attention_backward_dkdv" : "attention_backward_dq";
    plan.entry = key_value ? "b200_attention_backward_dkdv" : "b200_attention_backward_dq";
    plan.tail = {{"dtype", dtype_code(dtype)}, {"head_group", head_group}, {"causal", causal}};
    plan.workspace = true;
    plan.alignment = 16;
    return plan;
  }
  if (c.of("region_fold") == 1) {
    // ---- flash attention: region_fold with Q.K^T and P.V contractions --------
    require(c.of("contract") == 2 && c.of("parallel") == 2 && c.of("transpose") == 1 && c.of("reduce") == 3 &&
                c.of("view_load") == 3 && c.of("view_store") == 1 && c.of("unary<exp2>") == 3 &&
                c.of("binary<true_divide>") == 1 && c.of("cast") == 2 && c.of("binary<maximum_num>") == 2 &&
                c.of("for") == 0 && c.of("compare") <= 1 && c.of("binary<floor_divide>") <= 1,
            "region_fold program is not the online-softmax attention summary");
    for (const Operation &op : operations) {
      if (op.name == "unary" && op.kind == "exp2") require(op.approximate && op.flush_to_zero, "exp2 must be approximate with flush_to_zero");
      if (op.name == "binary" && op.kind == "true_divide") require(op.approximate && op.flush_to_zero, "final division must be approximate with flush_to_zero");
      if (op.name == "compare") require(op.kind == "ge", "causal mask must be query >= key");
    }
    require(p.size() == 5 && p[4].kind == Parameter::kScalar && p[4].dtype == "f32", "attention takes q, k, v, output, scale");
    const std::string dtype = p[0].dtype;
    require(dtype == "bf16" || dtype == "f16", "attention element type must be bf16 or f16");
    require(view_is(p[0], 4, 0, dtype) && view_is(p[1], 4, 0, dtype) && view_is(p[2], 4, 0, dtype) && view_is(p[3], 4, 1, dtype),
            "attention views must be rank-4 In,In,In,Out of one element type");
    long long head_group = 1;
    for (const Operation &op : operations)
      if (op.name == "binary" && op.kind == "floor_divide") {
        require(op.operands.size() == 2, "floor_divide arity");
        head_group = integer_constant(operations, op.operands[1]);
      }
    require(head_group >= 1, "HEAD_GROUP must be positive");
    plan.family = "flash_attention";
    plan.entry = "b200_flash_attention";
    plan.tail = {{"dtype", dtype_code(dtype)}, {"head_group", head_group}, {"causal", c.of("compare") == 1}};
    plan.workspace = true;
    plan.alignment = 16;
    return plan;
  }
  if (c.of("contract") == 1) {
    // ---- dense GEMM: one (m,k).(k,n) contraction, narrowing cast ------------
    require(c.of("parallel") == 0 && c.of("for") == 0 && c.of("reduce") == 0 && c.of("view_load") == 2 &&
                c.of("view_store") == 1 && c.of("cast") == 1 && c.of("transpose") == 0 && c.of("unary") == 0 &&
                c.of("binary") == c.of("binary<maximum>") && c.of("binary<maximum>") <= 1,
            "contraction program is not cast(matmul(a, b)) with optional ReLU");
    require(p.size() == 3, "gemm takes a, b, c");
    const std::string dtype = p[0].dtype;
    require(dtype == "f16" || dtype == "bf16", "gemm element type must be f16 or bf16 (f32 accumulate)");
    require(view_is(p[0], 2, 0, dtype) && view_is(p[1], 2, 0, dtype) && view_is(p[2], 2, 1, dtype), "gemm views must be rank-2 In,In,Out");
    require(p[0].dimensions[1] == p[1].dimensions[0] && p[0].dimensions[0] == p[2].dimensions[0] &&
                p[1].dimensions[1] == p[2].dimensions[1], "gemm dimensions must be (M,K),(K,N),(M,N)");
    bool found = false;
    for (const Operation &op : operations)
      if (op.name == "contract") {
        found = op.line.find("reduce = [[1 : i64, 0 : i64]]") != std::string::npos && op.line.find("batch = []") != std::string::npos &&
                op.line.find("-> tensor<?x?xf32") != std::string::npos;
      }
    require(found, "contraction must pair a's axis 1 with b's axis 0 and accumulate in f32");
    plan.family = "gemm";
    plan.entry = "b200_gemm";
    plan.tail = {{"dtype", dtype_code(dtype)}, {"relu", c.of("binary<maximum>")}};
    plan.workspace = true;
    plan.alignment = 16;
    return plan;
  }
  if (c.of("for") == 1) {
    // ---- CSR SpMM / SpMV: parallel rows, ordered loop over the row's non-zeros ----
    require(c.of("parallel") == 1 && c.of("view_load") == 5 && c.of("view_store") == 1 &&
                c.of("assume_in_bounds") == 3 && c.of("binary<multiply>") == 1 && c.of("binary<add>") == 2 &&
                c.of("binary") == 3 && c.of("unary") == 0 && c.of("reduce") == 0 && c.of("cast") <= 1,
            "loop program is not the CSR row accumulation");
    require(p.size() == 5 && view_is(p[0], 1, 0, "i32") && view_is(p[1], 1, 0, "i32") && view_is(p[2], 1, 0, "f32"),
            "CSR kernels take row_offsets i32, column_indices i32, values f32 first");
    if (view_is(p[3], 1, 0, "f32") && view_is(p[4], 1, 1, "f32")) {
      plan.family = "csr_spmv";
      plan.entry = "b200_csr_spmv";
    } else {
      require(view_is(p[3], 2, 0, "f32") && view_is(p[4], 2, 1, "f32") && c.of("cast") == 0,
              "the dense operand and the output must both be f32 vectors or both f32 matrices");
      plan.family = "csr_spmm";
      plan.entry = "b200_csr_spmm";
      plan.workspace = true;   // per-call state: timeout report and the "rows ascend" word
    }
    plan.contiguous = {0, 1, 2};
    return plan;
  }
  if (!heavy && c.of("parallel") == 2 && c.of("reduce") == 1 && c.of("view_load") == 2 && c.of("view_store") == 1) {
    // ---- attention backward delta: row sums of f32(output) * f32(grad_output) -----------------
    require(c.of("cast") == 2 && c.of("unary") == 0 && c.of("binary") == 2 && c.of("binary<multiply>") == 1 &&
                c.of("binary<add>") == 1,
            "two-level row reduction is not sum(output * grad_output)");
    require(p.size() == 3, "attention_backward_delta takes output, grad_output, delta");
    const std::string dtype = p[0].dtype;
    require((dtype == "f16" || dtype == "bf16") && view_is(p[0], 4, 0, dtype) && view_is(p[1], 4, 0, dtype) &&
                view_is(p[2], 3, 1, "f32"),
            "attention_backward_delta views must be two rank-4 16-bit inputs and a rank-3 f32 output");
    plan.family = "attention_backward_delta";
    plan.entry = "b200_attention_backward_delta";
    plan.tail = {{"dtype", dtype_code(dtype)}};
    return plan;
  }
  if (!heavy && c.of("scatter_reduce") == 2) {
    // ---- LayerNorm backward, per row: dx and the bf16 partial sums of dw, db ------
    require(c.of("parallel") == 1 && c.of("reduce") == 2 && c.of("view_load") == 5 && c.of("view_store") == 1 &&
                c.of("unary") == 0 && c.of("cast") == 6 && c.of("binary") == 16 && c.of("binary<multiply>") == 8 &&
                c.of("binary<subtract>") == 3 && c.of("binary<add>") == 4 && c.of("binary<remainder>") == 1,
            "scatter-reduction program is not the LayerNorm backward row kernel");
    require(p.size() == 9 && view_is(p[0], 2, 0, "bf16") && view_is(p[1], 2, 0, "bf16") && view_is(p[2], 1, 0, "bf16") &&
                view_is(p[3], 1, 0, "f32") && view_is(p[4], 1, 0, "f32") && view_is(p[5], 2, 1, "bf16") &&
                view_is(p[6], 2, 2, "bf16") && view_is(p[7], 2, 2, "bf16") && p[8].kind == Parameter::kScalar &&
                p[8].dtype == "f32",
            "layer_norm_backward_rows takes x, dy, weight, mean, rstd, dx, dw_partial, db_partial, inverse_features");
    plan.family = "layer_norm_backward_rows";
    plan.entry = "b200_layer_norm_backward_rows";
    return plan;
  }
  if (!heavy && c.of("parallel") == 0 && c.of("reduce") == 2 && c.of("view_load") == 2 && c.of("view_store") == 2) {
    // ---- LayerNorm backward, reduction of the partial sums over the group axis ------
    require(c.of("cast") == 2 && c.of("unary") == 0 && c.of("binary") == 2 && c.of("binary<add>") == 2,
            "two-output reduction is not the LayerNorm backward partial-sum reduction");
    require(p.size() == 4 && view_is(p[0], 2, 0, "bf16") && view_is(p[1], 2, 0, "bf16") && view_is(p[2], 1, 1, "f32") &&
                view_is(p[3], 1, 1, "f32"),
            "layer_norm_backward_reduce takes dw_partial, db_partial (bf16) and dw, db (f32)");
    plan.family = "layer_norm_backward_reduce";
    plan.entry = "b200_layer_norm_backward_reduce";
    return plan;
  }
  if (!heavy && c.of("parallel") == 1 && c.of("reduce") == 1 && c.of("unary") == 0 && c.of("view_load") == 2 &&
      c.of("view_store") == 1) {
    // ---- softmax backward: p * (dy - sum(p * dy)) --------------------------------
    require(c.of("binary<multiply>") == 2 && c.of("binary<subtract>") == 1 && c.of("binary<add>") == 1 &&
                c.of("binary") == 4 && c.of("cast") == 0,
            "single-reduction program is not p * (dy - sum(p * dy))");
    require(p.size() == 3 && view_is(p[0], 2, 0, "f32") && view_is(p[1], 2, 0, "f32") && view_is(p[2], 2, 1, "f32"),
            "softmax_backward takes probabilities, upstream, gradient as f32 matrices");
    plan.family = "softmax_backward";
    plan.entry = "b200_softmax_backward";
    plan.tail = {{"dtype", 0}};
    return plan;
  }
  require(!heavy && c.of("parallel") == 1 && c.of("reduce") == 2 && c.of("view_store") == 1, "unrecognised structure");
  if (c.of("unary<exp>") == 1) {
    // ---- row softmax ----------------------------------------------------------
    require(c.of("view_load") == 1 && c.of("unary") == 1 && c.of("binary<maximum_num>") == 1 && c.of("binary<add>") == 1 &&
                c.of("binary<subtract>") == 1 && c.of("binary<true_divide>") == 1,
            "reduction program is not exp(x - max) / sum");
    require(p.size() == 2, "softmax takes x, y");
    const std::string dtype = p[0].dtype;
    require(dtype_code(dtype) >= 0 && view_is(p[0], 2, 0, dtype) && view_is(p[1], 2, 1, dtype), "softmax views must be rank-2 In,Out");
    if (dtype == "f32") require(c.of("binary<multiply>") == 1 && c.of("cast") == 0 && c.of("binary") == 5, "f32 softmax multiplies by the reciprocal");
    else require(c.of("binary<multiply>") == 0 && c.of("cast") == 2 && c.of("binary") == 4, "16-bit softmax divides, then narrows");
    plan.family = "softmax";
    plan.entry = "b200_softmax";
    plan.tail = {{"dtype", dtype_code(dtype)}};
    return plan;
  }
  if (c.of("unary<rsqrt>") == 1) {
    // ---- LayerNorm -----------------------------------------------------------
    require(c.of("view_load") == 3 && c.of("unary") == 1 && c.of("binary<add>") == 4, "normalisation program is not LayerNorm");
    require(p.size() == 6 && p[4].kind == Parameter::kScalar && p[4].dtype == "f32" && p[5].kind == Parameter::kScalar && p[5].dtype == "f32",
            "layer_norm takes x, weight, bias, y, inverse_features, epsilon");
    const std::string dtype = p[0].dtype;
    require(dtype_code(dtype) >= 0 && view_is(p[0], 2, 0, dtype) && view_is(p[1], 1, 0, dtype) && view_is(p[2], 1, 0, dtype) && view_is(p[3], 2, 1, dtype),
            "layer_norm views must be x(M,N), weight(N), bias(N), y(M,N)");
    bool centered;
    if (c.of("binary<multiply>") == 5 && c.of("binary<subtract>") == 1 && c.of("binary") == 10) centered = true;
    else if (c.of("binary<multiply>") == 6 && c.of("binary<subtract>") == 2 && c.of("binary") == 12) centered = false;
    else require(false, "variance is neither the centred two-pass nor the E[x^2]-mean^2 form");
    require(c.of("cast") == (dtype == "f32" ? 0 : 4), "statistics must be computed in f32");
    plan.family = "layer_norm";
    plan.entry = "b200_layer_norm";
    plan.tail = {{"dtype", dtype_code(dtype)}, {"centered", centered}};
    return plan;
  }
  require(false, "unrecognised structure");
  return plan;
}

// ---------------------------------------------------------------- JSON output
std::string quote(const std::string &text) {
  std::string out = "\"";
  for (char c : text) {
    if (c == '"' || c == '\\') { out += '\\'; out += c; }
    else if (c == '\n') out += "\\n";
    else out += c;
  }
  return out + "\"";
}

struct CompileOptions {
  std::string numerics = "source";
  std::map<std::string, bool> optimizations;
  bool remarks = false;
};

std::string metadata_json(const std::string &function, const std::vector<Parameter> &all, const Plan &plan,
                          const std::string &capabilities, const CompileOptions &options) {
  std::vector<Parameter> p;
  for (const Parameter &parameter : all)
    if (parameter.kind != Parameter::kConstexpr) p.push_back(parameter);
  std::ostringstream o;
  o << "{\n  \"provider\": \"b200\",\n  \"entry_name\": " << quote(function) << ",\n";
  o << "  \"target\": {\"family\": \"b200_native\", \"capabilities\": " << capabilities << "},\n";
  o << "  \"compile_options\": {\"numerics\": " << quote(options.numerics) << ", \"optimizations\": {";
  bool first = true;
  for (const auto &entry : options.optimizations) {
    o << (first ? "" : ", ") << quote(entry.first) << ": " << (entry.second ? "true" : "false");
    first = false;
  }
  o << "}, \"optimization_remarks\": " << (options.remarks ? "true" : "false") << "},\n";
  o << "  \"interface\": {\"parameters\": [\n";
  for (size_t i = 0; i < p.size(); ++i) {
    const Parameter &q = p[i];
    o << "    {";
    if (q.kind == Parameter::kScalar) {
      o << "\"kind\": \"scalar\", \"name\": " << quote(q.name) << ", \"dtype\": " << quote(q.dtype);
    } else {
      o << "\"kind\": \"view\", \"name\": " << quote(q.name) << ", \"dtype\": " << quote(q.dtype) << ", \"shape\": [";
      for (size_t a = 0; a < q.shape.size(); ++a) o << (a ? ", " : "") << q.shape[a];
      o << "], \"dimensions\": [";
      for (size_t a = 0; a < q.dimensions.size(); ++a) o << (a ? ", " : "") << q.dimensions[a];
      o << "], \"strides\": [";
      for (size_t a = 0; a < q.strides.size(); ++a) {
        o << (a ? ", " : "");
        if (q.strides[a].kind == Stride::kFree) o << "null";
        else if (q.strides[a].kind == Stride::kFixed) o << q.strides[a].value;
        else o << "{\"kind\": \"stride_symbol\", \"symbol\": " << quote(q.strides[a].symbol) << "}";
      }
      o << "], \"access\": " << q.access << ", \"alias\": " << quote(q.alias) << ", \"noalias\": " << (q.noalias ? "true" : "false");
    }
    o << "}" << (i + 1 < p.size() ? "," : "") << "\n";
  }
  o << "  ]},\n  \"native\": {\n    \"slots\": [\n";
  std::vector<std::string> slots;
  auto view_slots = [&](size_t position, const std::string &element, size_t rank) {
    std::ostringstream s;
    s << "{\"role\": \"pointer\", \"parameter\": " << position << ", \"carrier\": \"ptr\", \"element\": " << quote(element) << "}";
    slots.push_back(s.str());
    for (const char *role : {"extent", "stride"})
      for (size_t axis = 0; axis < rank; ++axis) {
        std::ostringstream t;
        t << "{\"role\": \"" << role << "\", \"parameter\": " << position << ", \"axis\": " << axis << ", \"carrier\": \"i64\"}";
        slots.push_back(t.str());
      }
  };
  for (size_t i = 0; i < p.size(); ++i) {
    if (p[i].kind == Parameter::kView) view_slots(i, p[i].dtype, p[i].shape.size());
    else {
      std::ostringstream s;
      s << "{\"role\": \"scalar\", \"parameter\": " << i << ", \"carrier\": " << quote(p[i].dtype) << "}";
      slots.push_back(s.str());
    }
  }
  if (plan.workspace) view_slots(p.size(), "i32", 1);
  for (size_t i = 0; i < slots.size(); ++i) o << "      " << slots[i] << (i + 1 < slots.size() ? "," : "") << "\n";
  o << "    ],\n    \"workspaces\": [";
  if (plan.workspace) o << "{\"position\": " << p.size() << ", \"dtype\": \"i32\", \"shape\": [64]}";
  o << "],\n    \"requirements\": {\"views\": [";
  first = true;
  std::vector<size_t> writable, readable;
  for (size_t i = 0; i < p.size(); ++i) {
    if (p[i].kind != Parameter::kView) continue;
    bool contiguous = false;
    for (int position : plan.contiguous) contiguous |= (size_t)position == i;
    o << (first ? "" : ", ") << "{\"parameter\": " << i << ", \"layout\": " << (contiguous ? "\"contiguous\"" : "\"strided\"")
      << ", \"alignment\": " << (plan.alignment ? plan.alignment : dtype_bytes(p[i].dtype)) << "}";
    first = false;
    (p[i].access == 0 ? readable : writable).push_back(i);
  }
  o << "], \"disjoint\": [";
  first = true;
  for (size_t w : writable)
    for (size_t r : readable) {
      o << (first ? "" : ", ") << "{\"left\": " << (r < w ? r : w) << ", \"right\": " << (r < w ? w : r) << "}";
      first = false;
    }
  o << "]}\n  },\n";
  o << "  \"b200\": {\"abi_version\": 1, \"family\": " << quote(plan.family) << ", \"entry\": " << quote(plan.entry) << ", \"tail\": [";
  for (size_t i = 0; i < plan.tail.size(); ++i)
    o << (i ? ", " : "") << "{\"name\": " << quote(plan.tail[i].name) << ", \"carrier\": \"i32\", \"value\": " << plan.tail[i].value << "}";
  o << "], \"stream\": true}\n}\n";
  return o.str();
}

std::string source_text(const std::string &function, const Plan &plan) {
  std::ostringstream o;
  o << "// intent_b200 launch descriptor (not generated device code: the kernel is\n"
       "// hand-written sm_100a CUDA inside libintent_b200.so)\n";
  o << "kernel " << function << "\nfamily " << plan.family << "\nentry " << plan.entry << "\n";
  for (const TailConstant &constant : plan.tail) o << "constant " << constant.name << " = " << constant.value << "\n";
  o << "workspace " << (plan.workspace ? "int32[64]" : "none") << "\nstream current\n";
  return o.str();
}

bool write_file(const std::string &path, const std::string &text) {
  std::ofstream out(path, std::ios::binary);
  out << text;
  return static_cast<bool>(out.flush());
}

bool option_value(const std::string &argument, const char *name, std::string *value) {
  const std::string prefix = std::string("--") + name + "=";
  if (argument.rfind(prefix, 0) != 0) return false;
  *value = argument.substr(prefix.size());
  return true;
}

bool parse_bool(const std::string &text, bool *value) {
  if (text == "true" || text == "1") { *value = true; return true; }
  if (text == "false" || text == "0") { *value = false; return true; }
  return false;
}

}  // namespace

int main(int argc, char **argv) {
  std::string target, target_options, input_stage = "kir", ir_output, source_output, metadata_output, input = "-", value;
  CompileOptions options;
  bool info = false, stop_kir = false, stop_shared = false, any_other = false, structure_only = false;
  for (int i = 1; i < argc; ++i) {
    const std::string argument = argv[i];
    bool flag = false;
    if (argument == "--compiler-info") { info = true; continue; }
    any_other = true;
    if (argument == "--structure") structure_only = true;     // print "<family> <hash>" of the program on stdin
    else if (argument == "--stop-after-kir") stop_kir = true;
    else if (argument == "--stop-after-shared") stop_shared = true;
    else if (option_value(argument, "target", &target)) {}
    else if (option_value(argument, "target-options", &target_options)) {}
    else if (option_value(argument, "input-stage", &input_stage)) {}
    else if (option_value(argument, "ir-output", &ir_output)) {}
    else if (option_value(argument, "source-output", &source_output)) {}
    else if (option_value(argument, "metadata-output", &metadata_output)) {}
    else if (option_value(argument, "tuning-config", &value)) {
      std::cerr << "b200 declares no tuning profile families; --tuning-config is not accepted\n";
      return kInvocation;
    } else if (option_value(argument, "numerics", &options.numerics)) {
      if (options.numerics != "source" && options.numerics != "relaxed_normalization") {
        std::cerr << "--numerics must be source or relaxed_normalization\n";
        return kInvocation;
      }
    } else if (option_value(argument, "optimization-remarks", &value)) {
      if (!parse_bool(value, &options.remarks)) { std::cerr << "--optimization-remarks takes true|false\n"; return kInvocation; }
    } else if (argument == "--optimization-remarks") options.remarks = true;
    else if (option_value(argument, "optimization", &value)) {
      size_t eq = value.find('=');
      if (eq == std::string::npos || eq == 0 || !parse_bool(value.substr(eq + 1), &flag) ||
          !options.optimizations.emplace(value.substr(0, eq), flag).second) {
        std::cerr << "--optimization requires a unique NAME=true|false: " << value << "\n";
        return kInvocation;
      }
    } else if (argument == "-" || argument[0] != '-') input = argument;
    else { std::cerr << "unknown option: " << argument << "\n"; return kInvocation; }
  }
  if (info) {
    if (any_other) { std::cerr << "--compiler-info does not compile a program\n"; return kInvocation; }
    std::cout << "{\"providers\": {\"b200\": {\"family\": \"b200_native\", \"available\": true, \"profiles\": []}}, "
                 "\"input_stages\": [\"kir\", \"shared\"], \"stages\": [\"kir\", \"shared\", \"provider\"], "
                 "\"outputs\": {\"kir\": [\"ir\"], \"shared\": [\"ir\"], \"provider\": [\"ir\", \"source\", \"metadata\"]}, "
                 "\"compile_options\": {\"numerics\": [\"source\", \"relaxed_normalization\"], \"optimizations\": {}, "
                 "\"optimization_remarks\": false}, \"failure_stages\": " << kFailureStages << "}\n";
    return 0;
  }
  if (structure_only) { target = "b200"; ir_output = source_output = "-"; }   // nothing is written in this mode
  if (stop_kir && stop_shared) { std::cerr << "--stop-after-kir and --stop-after-shared are mutually exclusive\n"; return kInvocation; }
  if (input_stage != "kir" && input_stage != "shared") { std::cerr << "--input-stage must be kir or shared\n"; return kInvocation; }
  if (!stop_kir && target.empty()) { std::cerr << "--target is required unless --stop-after-kir is selected\n"; return kInvocation; }
  if (stop_kir && (!target.empty() || !target_options.empty())) {
    std::cerr << "KIR output does not select a physical target\n";
    return kInvocation;
  }
  if (!target.empty() && target != "b200") { std::cerr << "unknown source provider: " << target << "\n"; return kInvocation; }
  const bool provider_stage = !stop_kir && !stop_shared;
  if (!provider_stage && (!source_output.empty() || !metadata_output.empty())) { std::cerr << "selected stage only emits IR\n"; return kInvocation; }
  if (ir_output.empty() || (provider_stage && source_output.empty())) {
    std::cerr << "--ir-output is required; provider compilation also requires --source-output\n";
    return kOutput;
  }
  if (!options.optimizations.empty()) {
    std::cerr << "b200 registers no optional transformations; --optimization is not accepted\n";
    return kInvocation;
  }

  std::string ir;
  if (input == "-") {
    std::ostringstream buffer;
    buffer << std::cin.rdbuf();
    ir = buffer.str();
  } else {
    std::ifstream file(input, std::ios::binary);
    if (!file) { std::cerr << "cannot read " << input << "\n"; return kInvocation; }
    std::ostringstream buffer;
    buffer << file.rdbuf();
    ir = buffer.str();
  }
  try {
    if (trim(ir).empty()) fail(kKernelIR, "empty kernel IR");
    std::string function;
    std::vector<Parameter> parameters = parse_signature(ir, &function);
    std::vector<Operation> operations = parse_operations(ir);
    if (structure_only) {
      const Plan plan = classify(parameters, operations);
      std::cout << plan.family << " " << std::hex << structure_hash(canonical_structure(ir, operations)) << "\n";
      return 0;
    }
    if (!provider_stage) {
      if (!write_file(ir_output, ir)) fail(kOutput, "cannot write " + ir_output);
      return 0;
    }
    const std::string capabilities = trim(target_options);
    if (capabilities.size() < 2 || capabilities.front() != '{' || capabilities.back() != '}')
      fail(kInvocation, "--target-options must be the JSON object of NVIDIA capability facts");
    if (capabilities.find("\"compute_capability_major\": 10") == std::string::npos &&
        capabilities.find("\"compute_capability_major\":10") == std::string::npos)
      fail(kProviderPipeline, "b200 holds sm_100a kernels only; the target reports another compute capability");
    const Plan plan = classify(parameters, operations);
    require_known_structure(plan.family, structure_hash(canonical_structure(ir, operations)));
    if (options.remarks) std::cerr << "remark: " << function << " -> " << plan.family << " (" << plan.entry << ")\n";
    if (!write_file(ir_output, ir)) fail(kOutput, "cannot write " + ir_output);
    if (!write_file(source_output, source_text(function, plan))) fail(kOutput, "cannot write " + source_output);
    if (!metadata_output.empty() &&
        !write_file(metadata_output, metadata_json(function, parameters, plan, capabilities, options)))
      fail(kOutput, "cannot write " + metadata_output);
  } catch (const Failure &failure) {
    std::cerr << failure.message << "\n";
    return failure.code;
  }
  return 0;
}

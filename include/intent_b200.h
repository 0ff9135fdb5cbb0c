/*
 * intent_b200 — C ABI of the B200 (sm_100a) operator provider for IntentDSL.
 *
 * Every operator entry follows the reference's native slot convention
 * (lib/Serialization/NativeABI.cpp:80-118; ctypes carriers in
 * python/intent/runtime/native.py:15-17): for each public parameter, in
 * declaration order,
 *     view   ->  void* aP, int64 aP_d0.., int64 aP_s0..   (extents, then element strides)
 *     scalar ->  its carrier (f32 -> float)
 * followed by invocation workspaces (same view layout), and then a
 * provider-private tail the reference's CPU entries do not have:
 *     int32 constants taken from the kernel's constexprs / element type, and
 *     void* stream  — the cudaStream_t to enqueue on (the caller passes the
 *                     framework's current stream; nothing here synchronises,
 *                     doc/getting-started/usage.en.md:53-55).
 * The reference's CPU entries return void (python/intent/runtime/mojo/program.py:302-304);
 * these return an int status instead of aborting, so a failing call never
 * takes the process down and never falls back to another provider
 * (doc/getting-started/usage.en.md:21).
 *
 * All pointers are device pointers on the current CUDA device.  The caller
 * owns every buffer and keeps it alive until the stream has run the work
 * (doc/getting-started/usage.en.md:50).
 */
#ifndef INTENT_B200_H
#define INTENT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_ABI_VERSION 1

/* status codes */
#define B200_OK 0
#define B200_ERR_INVALID_ARGUMENT 1   /* null pointer, negative extent, inconsistent shapes */
#define B200_ERR_UNSUPPORTED_LAYOUT 2 /* strides / alignment / sizes this entry does not accept */
#define B200_ERR_CUDA 3               /* a CUDA call failed; see b200_last_error */
#define B200_ERR_DEVICE 4             /* not an sm_100 device */
#define B200_ERR_DEVICE_TIMEOUT 5     /* a bounded device-side wait gave up (workspace status word) */

/* element type codes of the private tail */
#define B200_F32 0
#define B200_F16 1
#define B200_BF16 2

/* Number of int32 words every workspace view must hold (zero-initialised by
   the caller once; word 0 is a sticky device-side status, see b200_workspace_status). */
#define B200_WORKSPACE_WORDS 64

int b200_abi_version(void);
const char *b200_status_string(int status);
/* Copies the message of the most recent failing call on this thread. */
int b200_last_error(char *buffer, int64_t capacity);
/* B200_OK when `device` is an sm_100 part this library has code for. */
int b200_device_check(int device);

/*
 * The eight integer facts the reference reads through the CUDA driver in
 * resolve_cuda_device (python/intent/targets/nvidia/device.py:6-59), in its
 * order: multiprocessors, shared memory per multiprocessor, opt-in shared
 * memory per block, registers per multiprocessor, threads per block, compute
 * capability major, minor, single-to-double throughput ratio.
 */
int b200_device_capabilities(int device, int64_t *facts);

/*
 * Row softmax.  Replaces the kernel the reference generates for
 * stable_softmax / stable_softmax_f16 / chunked_softmax_bf16
 * (python/intent/examples/kernels/normalization/softmax.py:23-66), i.e. the
 * call made at python/intent/runtime/mojo/program.py:198-207 (CPU provider) or
 * python/intent/runtime/triton/program.py:370-389 (GPU provider).
 * f32: y = exp(x - max) * (1 / sum); f16/bf16: y = cast(exp(x - max) / sum).
 * Requires unit inner strides (x_s1 == y_s1 == 1); row pitches are free.
 */
int b200_softmax(const void *x, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                 void *y, int64_t y_d0, int64_t y_d1, int64_t y_s0, int64_t y_s1,
                 int32_t dtype, void *stream);

/*
 * Softmax backward: gradient = p * (dy - sum(p * dy)) per row, f32.  Replaces
 * softmax_backward (python/intent/examples/kernels/backward/softmax.py:9-24), the
 * kernel the reference pairs with stable_softmax for autograd
 * (examples/softmax_forward_backward.py:11-29).  Unit inner strides; any row
 * pitch or alignment (the reference instance has 4097 columns).
 */
int b200_softmax_backward(const void *probabilities, int64_t p_d0, int64_t p_d1, int64_t p_s0, int64_t p_s1,
                          const void *upstream, int64_t u_d0, int64_t u_d1, int64_t u_s0, int64_t u_s1,
                          void *gradient, int64_t g_d0, int64_t g_d1, int64_t g_s0, int64_t g_s1,
                          int32_t dtype, void *stream);

/*
 * LayerNorm backward, row kernel (bf16 operands, f32 arithmetic).  Replaces
 * layer_norm_backward_rows (python/intent/examples/kernels/backward/layer_norm.py:12-66):
 * dx = (w*dy - mean(w*dy) - xhat * mean(w*dy*xhat)) * rstd with xhat = (x - mean) * rstd,
 * and the scatter-reductions dw_partial[row % G] += bf16(dy * xhat),
 * db_partial[row % G] += dy, G = dw_d0.  The reference promises no order for
 * colliding updates (doc/dsl/types-numerics-and-effects.en.md:242); this entry
 * fixes one: a group's rows are dealt round-robin to 8 lanes, each lane folds its
 * rows in ascending order, the lane sums are combined in a fixed binary tree and
 * the total is added to the previous contents, every add rounded to bf16,
 * so results do not vary from run to run.  dw_partial / db_partial are InOut:
 * their contents are accumulated into.  Unit inner strides; N a multiple of 8
 * and at most 8192; x, dy, dx, the partial rows and weight 16-byte aligned
 * (else B200_ERR_UNSUPPORTED_LAYOUT).
 */
int b200_layer_norm_backward_rows(const void *x, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                                  const void *dy, int64_t dy_d0, int64_t dy_d1, int64_t dy_s0, int64_t dy_s1,
                                  const void *weight, int64_t w_d0, int64_t w_s0,
                                  const void *mean, int64_t mean_d0, int64_t mean_s0,
                                  const void *rstd, int64_t rstd_d0, int64_t rstd_s0,
                                  void *dx, int64_t dx_d0, int64_t dx_d1, int64_t dx_s0, int64_t dx_s1,
                                  void *dw_partial, int64_t dw_d0, int64_t dw_d1, int64_t dw_s0, int64_t dw_s1,
                                  void *db_partial, int64_t db_d0, int64_t db_d1, int64_t db_s0, int64_t db_s1,
                                  float inverse_features, void *stream);

/*
 * LayerNorm backward, reduction of the partial sums: dw[n] = sum_g f32(dw_partial[g, n]),
 * likewise db, groups ascending.  Replaces layer_norm_backward_reduce
 * (python/intent/examples/kernels/backward/layer_norm.py:69-90).  Unit inner strides.
 */
int b200_layer_norm_backward_reduce(const void *dw_partial, int64_t dw_d0, int64_t dw_d1, int64_t dw_s0, int64_t dw_s1,
                                    const void *db_partial, int64_t db_d0, int64_t db_d1, int64_t db_s0, int64_t db_s1,
                                    void *dw, int64_t o_d0, int64_t o_s0, void *db, int64_t b_d0, int64_t b_s0,
                                    void *stream);

/*
 * Attention backward, three kernels (f16 / bf16 operands, f32 arithmetic, natural-log LSE; views are
 * (batch, head, sequence, D) with unit innermost stride, D in {64, 128}).  They replace
 * attention_backward_delta, attention_backward_dkdv and attention_backward_dq
 * (python/intent/examples/kernels/backward/attention.py:16-33, 91-137, 171-211), which
 * python/intent/examples/programs/attention_backward.py:19-41 runs in this order.
 *   delta[b,h,q] = sum_d f32(output) * f32(grad_output)
 *   P = exp2(S * scale*log2e - lse*log2e), excluded pairs (key > query when causal) are 0
 *   dS = P * (dO . V^T - delta);  grad_v = f16(P)^T . dO;  grad_k = scale * f16(dS)^T . Q;
 *   grad_q = scale * f16(dS) . K
 * q, k, v, grad_output go through TMA: 16-byte aligned bases, outer strides multiples of 8
 * elements.  The gradient entries take the same B200_WORKSPACE_WORDS workspace view as
 * b200_flash_attention, then the int32 tail dtype, head_group, causal.
 */
int b200_attention_backward_delta(
        const void *output, int64_t output_d0, int64_t output_d1, int64_t output_d2, int64_t output_d3,
        int64_t output_s0, int64_t output_s1, int64_t output_s2, int64_t output_s3,
        const void *grad_output, int64_t grad_output_d0, int64_t grad_output_d1, int64_t grad_output_d2, int64_t grad_output_d3,
        int64_t grad_output_s0, int64_t grad_output_s1, int64_t grad_output_s2, int64_t grad_output_s3,
        void *delta, int64_t delta_d0, int64_t delta_d1, int64_t delta_d2, int64_t delta_s0, int64_t delta_s1, int64_t delta_s2,
        int32_t dtype, void *stream);
int b200_attention_backward_dkdv(
        const void *q, int64_t q_d0, int64_t q_d1, int64_t q_d2, int64_t q_d3,
        int64_t q_s0, int64_t q_s1, int64_t q_s2, int64_t q_s3,
        const void *k, int64_t k_d0, int64_t k_d1, int64_t k_d2, int64_t k_d3,
        int64_t k_s0, int64_t k_s1, int64_t k_s2, int64_t k_s3,
        const void *v, int64_t v_d0, int64_t v_d1, int64_t v_d2, int64_t v_d3,
        int64_t v_s0, int64_t v_s1, int64_t v_s2, int64_t v_s3,
        const void *grad_output, int64_t grad_output_d0, int64_t grad_output_d1, int64_t grad_output_d2, int64_t grad_output_d3,
        int64_t grad_output_s0, int64_t grad_output_s1, int64_t grad_output_s2, int64_t grad_output_s3,
        const void *lse, int64_t lse_d0, int64_t lse_d1, int64_t lse_d2, int64_t lse_s0, int64_t lse_s1, int64_t lse_s2,
        const void *delta, int64_t delta_d0, int64_t delta_d1, int64_t delta_d2, int64_t delta_s0, int64_t delta_s1, int64_t delta_s2,
        void *grad_k, int64_t grad_k_d0, int64_t grad_k_d1, int64_t grad_k_d2, int64_t grad_k_d3,
        int64_t grad_k_s0, int64_t grad_k_s1, int64_t grad_k_s2, int64_t grad_k_s3,
        void *grad_v, int64_t grad_v_d0, int64_t grad_v_d1, int64_t grad_v_d2, int64_t grad_v_d3,
        int64_t grad_v_s0, int64_t grad_v_s1, int64_t grad_v_s2, int64_t grad_v_s3,
        float scale, void *workspace, int64_t ws_d0, int64_t ws_s0, int32_t dtype, int32_t head_group, int32_t causal,
        void *stream);
int b200_attention_backward_dq(
        const void *q, int64_t q_d0, int64_t q_d1, int64_t q_d2, int64_t q_d3,
        int64_t q_s0, int64_t q_s1, int64_t q_s2, int64_t q_s3,
        const void *k, int64_t k_d0, int64_t k_d1, int64_t k_d2, int64_t k_d3,
        int64_t k_s0, int64_t k_s1, int64_t k_s2, int64_t k_s3,
        const void *v, int64_t v_d0, int64_t v_d1, int64_t v_d2, int64_t v_d3,
        int64_t v_s0, int64_t v_s1, int64_t v_s2, int64_t v_s3,
        const void *grad_output, int64_t grad_output_d0, int64_t grad_output_d1, int64_t grad_output_d2, int64_t grad_output_d3,
        int64_t grad_output_s0, int64_t grad_output_s1, int64_t grad_output_s2, int64_t grad_output_s3,
        const void *lse, int64_t lse_d0, int64_t lse_d1, int64_t lse_d2, int64_t lse_s0, int64_t lse_s1, int64_t lse_s2,
        const void *delta, int64_t delta_d0, int64_t delta_d1, int64_t delta_d2, int64_t delta_s0, int64_t delta_s1, int64_t delta_s2,
        void *grad_q, int64_t grad_q_d0, int64_t grad_q_d1, int64_t grad_q_d2, int64_t grad_q_d3,
        int64_t grad_q_s0, int64_t grad_q_s1, int64_t grad_q_s2, int64_t grad_q_s3,
        float scale, void *workspace, int64_t ws_d0, int64_t ws_s0, int32_t dtype, int32_t head_group, int32_t causal,
        void *stream);

/*
 * LayerNorm forward.  Replaces layer_norm_f16 / layer_norm_bf16 (centred
 * two-pass variance) and weighted_layer_norm (f32, E[x^2] - mean^2)
 * (python/intent/examples/kernels/normalization/layer_norm.py:9-85).
 * Statistics in f32; `centered` selects the variance form (1 for the 16-bit
 * kernels, 0 for weighted_layer_norm).  Requires unit inner strides.
 */
int b200_layer_norm(const void *x, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                    const void *weight, int64_t w_d0, int64_t w_s0,
                    const void *bias, int64_t b_d0, int64_t b_s0,
                    void *y, int64_t y_d0, int64_t y_d1, int64_t y_s0, int64_t y_s1,
                    float inverse_features, float epsilon,
                    int32_t dtype, int32_t centered, void *stream);

/*
 * Dense GEMM C = cast(A . B), f16 or bf16 operands, f32 accumulation on the
 * tcgen05 tensor cores.  Replaces gemm (ACTIVATION NONE / RELU) and bf16_gemm
 * (python/intent/examples/kernels/contraction/gemm.py:54-92).
 * a is (M,K), b is (K,N), c is (M,N) in element strides.  Accepted layouts:
 * a K-major (a_s1 == 1); b K-major (b_s0 == 1, "column-major B") or N-major
 * (b_s1 == 1, plain row-major (K,N)); c row-major (c_s1 == 1); leading strides
 * multiples of 8 elements and 16-byte aligned bases (TMA requirements).
 * workspace: B200_WORKSPACE_WORDS int32 words, zeroed once by the caller.
 */
int b200_gemm(const void *a, int64_t a_d0, int64_t a_d1, int64_t a_s0, int64_t a_s1,
              const void *b, int64_t b_d0, int64_t b_d1, int64_t b_s0, int64_t b_s1,
              void *c, int64_t c_d0, int64_t c_d1, int64_t c_s0, int64_t c_s1,
              void *workspace, int64_t ws_d0, int64_t ws_s0,
              int32_t dtype, int32_t relu, void *stream);

/*
 * b200_gemm for callers that cannot allocate device memory.  It has no
 * counterpart in the reference, whose runtime always allocates invocation
 * workspaces itself (python/intent/runtime/native.py:207-209).
 *
 * Who needs it: code that runs where cudaMalloc is off limits — a host
 * function driven from inside another framework's stream-ordered region, a
 * real-time or safety-partitioned process whose memory budget is fixed at
 * start-up, a plugin that is handed device buffers but no allocator.  Such a
 * caller cannot provide b200_gemm's workspace view.  Here the status words the
 * kernel's bounded waits use live in a device array that is part of this
 * library: B200_WORKSPACE_WORDS int32 words (256 bytes), held by every GPU
 * that loads the library until the process exits.  The call itself makes no
 * cudaMalloc / cudaFree and no other allocating library call.  On the host it
 * remembers one thing per device for the life of the process: the array's
 * address (a table of 64 pointers inside the library), so a device that is
 * reset while the process keeps running is not supported.
 *
 * Arguments are b200_gemm's without the workspace view, plus wait_and_check:
 *   0  enqueue only, like b200_gemm; a device-side timeout goes unreported;
 *   1  also synchronise `stream` and return B200_ERR_DEVICE_TIMEOUT if a
 *      bounded wait gave up.
 * Limits: each of M, N, K at most B200_STATIC_SCRATCH_MAX_EXTENT; larger
 * problems are refused with B200_ERR_UNSUPPORTED_LAYOUT.  Layout rules are
 * b200_gemm's except for B, which must be K-major here (b_s0 == 1, the
 * "column-major (K,N)" layout); b200_gemm's second layout, N-major B, is
 * refused with B200_ERR_UNSUPPORTED_LAYOUT.
 * The first call on a device looks the array's address up (one
 * cudaGetSymbolAddress with that device current); make that call before any
 * stream capture begins.  All calls on one GPU share the array: every call
 * clears the status words on `stream` before its kernel, so calls that
 * overlap on the GPU (different streams) race on them and may lose or
 * misattribute a timeout report; results in C are unaffected.
 */
#define B200_STATIC_SCRATCH_MAX_EXTENT 2147483647LL
int b200_gemm_static_scratch(const void *a, int64_t a_d0, int64_t a_d1, int64_t a_s0, int64_t a_s1,
                             const void *b, int64_t b_d0, int64_t b_d1, int64_t b_s0, int64_t b_s1,
                             void *c, int64_t c_d0, int64_t c_d1, int64_t c_s0, int64_t c_s1,
                             int32_t dtype, int32_t relu, int32_t wait_and_check, void *stream);

/*
 * Flash-attention forward (online softmax over key tiles), bf16 or f16.
 * Replaces flash_attention_bf16_fwd, flash_attention_fwd and
 * flash_gqa_attention_fwd
 * (python/intent/examples/kernels/streaming/attention.py:428-553).
 * q (B,HQ,Q,D), k (B,HK,K,D), v (B,HK,K,DV), o (B,HQ,Q,DV); key head =
 * query head / head_group.  exp2 and the final reciprocal use
 * ex2.approx.ftz / div.approx.ftz as the reference's NVIDIA target does
 * (lib/Target/NVIDIA/IR/Target.cpp:62-86).  Requires unit innermost strides,
 * D == DV in {64, 128}, other strides positive multiples of 8 elements, 16-byte
 * aligned bases and scale > 0.  An empty key sequence yields zeros.
 * Numerics, where they differ from the reference's fold (which rescales at every
 * key chunk): the running maximum m a row's exponentials are taken against is only
 * replaced -- and O and the row sum rescaled by exp2(m_old - m_new) -- when a key
 * tile's maximum exceeds m by more than 8 (log2 units, i.e. 2^8).  Between rescales
 * p = exp2(s*scale*log2e - m) can reach 2^8, well inside f16/bf16/f32 range; P is
 * rounded to the operand type before P.V and the row sum is accumulated in f32 from
 * the unrounded p.  The result equals the reference's up to rounding; the parity
 * tests allow 1e-2 relative.
 */
int b200_flash_attention(const void *q, int64_t q_d0, int64_t q_d1, int64_t q_d2, int64_t q_d3,
                         int64_t q_s0, int64_t q_s1, int64_t q_s2, int64_t q_s3,
                         const void *k, int64_t k_d0, int64_t k_d1, int64_t k_d2, int64_t k_d3,
                         int64_t k_s0, int64_t k_s1, int64_t k_s2, int64_t k_s3,
                         const void *v, int64_t v_d0, int64_t v_d1, int64_t v_d2, int64_t v_d3,
                         int64_t v_s0, int64_t v_s1, int64_t v_s2, int64_t v_s3,
                         void *o, int64_t o_d0, int64_t o_d1, int64_t o_d2, int64_t o_d3,
                         int64_t o_s0, int64_t o_s1, int64_t o_s2, int64_t o_s3,
                         float scale,
                         void *workspace, int64_t ws_d0, int64_t ws_s0,
                         int32_t dtype, int32_t head_group, int32_t causal, void *stream);

/*
 * CSR SpMM  Y = A . X, i32 indices, f32 values, strict source-order
 * accumulation per row with an unfused multiply then add, so results are
 * bit-identical to a sequential left-to-right evaluation.  Replaces csr_spmm
 * (python/intent/examples/kernels/sparse/csr_spmm.py:12-33).
 * Indices are trusted as the kernel's assume_in_bounds states
 * (csr_spmm.py:26-29); b200_csr_validate checks them on the device.
 * Requires contiguous index/value arrays and unit inner strides of X and Y.
 * row_offsets may be a block of a longer offsets array (absolute offsets into
 * column_indices / values): row r covers non-zeros [row_offsets[r], row_offsets[r+1]).
 *
 * The workspace is invocation-owned like the reference's native workspaces
 * (python/intent/runtime/native.py:207-209): B200_WORKSPACE_WORDS int32 words,
 * zeroed once by the caller.  Word 2 carries, from the first launch of a call
 * to its later ones, whether every row ascends (a call on an X larger than L2
 * runs as several launches over column blocks, and falls back to one pass in
 * storage order when a row does not ascend); words 0-1 are not written (the
 * kernels have no bounded wait).  All state of a call lives in its workspace:
 * calls with distinct workspaces may overlap on different streams.
 */
int b200_csr_spmm(const void *row_offsets, int64_t ro_d0, int64_t ro_s0,
                  const void *column_indices, int64_t ci_d0, int64_t ci_s0,
                  const void *values, int64_t va_d0, int64_t va_s0,
                  const void *dense, int64_t x_d0, int64_t x_d1, int64_t x_s0, int64_t x_s1,
                  void *output, int64_t y_d0, int64_t y_d1, int64_t y_s0, int64_t y_s1,
                  void *workspace, int64_t ws_d0, int64_t ws_s0,
                  void *stream);

/*
 * CSR SpMV  y = A . x: csr_spmm with a single feature, same strict storage-order
 * accumulation (bit-identical to the sequential sum).  Replaces csr_spmv
 * (python/intent/examples/kernels/sparse/csr_spmv.py:11-29), the reference's
 * registered sparse program (python/intent/examples/programs/irregular.py:27-33).
 * Index/value arrays contiguous; x and y may have any stride.
 */
int b200_csr_spmv(const void *row_offsets, int64_t ro_d0, int64_t ro_s0,
                  const void *column_indices, int64_t ci_d0, int64_t ci_s0,
                  const void *values, int64_t va_d0, int64_t va_s0,
                  const void *vector, int64_t x_d0, int64_t x_s0,
                  void *output, int64_t y_d0, int64_t y_s0, void *stream);

/*
 * Device-side check of a CSR structure (monotone offsets within [0,nnz],
 * columns within [0,columns)).  No counterpart entry in the reference, whose
 * kernel assumes validity (csr_spmm.py:26-29).  Synchronises the stream.
 * Returns B200_OK or B200_ERR_INVALID_ARGUMENT with *where = first bad position.
 */
int b200_csr_validate(const void *row_offsets, int64_t rows, const void *column_indices,
                      int64_t nnz, int64_t columns, int64_t *where, void *stream);

/*
 * Measures what bounds the SpMM gathers on this device: `gathers` reads of
 * 512-byte rows at pseudo-random positions of `table` (table_rows x 128 f32).
 * variant 0..3: 4, 8, 16, 32 loads in flight per lane (64 warps per SM).
 * hints != 0 asks L2 to keep the gathered lines.  `sink` (>= 5 MiB) is never
 * written in practice; `workspace` as for b200_csr_spmm.  A measurement
 * aid with no counterpart in the reference: bench.py times it to report the
 * gather ceiling beside the SpMM figure.
 */
int b200_gather_probe(const void *table, int64_t table_rows, int64_t gathers, int32_t variant,
                      int32_t hints, void *sink, void *workspace, void *stream);

/*
 * Runs the bounded-wait path of the tensor-core kernels on purpose: one CTA waits, with a limit
 * of `limit_cycles` (1e3..2e8), for an mbarrier that nothing arrives on.  The wait gives up,
 * words 0-1 of the workspace become {1, site 9}, words 8-9 record {0 = "did not arrive", 1 =
 * "another warp saw the abort flag"}, and the kernel returns; b200_workspace_status then
 * reports B200_ERR_DEVICE_TIMEOUT.  Nothing faults or hangs.  For tests of the failure
 * reporting; no counterpart in the reference, which has no device-side waits of its own.
 */
int b200_selftest_bounded_wait(void *workspace, int64_t ws_d0, int64_t ws_s0, int64_t limit_cycles, void *stream);

/*
 * Reads word 0 of a workspace after synchronising `stream`: B200_OK, or
 * B200_ERR_DEVICE_TIMEOUT when a bounded wait inside a kernel gave up.
 * `detail` (may be null) receives word 1, which names the wait that ran out.
 */
int b200_workspace_status(const void *workspace, int32_t *detail, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* INTENT_B200_H */

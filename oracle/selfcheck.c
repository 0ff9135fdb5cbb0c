/* TEST INFRASTRUCTURE: drives the CPU oracle on small cases of the five operators so that it
 * can be run under AddressSanitizer / UndefinedBehaviorSanitizer (tests/test_host_sanitizers.py
 * builds this file together with oracle.c).  Exact-size heap buffers make any read or write
 * past an operand visible; ragged and empty CSR rows, one-column rows and several worker
 * counts are included.  Results are only sanity-checked here: parity lives in the Python tests. */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

int oracle_softmax(const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, int64_t);
int oracle_layer_norm(const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t,
                      int64_t, int64_t, int64_t, float, float, int, int64_t);
int oracle_gemm(const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                int64_t, int64_t, int64_t, int, int, int64_t);
int oracle_attention(const void *, const void *, const void *, void *, int64_t, int64_t, int64_t, int64_t, int64_t,
                     int64_t, int64_t, const int64_t *, const int64_t *, const int64_t *, const int64_t *, float,
                     int64_t, int, int, int64_t, int64_t, int64_t, int64_t);
int oracle_csr_validate(const int32_t *, const int32_t *, int64_t, int64_t, int64_t, int64_t *);
int oracle_csr_spmm(const int32_t *, const int32_t *, const float *, const float *, float *, int64_t, int64_t,
                    int64_t, int64_t, int64_t, int64_t, int64_t, int64_t);
int oracle_csr_spmv(const int32_t *, const int32_t *, const float *, const float *, float *, int64_t, int64_t,
                    int64_t, int64_t);

static uint32_t state = 12345u;
static float uniform(void) {
  state = state * 1664525u + 1013904223u;
  return (float)(state >> 8) / 16777216.0f * 2.0f - 1.0f;
}
/* f32 -> bf16 bits, round to nearest even (inputs here are finite) */
static uint16_t bf16(float value) {
  union { float f; uint32_t u; } bits = {value};
  return (uint16_t)((bits.u + 0x7fffu + ((bits.u >> 16) & 1u)) >> 16);
}
static float *floats(size_t count) {
  float *p = (float *)malloc(count ? count * sizeof(float) : 1);
  for (size_t i = 0; i < count; ++i) p[i] = uniform();
  return p;
}
static uint16_t *halves(size_t count) {
  uint16_t *p = (uint16_t *)malloc(count ? count * 2 : 1);
  for (size_t i = 0; i < count; ++i) p[i] = bf16(uniform());
  return p;
}
#define CHECK(condition)                                                          \
  do {                                                                            \
    if (!(condition)) { fprintf(stderr, "selfcheck failed: %s (line %d)\n", #condition, __LINE__); return 1; } \
  } while (0)

int main(void) {
  for (int64_t workers = 1; workers <= 3; ++workers) {
    /* softmax f32: ragged widths incl. a single column */
    const int64_t widths[] = {1, 7, 64, 1000};
    for (int w = 0; w < 4; ++w) {
      const int64_t m = 5, n = widths[w];
      float *x = floats((size_t)(m * n)), *y = floats((size_t)(m * n));
      CHECK(oracle_softmax(x, y, m, n, n, 1, n, 1, 0, workers) == 0);
      for (int64_t r = 0; r < m; ++r) {
        double sum = 0.0;
        for (int64_t c = 0; c < n; ++c) sum += y[r * n + c];
        CHECK(fabs(sum - 1.0) < 1e-4);
      }
      free(x); free(y);
    }
    /* layer norm bf16 (dtype code 2) */
    {
      const int64_t m = 6, n = 96;
      uint16_t *x = halves((size_t)(m * n)), *g = halves((size_t)n), *b = halves((size_t)n), *y = halves((size_t)(m * n));
      CHECK(oracle_layer_norm(x, g, b, y, m, n, n, 1, 1, 1, n, 1, 1.0f / (float)n, 1e-5f, 2, workers) == 0);
      free(x); free(g); free(b); free(y);
    }
    /* gemm bf16: K-major B (strides 1, K), a block of rows only */
    {
      const int64_t m = 9, n = 11, k = 40;
      uint16_t *a = halves((size_t)(m * k)), *bt = halves((size_t)(n * k)), *c = halves((size_t)(m * n));
      CHECK(oracle_gemm(a, bt, c, 2, 5, n, k, k, 1, 1, k, n, 1, 2, 1, workers) == 0);
      free(a); free(bt); free(c);
    }
    /* attention bf16: GQA (4 query heads on 2 key heads), causal, chunks that do not divide the sequence */
    {
      const int64_t batch = 1, hq = 4, hk = 2, s = 37, d = 64;
      uint16_t *q = halves((size_t)(batch * hq * s * d)), *kk = halves((size_t)(batch * hk * s * d)),
               *v = halves((size_t)(batch * hk * s * d)), *o = halves((size_t)(batch * hq * s * d));
      const int64_t qs[4] = {hq * s * d, s * d, d, 1}, ks[4] = {hk * s * d, s * d, d, 1};
      CHECK(oracle_attention(q, kk, v, o, batch, hq, hk, s, s, d, d, qs, ks, ks, qs, 0.125f, 2, 1, 2, 16, 0,
                             batch * hq, workers) == 0);
      free(q); free(kk); free(v); free(o);
    }
    /* CSR: empty rows, a long row, a last row that ends the arrays */
    {
      const int64_t rows = 6, columns = 9, features = 5;
      const int32_t offsets[7] = {0, 0, 3, 3, 12, 13, 13};
      int32_t cols[13];
      for (int i = 0; i < 13; ++i) cols[i] = (int32_t)((i * 5) % columns);
      float *values = floats(13), *dense = floats((size_t)(columns * features)), *out = floats((size_t)(rows * features));
      int32_t *heap_offsets = (int32_t *)malloc(sizeof offsets), *heap_cols = (int32_t *)malloc(sizeof cols);
      for (int i = 0; i < 7; ++i) heap_offsets[i] = offsets[i];
      for (int i = 0; i < 13; ++i) heap_cols[i] = cols[i];
      int64_t where = -1;
      CHECK(oracle_csr_validate(heap_offsets, heap_cols, rows, 13, columns, &where) == 0);
      CHECK(oracle_csr_spmm(heap_offsets, heap_cols, values, dense, out, 0, rows, features, features, 1, features, 1,
                            workers) == 0);
      for (int64_t f = 0; f < features; ++f) CHECK(out[0 * features + f] == 0.0f && out[5 * features + f] == 0.0f);
      float *vector = floats((size_t)columns), *result = floats((size_t)rows);
      CHECK(oracle_csr_spmv(heap_offsets, heap_cols, values, vector, result, rows, 1, 1, workers) == 0);
      CHECK(result[2] == 0.0f);
      heap_cols[4] = (int32_t)columns;                 /* out of range: the validator must say where */
      CHECK(oracle_csr_validate(heap_offsets, heap_cols, rows, 13, columns, &where) != 0 && where == 4);
      free(values); free(dense); free(out); free(heap_offsets); free(heap_cols); free(vector); free(result);
    }
  }
  printf("selfcheck ok\n");
  return 0;
}

/*
 * TEST INFRASTRUCTURE - not product code.  Only tests, the smoke check and the CPU-baseline leg of
 * the benchmark may call this; the shipped operators never do.
 *
 * Plain-C restatement of the upstream project's sequential CPU loops for the reduction hot path.
 * Each function names the upstream loop it follows (file:line within rusty1s/pytorch_scatter).
 * Parity status: PINNED - tests/test_oracle.py checks every function here against the upstream
 * test-suite's known-answer tables and against outputs of the upstream CPU libraries themselves
 * (tests/golden/, produced by tests/golden/make_golden.py).
 *
 * Shapes are the flattened ones of the upstream loops: src [B,E,K], out [B,N,K], int64 indices.
 * One instantiation per arithmetic type: f32, f64, i32, i64, u8, i8, i16.  16-bit floats are checked through the
 * f32 instantiation on up-converted inputs (upstream accumulates them in fp32 for the segment ops,
 * csrc/cpu/segment_csr_cpu.cpp:62) and rounded by the caller.
 *
 * reduce codes: 0 sum, 1 mean, 2 min, 3 max, 4 mul (csrc/cpu/reducer.h:6-11).
 */
#include <float.h>
#include <limits.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

enum { R_SUM = 0, R_MEAN = 1, R_MIN = 2, R_MAX = 3, R_MUL = 4 };

#define DEFINE_ORACLE(SUFFIX, T, TMAX, TLOWEST)                                                            \
  /* identity of a reduction: csrc/cpu/reducer.h:44-53 */                                                  \
  static T init_##SUFFIX(int reduce) {                                                                     \
    if (reduce == R_MUL) return (T)1;                                                                      \
    if (reduce == R_MIN) return TMAX;                                                                      \
    if (reduce == R_MAX) return TLOWEST;                                                                   \
    return (T)0;                                                                                           \
  }                                                                                                        \
  /* one update step, strict comparisons so the first winner stays: csrc/cpu/reducer.h:55-68 */            \
  static void update_##SUFFIX(int reduce, T *val, T new_val, int64_t *arg, int64_t new_arg) {              \
    if (reduce == R_SUM || reduce == R_MEAN) *val = *val + new_val;                                        \
    else if (reduce == R_MUL) *val = *val * new_val;                                                       \
    else if ((reduce == R_MIN && new_val < *val) || (reduce == R_MAX && new_val > *val)) {                 \
      *val = new_val;                                                                                      \
      *arg = new_arg;                                                                                      \
    }                                                                                                      \
  }                                                                                                        \
  /* result write: csrc/cpu/reducer.h:70-83 (count is an int upstream) */                                  \
  static void write_##SUFFIX(int reduce, T *address, T val, int64_t *arg_address, int64_t arg, int count) {\
    if (reduce == R_SUM || reduce == R_MUL) *address = val;                                                \
    else if (reduce == R_MEAN) *address = val / (T)(count > 0 ? count : 1);                                \
    else if (count > 0) {                                                                                  \
      *address = val;                                                                                      \
      *arg_address = arg;                                                                                  \
    } else                                                                                                 \
      *address = (T)0;                                                                                     \
  }                                                                                                        \
                                                                                                           \
  /* segment_csr_cpu main loop: csrc/cpu/segment_csr_cpu.cpp:69-87.  arg_out must be pre-filled with E */  \
  /* by the caller for min/max (csrc/cpu/segment_csr_cpu.cpp:44-48).  indptr row b at b*ip_bstride.    */  \
  void oracle_segment_csr_##SUFFIX(const T *src, const int64_t *indptr, T *out, int64_t *arg_out,          \
                                   int64_t B, int64_t E, int64_t K, int64_t N, int64_t ip_bstride,         \
                                   int reduce) {                                                           \
    T *vals = (T *)malloc(sizeof(T) * (size_t)(K > 0 ? K : 1));                                            \
    int64_t *args = (int64_t *)calloc((size_t)(K > 0 ? K : 1), sizeof(int64_t));                           \
    for (int64_t b = 0; b < B; b++)                                                                        \
      for (int64_t n = 0; n < N; n++) {                                                                    \
        const int64_t row_start = indptr[b * ip_bstride + n], row_end = indptr[b * ip_bstride + n + 1];    \
        for (int64_t k = 0; k < K; k++) vals[k] = init_##SUFFIX(reduce);                                   \
        for (int64_t e = row_start; e < row_end; e++)                                                      \
          for (int64_t k = 0; k < K; k++)                                                                  \
            update_##SUFFIX(reduce, &vals[k], src[(b * E + e) * K + k], &args[k], e);                      \
        for (int64_t k = 0; k < K; k++)                                                                    \
          write_##SUFFIX(reduce, out + (b * N + n) * K + k, vals[k],                                       \
                         arg_out ? arg_out + (b * N + n) * K + k : NULL, args[k],                          \
                         (int)(row_end - row_start));                                                      \
      }                                                                                                    \
    free(vals);                                                                                            \
    free(args);                                                                                            \
  }                                                                                                        \
                                                                                                           \
  /* gather_csr_cpu main loop: csrc/cpu/segment_csr_cpu.cpp:143-158.  src [B,N,K] -> out [B,E,K] */        \
  void oracle_gather_csr_##SUFFIX(const T *src, const int64_t *indptr, T *out, int64_t B, int64_t E,       \
                                  int64_t K, int64_t N, int64_t ip_bstride) {                              \
    for (int64_t b = 0; b < B; b++)                                                                        \
      for (int64_t n = 0; n < N; n++) {                                                                    \
        const int64_t row_start = indptr[b * ip_bstride + n], row_end = indptr[b * ip_bstride + n + 1];    \
        for (int64_t e = row_start; e < row_end; e++)                                                      \
          for (int64_t k = 0; k < K; k++) out[(b * E + e) * K + k] = src[(b * N + n) * K + k];             \
      }                                                                                                    \
  }                                                                                                        \
                                                                                                           \
  /* segment_coo_cpu main loop: csrc/cpu/segment_coo_cpu.cpp:84-137.  `out` must hold the caller's     */  \
  /* values when has_out, is filled with the identity here otherwise; arg_out pre-filled with E;        */  \
  /* count_out [B,N] zero-filled by the caller for mean.  index row b at b*ix_bstride.                  */  \
  void oracle_segment_coo_##SUFFIX(const T *src, const int64_t *index, T *out, int64_t *arg_out,           \
                                   T *count_out, int64_t B, int64_t E, int64_t K, int64_t N,               \
                                   int64_t ix_bstride, int reduce, int has_out) {                          \
    if (!has_out)                                                                                          \
      for (int64_t i = 0; i < B * N * K; i++) out[i] = init_##SUFFIX(reduce);                              \
    if (E == 0) return;                                                                                    \
    T *vals = (T *)malloc(sizeof(T) * (size_t)(K > 0 ? K : 1));                                            \
    int64_t *args = (int64_t *)calloc((size_t)(K > 0 ? K : 1), sizeof(int64_t));                           \
    for (int64_t b = 0; b < B; b++) {                                                                      \
      const int64_t *ix = index + b * ix_bstride;                                                          \
      int64_t idx = ix[0], row_start = 0;                                                                  \
      /* upstream seeds the first run from row 0 of the batch, not from row idx (segment_coo_cpu.cpp:91-92) */\
      for (int64_t k = 0; k < K; k++) vals[k] = out[(b * N + 0) * K + k];                                  \
      for (int64_t e = 0; e < E; e++) {                                                                    \
        for (int64_t k = 0; k < K; k++)                                                                    \
          update_##SUFFIX(reduce, &vals[k], src[(b * E + e) * K + k], &args[k], e);                        \
        const int last = (e == E - 1);                                                                     \
        const int64_t next_idx = last ? idx : ix[e + 1];                                                   \
        if (last || idx != next_idx) {                                                                     \
          for (int64_t k = 0; k < K; k++) {                                                                \
            write_##SUFFIX(reduce, out + (b * N + idx) * K + k, vals[k],                                   \
                           arg_out ? arg_out + (b * N + idx) * K + k : NULL, args[k],                      \
                           (int)(e + 1 - row_start));                                                      \
            if (!last) vals[k] = out[(b * N + next_idx) * K + k];                                          \
          }                                                                                                \
          if (reduce == R_MEAN && count_out) count_out[b * N + idx] = (T)(e + 1 - row_start);              \
          row_start = e + 1;                                                                               \
        }                                                                                                  \
        idx = next_idx;                                                                                    \
      }                                                                                                    \
    }                                                                                                      \
    if (!has_out && (reduce == R_MIN || reduce == R_MAX))                                                  \
      for (int64_t i = 0; i < B * N * K; i++)                                                              \
        if (out[i] == init_##SUFFIX(reduce)) out[i] = (T)0;                                                \
    if (reduce == R_MEAN && count_out)                                                                     \
      for (int64_t i = 0; i < B * N; i++)                                                                  \
        if (count_out[i] < (T)1) count_out[i] = (T)1;                                                      \
    free(vals);                                                                                            \
    free(args);                                                                                            \
  }                                                                                                        \
                                                                                                           \
  /* gather_coo_cpu main loop: csrc/cpu/segment_coo_cpu.cpp:192-211.  src [B,N,K] -> out [B,E,K] */        \
  void oracle_gather_coo_##SUFFIX(const T *src, const int64_t *index, T *out, int64_t B, int64_t E,        \
                                  int64_t K, int64_t N, int64_t ix_bstride) {                              \
    for (int64_t b = 0; b < B; b++)                                                                        \
      for (int64_t e = 0; e < E; e++) {                                                                    \
        const int64_t idx = index[b * ix_bstride + e];                                                     \
        for (int64_t k = 0; k < K; k++) out[(b * E + e) * K + k] = src[(b * N + idx) * K + k];             \
      }                                                                                                    \
  }                                                                                                        \
                                                                                                           \
  /* scatter_cpu main loop: csrc/cpu/scatter_cpu.cpp:63-82.  index addressed with three strides over */    \
  /* the flattened [B,E,K] view.  `out` holds the caller's values when has_out; arg_out pre-filled.  */    \
  /* For reduce == mean this computes the sum, the element count in count_out [Bc,N,Kc] (int64) and  */    \
  /* the divide the way the Python wrapper does: torch_scatter/scatter.py:44-66 (true divide for     */    \
  /* floats, floor divide for integers, selected by is_float).                                        */    \
  void oracle_scatter_##SUFFIX(const T *src, const int64_t *index, T *out, int64_t *arg_out,               \
                               int64_t *count_out, int64_t B, int64_t E, int64_t K, int64_t N, int64_t sb, \
                               int64_t se, int64_t sk, int reduce, int has_out, int is_float) {            \
    const int r = (reduce == R_MEAN) ? R_SUM : reduce;                                                     \
    if (!has_out)                                                                                          \
      for (int64_t i = 0; i < B * N * K; i++) out[i] = init_##SUFFIX(r);                                   \
    const int64_t Bc = sb ? B : 1, Kc = sk ? K : 1;                                                        \
    if (reduce == R_MEAN) memset(count_out, 0, sizeof(int64_t) * (size_t)(Bc * N * Kc));                   \
    for (int64_t b = 0; b < B; b++)                                                                        \
      for (int64_t e = 0; e < E; e++)                                                                      \
        for (int64_t k = 0; k < K; k++) {                                                                  \
          const int64_t idx = index[b * sb + e * se + k * sk];                                             \
          update_##SUFFIX(r, out + (b * N + idx) * K + k, src[(b * E + e) * K + k],                        \
                          arg_out ? arg_out + (b * N + idx) * K + k : NULL, e);                            \
          if (reduce == R_MEAN && (sb || b == 0) && (sk || k == 0))                                        \
            count_out[((sb ? b : 0) * N + idx) * Kc + (sk ? k : 0)] += 1;                                  \
        }                                                                                                  \
    if (!has_out && (r == R_MIN || r == R_MAX))                                                            \
      for (int64_t i = 0; i < B * N * K; i++)                                                              \
        if (out[i] == init_##SUFFIX(r)) out[i] = (T)0;                                                     \
    if (reduce == R_MEAN)                                                                                  \
      for (int64_t b = 0; b < B; b++)                                                                      \
        for (int64_t n = 0; n < N; n++)                                                                    \
          for (int64_t k = 0; k < K; k++) {                                                                \
            int64_t c = count_out[((sb ? b : 0) * N + n) * Kc + (sk ? k : 0)];                             \
            if (c < 1) c = 1;                                                                              \
            T *o = out + (b * N + n) * K + k;                                                              \
            if (is_float) *o = *o / (T)c;                                                                  \
            else {                                                                                         \
              T q = *o / (T)c;                                                                             \
              if ((*o - q * (T)c != (T)0) && (*o < (T)0)) q = q - (T)1;                                    \
              *o = q;                                                                                      \
            }                                                                                              \
          }                                                                                                \
  }

DEFINE_ORACLE(f32, float, FLT_MAX, -FLT_MAX)
DEFINE_ORACLE(f64, double, DBL_MAX, -DBL_MAX)
DEFINE_ORACLE(i32, int32_t, INT32_MAX, INT32_MIN)
DEFINE_ORACLE(i64, int64_t, INT64_MAX, INT64_MIN)
/* the narrow integers upstream dispatches as well (AT_DISPATCH_ALL_TYPES_AND2): arithmetic in the type itself, i.e.
 * promoted to int and narrowed back after every step, as the C++ loops do */
DEFINE_ORACLE(u8, uint8_t, UINT8_MAX, 0)
DEFINE_ORACLE(i8, int8_t, INT8_MAX, INT8_MIN)
DEFINE_ORACLE(i16, int16_t, INT16_MAX, INT16_MIN)

// scatter (unsorted index) for sm_100a.
//
// Accumulation happens in a target buffer of the accumulation type U: `out` itself for 32/64-bit
// types, an fp32 workspace for fp16/bf16 (so 16-bit sums are accumulated in fp32 and rounded once).
//   SUM/MEAN  vectorised reductions: one red.global.add.v4.f32 per 16 bytes for fp32 targets, native
//             atomic adds for f64/i32/i64.  MEAN counts elements per target in an int32 tensor and a
//             finalize pass divides.
//   MIN/MAX   floating targets are kept as order-preserving integer keys so that a single native
//             atomicMin/atomicMax resolves each update; a plain load filters updates that cannot win.
//             A second pass finds the arg index as the smallest position whose value equals the
//             result (atomicMin on int64), which is the first-occurrence rule of the CPU loop
//             (csrc/cpu/reducer.h:63-67).
//   MUL       compare-and-swap loop (kept for operator-set completeness).
// When the index is the same for all K features of a row (a broadcast 1-D index, stride_k == 0) the
// row kernels read it once per row and move the row in 16-byte packs; otherwise an element kernel
// handles one (b,e,k) per thread.
//
// Replaces scatter_kernel / scatter_arg_kernel of the upstream project
// (csrc/cuda/scatter_cuda.cu:13-56): one atomic per element, CAS loops for float MIN/MAX and all
// 16-bit types, K redundant index loads per row and a racy arg pass.
#include <cstdlib>

#include "common.cuh"

namespace tsb {
namespace {

// ---- order-preserving integer keys -----------------------------------------------------------
template <typename U> struct KeyOf { using type = U; };
template <> struct KeyOf<float> { using type = int32_t; };
template <> struct KeyOf<double> { using type = int64_t; };
template <typename U> using key_t = typename KeyOf<U>::type;

// -0.0 is folded onto +0.0 first (the CPU comparison treats them as equal).
__device__ __forceinline__ int32_t enc_key(float f) {
  const int32_t b = __float_as_int(f + 0.0f);
  return b >= 0 ? b : (b ^ 0x7fffffff);
}
__device__ __forceinline__ int64_t enc_key(double f) {
  const int64_t b = __double_as_longlong(f + 0.0);
  return b >= 0 ? b : (b ^ 0x7fffffffffffffffLL);
}
__device__ __forceinline__ int32_t enc_key(int32_t v) { return v; }
__device__ __forceinline__ int64_t enc_key(int64_t v) { return v; }
template <typename U> __device__ __forceinline__ U dec_key(key_t<U> k);
template <> __device__ __forceinline__ float dec_key<float>(int32_t k) { return __int_as_float(k >= 0 ? k : (k ^ 0x7fffffff)); }
template <> __device__ __forceinline__ double dec_key<double>(int64_t k) {
  return __longlong_as_double(k >= 0 ? k : (k ^ 0x7fffffffffffffffLL));
}
template <> __device__ __forceinline__ int32_t dec_key<int32_t>(int32_t k) { return k; }
template <> __device__ __forceinline__ int64_t dec_key<int64_t>(int64_t k) { return k; }

template <typename U> __device__ __forceinline__ bool is_nan(U) { return false; }
template <> __device__ __forceinline__ bool is_nan<float>(float v) { return v != v; }
template <> __device__ __forceinline__ bool is_nan<double>(double v) { return v != v; }

// ---- atomics on the target ---------------------------------------------------------------------
__device__ __forceinline__ void atom_add(float *a, float v) { atomicAdd(a, v); }
__device__ __forceinline__ void atom_add(double *a, double v) { atomicAdd(a, v); }
__device__ __forceinline__ void atom_add(int32_t *a, int32_t v) { atomicAdd(a, v); }
__device__ __forceinline__ void atom_add(int64_t *a, int64_t v) {
  atomicAdd(reinterpret_cast<unsigned long long *>(a), (unsigned long long)v);
}
__device__ __forceinline__ void red_add_v4(float *a, float x, float y, float z, float w) {
  asm volatile("red.global.v4.f32.add [%0], {%1, %2, %3, %4};" ::"l"(a), "f"(x), "f"(y), "f"(z), "f"(w) : "memory");
}

__device__ __forceinline__ void atom_mul(float *a, float v) {
  int *ai = reinterpret_cast<int *>(a);
  int old = *ai, assumed;
  do {
    assumed = old;
    old = atomicCAS(ai, assumed, __float_as_int(__int_as_float(assumed) * v));
  } while (assumed != old);
}
__device__ __forceinline__ void atom_mul(double *a, double v) {
  unsigned long long *ai = reinterpret_cast<unsigned long long *>(a);
  unsigned long long old = *ai, assumed;
  do {
    assumed = old;
    old = atomicCAS(ai, assumed, (unsigned long long)__double_as_longlong(__longlong_as_double((long long)assumed) * v));
  } while (assumed != old);
}
__device__ __forceinline__ void atom_mul(int32_t *a, int32_t v) {
  int old = *a, assumed;
  do {
    assumed = old;
    old = atomicCAS(a, assumed, assumed * v);
  } while (assumed != old);
}
__device__ __forceinline__ void atom_mul(int64_t *a, int64_t v) {
  unsigned long long *ai = reinterpret_cast<unsigned long long *>(a);
  unsigned long long old = *ai, assumed;
  do {
    assumed = old;
    old = atomicCAS(ai, assumed, (unsigned long long)((long long)assumed * v));
  } while (assumed != old);
}

__device__ __forceinline__ void atom_min_key(int32_t *a, int32_t k) {
  if (k < *reinterpret_cast<volatile int32_t *>(a)) atomicMin(a, k);
}
__device__ __forceinline__ void atom_max_key(int32_t *a, int32_t k) {
  if (k > *reinterpret_cast<volatile int32_t *>(a)) atomicMax(a, k);
}
__device__ __forceinline__ void atom_min_key(int64_t *a, int64_t k) {
  if (k < *reinterpret_cast<volatile int64_t *>(a)) atomicMin(reinterpret_cast<long long *>(a), (long long)k);
}
__device__ __forceinline__ void atom_max_key(int64_t *a, int64_t k) {
  if (k > *reinterpret_cast<volatile int64_t *>(a)) atomicMax(reinterpret_cast<long long *>(a), (long long)k);
}

template <int OP, typename U> __device__ __forceinline__ void apply_one(U *addr, U x) {
  if (OP == kSum) {
    atom_add(addr, x);
  } else if (OP == kMul) {
    atom_mul(addr, x);
  } else {
    if (is_nan(x)) return;  // a NaN never wins a strict comparison
    key_t<U> *ka = reinterpret_cast<key_t<U> *>(addr);
    if (OP == kMin) atom_min_key(ka, enc_key(x));
    else atom_max_key(ka, enc_key(x));
  }
}

template <int OP, typename T, int VEC>
__device__ __forceinline__ void apply_pack(acc_t<T> *addr, const Pack<T, VEC> &v) {
  using U = acc_t<T>;
  if constexpr (OP == kSum && std::is_same<U, float>::value && (VEC % 4 == 0)) {
#pragma unroll
    for (int i = 0; i < VEC; i += 4) {
      red_add_v4(addr + i, to_acc<T>(v.v[i]), to_acc<T>(v.v[i + 1]), to_acc<T>(v.v[i + 2]), to_acc<T>(v.v[i + 3]));
    }
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) apply_one<OP, U>(addr + i, to_acc<T>(v.v[i]));
  }
}

struct ScatterParams {
  const void *src;
  const int64_t *index;
  void *out;        // [B,N,K] of T
  void *target;     // [B,N,K] of acc_t<T>: == out, or the fp32 workspace
  int64_t *arg_out;
  int32_t *count;   // [Bc,N,Kc] or null
  int64_t B, E, K, N, sb, se, sk;
  int l_log2;
  int fresh;
};

// ---- row kernels: index constant along k ------------------------------------------------------
template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(kThreads) scatter_rows_kernel(ScatterParams p) {
  using U = acc_t<T>;
  const T *__restrict__ src = static_cast<const T *>(p.src);
  U *target = static_cast<U *>(p.target);
  const int L = 1 << p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t entry = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> p.l_log2;
  const int col = threadIdx.x & (L - 1);
  if (entry >= p.B * p.E) return;
  const int64_t b = entry / p.E, e = entry - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se];
  if (idx < 0 || idx >= p.N) return;
  const T *srow = src + entry * p.K;
  U *trow = target + (b * p.N + idx) * p.K;
  for (int64_t c = col; c < Kv; c += L) apply_pack<OP, T, VEC>(trow + c * VEC, ld_stream<T, VEC>(srow + c * VEC));
  // one count per row of the index itself: a batch-broadcast index is counted for b == 0 only
  if (p.count != nullptr && col == 0 && (p.sb != 0 || b == 0)) atomicAdd(p.count + (p.sb ? b : 0) * p.N + idx, 1);
}

// Row kernel restricted to the target rows [lo, hi) (rows counted over all batches, b*N + idx).
// When the output is larger than L2, the launcher runs one such pass per slice of the output so that
// the slice being accumulated stays L2-resident: every pass re-reads the whole index (8 bytes per
// entry) but only the source rows whose target lies in the slice, and the read-modify-write traffic
// of the atomics no longer reaches DRAM.  A warp issues the index loads
// of its 128 consecutive entries, compacts the matching ones through shared memory and then moves
// them 32/L rows per step, four steps in flight.
constexpr int kRangeBatches = 4;  // 32-entry batches a warp looks at per launch slot

template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(kThreads) scatter_rows_range_kernel(ScatterParams p, int64_t lo, int64_t hi) {
  using U = acc_t<T>;
  constexpr int kWarps = kThreads / 32;
  constexpr int kSteps = 4;
  constexpr int kCap = 32 * kRangeBatches;
  __shared__ int64_t s_ent[kWarps][kCap];
  __shared__ int64_t s_trow[kWarps][kCap];
  const T *__restrict__ src = static_cast<const T *>(p.src);
  U *target = static_cast<U *>(p.target);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = 1 << p.l_log2;
  const int col = lane & (L - 1);
  const int sub = lane >> p.l_log2;
  const int eps = 32 >> p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t M = p.B * p.E;
  const int64_t base = ((int64_t)blockIdx.x * kWarps + warp) * kCap;
  if (base >= M) return;  // warp-uniform
  // all index loads of the warp's batches are issued before any is used
  int64_t ent[kRangeBatches], trow[kRangeBatches];
#pragma unroll
  for (int q = 0; q < kRangeBatches; ++q) {
    ent[q] = base + q * 32 + lane;
    trow[q] = -1;
    if (ent[q] < M) {
      const int64_t b = (p.B == 1) ? 0 : ent[q] / p.E;
      const int64_t e = ent[q] - b * p.E;
      const int64_t idx = p.index[b * p.sb + e * p.se];
      if (idx >= 0 && idx < p.N) trow[q] = b * p.N + idx;
    }
  }
  int n = 0;
#pragma unroll
  for (int q = 0; q < kRangeBatches; ++q) {
    const bool match = trow[q] >= lo && trow[q] < hi;
    const unsigned mask = __ballot_sync(kFullMask, match);
    if (match) {
      const int r = n + __popc(mask & ((1u << lane) - 1u));
      s_ent[warp][r] = ent[q];
      s_trow[warp][r] = trow[q];
    }
    n += __popc(mask);
  }
  __syncwarp();
  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;
    for (int i = 0; i < n; i += kSteps * eps) {
      Pack<T, VEC> v[kSteps];
      int64_t tr[kSteps];
      bool ok[kSteps];
#pragma unroll
      for (int u = 0; u < kSteps; ++u) {
        const int m = i + u * eps + sub;
        ok[u] = col_ok && m < n;
        if (ok[u]) {
          tr[u] = s_trow[warp][m];
          v[u] = ld_stream<T, VEC>(src + s_ent[warp][m] * p.K + c * VEC);
        }
      }
#pragma unroll
      for (int u = 0; u < kSteps; ++u) {
        if (ok[u]) {
          apply_pack<OP, T, VEC>(target + tr[u] * p.K + c * VEC, v[u]);
          if (p.count != nullptr && c == 0) {
            const int64_t b = tr[u] / p.N;
            if (p.sb != 0 || b == 0) atomicAdd(p.count + (p.sb ? tr[u] : tr[u] - b * p.N), 1);
          }
        }
      }
    }
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) scatter_elems_kernel(ScatterParams p) {
  using U = acc_t<T>;
  const T *__restrict__ src = static_cast<const T *>(p.src);
  U *target = static_cast<U *>(p.target);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= p.B * p.E * p.K) return;
  const int64_t k = i % p.K, be = i / p.K;
  const int64_t b = be / p.E, e = be - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se + k * p.sk];
  if (idx < 0 || idx >= p.N) return;
  apply_one<OP, U>(target + (b * p.N + idx) * p.K + k, to_acc<T>(src[i]));
  if (p.count != nullptr && (p.sb != 0 || b == 0)) atomicAdd(p.count + ((p.sb ? b : 0) * p.N + idx) * p.K + k, 1);
}

// ---- init / finalize ---------------------------------------------------------------------------
template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) scatter_init_kernel(const T *out, acc_t<T> *target, int64_t total, int fresh) {
  using U = acc_t<T>;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const U v = fresh ? reduce_identity<T, OP>() : to_acc<T>(out[i]);
  if (OP == kMin || OP == kMax) reinterpret_cast<key_t<U> *>(target)[i] = enc_key(v);
  else target[i] = v;
}

template <typename T> __device__ __forceinline__ T mean_div(T v, int32_t c) { return v / (T)c; }
template <> __device__ __forceinline__ __half mean_div<__half>(__half v, int32_t c) {
  return __float2half_rn(__half2float(v) / __half2float(__int2half_rn(c)));
}
template <> __device__ __forceinline__ __nv_bfloat16 mean_div<__nv_bfloat16>(__nv_bfloat16 v, int32_t c) {
  return __float2bfloat16_rn(__bfloat162float(v) / __bfloat162float(__int2bfloat16_rn(c)));
}
// integer mean rounds toward -inf (torch_scatter/scatter.py:65, div_ with rounding_mode='floor')
template <> __device__ __forceinline__ int32_t mean_div<int32_t>(int32_t v, int32_t c) {
  int32_t q = v / c;
  if ((v % c != 0) && (v < 0)) --q;
  return q;
}
template <> __device__ __forceinline__ int64_t mean_div<int64_t>(int64_t v, int32_t c) {
  int64_t q = v / c;
  if ((v % c != 0) && (v < 0)) --q;
  return q;
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
scatter_finalize_kernel(T *out, const acc_t<T> *target, const int32_t *count, int64_t total, int64_t N, int64_t K,
                        int fresh, int count_b, int count_k) {
  using U = acc_t<T>;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  U v;
  if (OP == kMin || OP == kMax) {
    v = dec_key<U>(reinterpret_cast<const key_t<U> *>(target)[i]);
    if (fresh && v == reduce_identity<T, OP>()) v = (U)0;
  } else {
    v = target[i];
  }
  T r = from_acc<T>(v);
  if (count != nullptr) {
    const int64_t k = i % K, bn = i / K;
    const int64_t n = bn % N, b = bn / N;
    int32_t c = count[((count_b ? b : 0) * N + n) * (count_k ? K : 1) + (count_k ? k : 0)];
    r = mean_div<T>(r, c < 1 ? 1 : c);
  }
  out[i] = r;
}

__global__ void __launch_bounds__(kThreads) fill_i64_kernel(int64_t *p, int64_t total, int64_t value) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < total) p[i] = value;
}

// ---- arg pass ----------------------------------------------------------------------------------
__device__ __forceinline__ void arg_min(int64_t *a, int64_t e) {
  if (e < *reinterpret_cast<volatile int64_t *>(a)) atomicMin(reinterpret_cast<long long *>(a), (long long)e);
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads) scatter_arg_rows_kernel(ScatterParams p) {
  const T *__restrict__ src = static_cast<const T *>(p.src);
  const T *__restrict__ out = static_cast<const T *>(p.out);
  const int L = 1 << p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t entry = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> p.l_log2;
  const int col = threadIdx.x & (L - 1);
  if (entry >= p.B * p.E) return;
  const int64_t b = entry / p.E, e = entry - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se];
  if (idx < 0 || idx >= p.N) return;
  const int64_t obase = (b * p.N + idx) * p.K;
  for (int64_t c = col; c < Kv; c += L) {
    const Pack<T, VEC> v = ld_stream<T, VEC>(src + entry * p.K + c * VEC);
    const Pack<T, VEC> o = ld_pack<T, VEC>(out + obase + c * VEC);
#pragma unroll
    for (int i = 0; i < VEC; ++i)
      if (to_acc<T>(v.v[i]) == to_acc<T>(o.v[i])) arg_min(p.arg_out + obase + c * VEC + i, e);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) scatter_arg_elems_kernel(ScatterParams p) {
  const T *__restrict__ src = static_cast<const T *>(p.src);
  const T *__restrict__ out = static_cast<const T *>(p.out);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= p.B * p.E * p.K) return;
  const int64_t k = i % p.K, be = i / p.K;
  const int64_t b = be / p.E, e = be - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se + k * p.sk];
  if (idx < 0 || idx >= p.N) return;
  const int64_t o = (b * p.N + idx) * p.K + k;
  if (to_acc<T>(src[i]) == to_acc<T>(out[o])) arg_min(p.arg_out + o, e);
}

// ---- backward of SUM / MEAN: a gather --------------------------------------------------------
struct ScatterBwParams {
  const void *grad_out;
  const int64_t *index;
  void *grad_in;
  const int32_t *count;
  int64_t B, E, K, N, sb, se, sk;
  int l_log2;
};

template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads) scatter_bw_rows_kernel(ScatterBwParams p) {
  const T *__restrict__ go = static_cast<const T *>(p.grad_out);
  T *__restrict__ gi = static_cast<T *>(p.grad_in);
  const int L = 1 << p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t entry = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> p.l_log2;
  const int col = threadIdx.x & (L - 1);
  if (entry >= p.B * p.E) return;
  const int64_t b = entry / p.E, e = entry - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se];
  if (idx < 0 || idx >= p.N) return;
  int32_t cnt = 1;
  if (p.count != nullptr) {
    cnt = p.count[(p.sb ? b : 0) * p.N + idx];
    if (cnt < 1) cnt = 1;
  }
  for (int64_t c = col; c < Kv; c += L) {
    Pack<T, VEC> v = ld_pack<T, VEC>(go + (b * p.N + idx) * p.K + c * VEC);
    if (p.count != nullptr) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) v.v[i] = mean_div<T>(v.v[i], cnt);
    }
    st_stream<T, VEC>(gi + entry * p.K + c * VEC, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) scatter_bw_elems_kernel(ScatterBwParams p) {
  const T *__restrict__ go = static_cast<const T *>(p.grad_out);
  T *__restrict__ gi = static_cast<T *>(p.grad_in);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= p.B * p.E * p.K) return;
  const int64_t k = i % p.K, be = i / p.K;
  const int64_t b = be / p.E, e = be - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se + k * p.sk];
  if (idx < 0 || idx >= p.N) return;
  T v = go[(b * p.N + idx) * p.K + k];
  if (p.count != nullptr) {
    int32_t cnt = p.count[((p.sb ? b : 0) * p.N + idx) * (p.sk ? p.K : 1) + (p.sk ? k : 0)];
    v = mean_div<T>(v, cnt < 1 ? 1 : cnt);
  }
  gi[i] = v;
}

inline int64_t env_bytes(const char *name, int64_t fallback) {
  const char *v = std::getenv(name);
  if (v == nullptr || *v == '\0') return fallback;
  const long long x = std::atoll(v);
  return x > 0 ? (int64_t)x : fallback;
}

inline bool grid_for(int64_t threads, unsigned *blocks) {
  const int64_t nb = (threads + kThreads - 1) / kThreads;
  if (nb > 2147483647LL) return false;
  *blocks = (unsigned)nb;
  return true;
}

template <typename T, int OP>
int run_scatter(ScatterParams p, int reduce, cudaStream_t stream) {
  using U = acc_t<T>;
  constexpr bool k16 = sizeof(T) == 2;
  constexpr bool kMinMax = (OP == kMin || OP == kMax);
  constexpr bool kKeyed = kMinMax && !std::is_same<key_t<U>, U>::value;
  constexpr int kFull = full_vec<T>();
  const int64_t total = p.B * p.N * p.K;
  const bool mean = reduce == TSB_MEAN;
  unsigned blocks = 0;

  // An output larger than L2 is accumulated slice by slice (see scatter_rows_range_kernel) when the
  // index is constant along the features and a source row is big enough to pay for re-reading the index.
  const int64_t slice_bytes = env_bytes("TSB_SCATTER_SLICE_BYTES", 128ll << 20);  // test / tuning hook
  const int64_t target_row_bytes = p.K * (int64_t)sizeof(U);
  int64_t slice_rows = target_row_bytes > 0 ? slice_bytes / target_row_bytes : 0;
  if (slice_rows < 1) slice_rows = 1;
  const bool sliced = OP == kSum && p.sk == 0 && p.E > 0 && p.B * p.N > slice_rows + slice_rows / 2 &&
                      p.K * (int64_t)sizeof(T) >= 128;

  // 1. bring the target to its starting state
  if (total > 0) {
    const bool need_init = k16 || kKeyed || p.fresh;
    if (need_init) {
      if (!k16 && !kMinMax && OP == kSum) {
        // sliced passes zero each slice right before accumulating into it (it then never leaves L2)
        if (!sliced && cudaMemsetAsync(p.target, 0, (size_t)total * sizeof(U), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
      } else {
        if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
        scatter_init_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(static_cast<const T *>(p.out),
                                                                     static_cast<U *>(p.target), total, p.fresh);
      }
    }
    if (mean) {
      const int64_t cn = (p.sb ? p.B : 1) * p.N * (p.sk ? p.K : 1);
      if (cudaMemsetAsync(p.count, 0, (size_t)cn * sizeof(int32_t), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
    }
  }

  // 2. the atomics pass
  const bool rows = p.sk == 0;
  const bool vec_ok = rows && (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.target) && aligned16(p.out);
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);
  p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  if (total > 0 && p.E > 0) {
    if (sliced) {
      if (!grid_for((p.B * p.E + kRangeBatches - 1) / kRangeBatches, &blocks)) return TSB_ERR_TOO_LARGE;  // 128 entries per warp
      const bool zero_slices = !k16 && p.fresh;
      for (int64_t lo = 0; lo < p.B * p.N; lo += slice_rows) {
        const int64_t hi = lo + slice_rows < p.B * p.N ? lo + slice_rows : p.B * p.N;
        if (zero_slices && cudaMemsetAsync(static_cast<U *>(p.target) + lo * p.K, 0,
                                           (size_t)((hi - lo) * p.K) * sizeof(U), stream) != cudaSuccess)
          return TSB_ERR_LAUNCH;
        if (vec_ok) scatter_rows_range_kernel<T, OP, kFull><<<blocks, kThreads, 0, stream>>>(p, lo, hi);
        else scatter_rows_range_kernel<T, OP, 1><<<blocks, kThreads, 0, stream>>>(p, lo, hi);
      }
    } else if (rows) {
      if (!grid_for((p.B * p.E) << p.l_log2, &blocks)) return TSB_ERR_TOO_LARGE;
      if (vec_ok) scatter_rows_kernel<T, OP, kFull><<<blocks, kThreads, 0, stream>>>(p);
      else scatter_rows_kernel<T, OP, 1><<<blocks, kThreads, 0, stream>>>(p);
    } else {
      if (!grid_for(p.B * p.E * p.K, &blocks)) return TSB_ERR_TOO_LARGE;
      scatter_elems_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(p);
    }
  }

  // 3. finalize: decode keys, mask untouched MIN/MAX slots, round fp32 accumulators, divide for MEAN
  if (total > 0 && (k16 || kMinMax || mean)) {
    if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
    scatter_finalize_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(
        static_cast<T *>(p.out), static_cast<const U *>(p.target), mean ? p.count : nullptr, total, p.N, p.K,
        p.fresh, p.sb != 0, p.sk != 0);
  }

  // 4. arg pass
  if (kMinMax && total > 0) {
    if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
    fill_i64_kernel<<<blocks, kThreads, 0, stream>>>(p.arg_out, total, p.E);
    if (p.E > 0) {
      if (rows) {
        if (!grid_for((p.B * p.E) << p.l_log2, &blocks)) return TSB_ERR_TOO_LARGE;
        if (vec_ok) scatter_arg_rows_kernel<T, kFull><<<blocks, kThreads, 0, stream>>>(p);
        else scatter_arg_rows_kernel<T, 1><<<blocks, kThreads, 0, stream>>>(p);
      } else {
        if (!grid_for(p.B * p.E * p.K, &blocks)) return TSB_ERR_TOO_LARGE;
        scatter_arg_elems_kernel<T><<<blocks, kThreads, 0, stream>>>(p);
      }
    }
  }
  return launch_status();
}

template <typename T>
int run_scatter_backward(ScatterBwParams p, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  if (p.B * p.E * p.K == 0 || p.N == 0) return TSB_OK;
  unsigned blocks = 0;
  const bool rows = p.sk == 0;
  const bool vec_ok = rows && (p.K % kFull == 0) && aligned16(p.grad_out) && aligned16(p.grad_in);
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);
  p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  if (rows) {
    if (!grid_for((p.B * p.E) << p.l_log2, &blocks)) return TSB_ERR_TOO_LARGE;
    if (vec_ok) scatter_bw_rows_kernel<T, kFull><<<blocks, kThreads, 0, stream>>>(p);
    else scatter_bw_rows_kernel<T, 1><<<blocks, kThreads, 0, stream>>>(p);
  } else {
    if (!grid_for(p.B * p.E * p.K, &blocks)) return TSB_ERR_TOO_LARGE;
    scatter_bw_elems_kernel<T><<<blocks, kThreads, 0, stream>>>(p);
  }
  return launch_status();
}

}  // namespace
}  // namespace tsb

extern "C" size_t tsb_scatter_workspace_bytes(int64_t B, int64_t N, int64_t K, int dtype, int reduce) {
  (void)reduce;
  if (B < 0 || N < 0 || K < 0) return 0;
  if (dtype == TSB_F16 || dtype == TSB_BF16) return (size_t)B * (size_t)N * (size_t)K * sizeof(float);
  return 0;
}

extern "C" int tsb_scatter(const void *src, const int64_t *index, void *out, int64_t *arg_out, int32_t *count_out,
                           int64_t B, int64_t E, int64_t K, int64_t N, int64_t idx_stride_b, int64_t idx_stride_e,
                           int64_t idx_stride_k, int dtype, int reduce, int out_seeded, void *workspace,
                           size_t workspace_bytes, tsb_stream_t stream_) {
  using namespace tsb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (B * N * K == 0) return TSB_OK;
  if (out == nullptr) return TSB_ERR_ARG;
  if (B * E * K > 0 && (src == nullptr || index == nullptr)) return TSB_ERR_ARG;
  if ((reduce == TSB_MIN || reduce == TSB_MAX) && arg_out == nullptr) return TSB_ERR_ARG;
  if (reduce == TSB_MEAN && count_out == nullptr) return TSB_ERR_ARG;
  const size_t need = tsb_scatter_workspace_bytes(B, N, K, dtype, reduce);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) return TSB_ERR_WORKSPACE;
  ScatterParams p;
  p.src = src; p.index = index; p.out = out;
  p.target = need > 0 ? workspace : out;
  p.arg_out = arg_out;
  p.count = reduce == TSB_MEAN ? count_out : nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.sb = idx_stride_b; p.se = idx_stride_e; p.sk = idx_stride_k;
  p.l_log2 = 0;
  p.fresh = out_seeded ? 0 : 1;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    switch (reduce) {
      case TSB_SUM:
      case TSB_MEAN: return run_scatter<scalar_t, kSum>(p, reduce, stream);
      case TSB_MIN: return run_scatter<scalar_t, kMin>(p, reduce, stream);
      case TSB_MAX: return run_scatter<scalar_t, kMax>(p, reduce, stream);
      case TSB_MUL: return run_scatter<scalar_t, kMul>(p, reduce, stream);
      default: return TSB_ERR_REDUCE;
    }
  });
}

extern "C" int tsb_scatter_backward(const void *grad_out, const int64_t *index, void *grad_in, const int32_t *count,
                                    int64_t B, int64_t E, int64_t K, int64_t N, int64_t idx_stride_b,
                                    int64_t idx_stride_e, int64_t idx_stride_k, int dtype, tsb_stream_t stream) {
  using namespace tsb;
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (B * E * K == 0 || N == 0) return TSB_OK;
  if (grad_out == nullptr || index == nullptr || grad_in == nullptr) return TSB_ERR_ARG;
  ScatterBwParams p;
  p.grad_out = grad_out; p.index = index; p.grad_in = grad_in; p.count = count;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.sb = idx_stride_b; p.se = idx_stride_e; p.sk = idx_stride_k;
  p.l_log2 = 0;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    return run_scatter_backward<scalar_t>(p, reinterpret_cast<cudaStream_t>(stream));
  });
}

// scatter (unsorted index) for sm_100a.
//
// Accumulation happens in a target buffer of the accumulation type U: `out` itself for 32/64-bit
// types, an fp32 workspace for fp16/bf16 (so 16-bit sums are accumulated in fp32 and rounded once).
//   SUM/MEAN  vectorised reductions: one red.global.add.v4.f32 per 16 bytes for fp32 targets, native
//             atomic adds for f64/i32/i64.  MEAN counts elements per target in an int32 tensor and a
//             finalize pass divides.
//   MIN/MAX   4-byte accumulation types (fp32, int32, and fp16/bf16 compared as fp32): the value's
//             order-preserving key and the element's position are packed into 64 bits and ONE native
//             64-bit atomicMax/atomicMin settles value and arg together, first occurrence winning ties
//             as in the CPU loop (csrc/cpu/reducer.h:63-67); a plain load filters updates that cannot
//             win.  8-byte types keep ordered keys plus a second pass that takes the smallest position
//             whose value equals the result.
//   MUL       compare-and-swap loop (kept for operator-set completeness).
// When the index is the same for all K features of a row (a broadcast 1-D index, stride_k == 0) the
// row kernel reads it once per row, moves the row in 16-byte packs and combines the entries of a warp
// that share a target before touching global memory; otherwise an element kernel handles one (b,e,k)
// per thread.  Small outputs are accumulated into several copies (less contention per address),
// outputs larger than L2 slice by slice (the slice being accumulated stays L2-resident).
//
// Replaces scatter_kernel / scatter_arg_kernel of the upstream project
// (csrc/cuda/scatter_cuda.cu:13-56): one atomic per element, CAS loops for float MIN/MAX and all
// 16-bit types, K redundant index loads per row and a racy arg pass.
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "scatter_grouped.cuh"

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
  int replicas;        // copies of the output the updates are spread over (1: none)
  int binned;          // 1: scatter_rows_binned_kernel is launched too and takes the indices the probe calls skewed
  const int *clustered;  // device flags written by scatter_probe_kernel: [0] 1 = neighbouring entries share targets,
                         // [1] 1 = entries far apart often share targets (a skewed index)
};

// One CTA looks at four windows of 256 consecutive index entries and counts neighbours that name the
// same target.  An index where that is common (an edge list sorted or clustered by destination) is
// handed to the run-combining kernel, any other to the direct kernels; the verdict is a device-side
// flag, so choosing the variant costs no host synchronisation.
__global__ void __launch_bounds__(kThreads) scatter_probe_kernel(ScatterParams p, int *clustered, int forced, int forced_skew) {
  __shared__ int s_equal, s_pairs, s_far_equal, s_far_pairs;
  if (threadIdx.x == 0) { s_equal = 0; s_pairs = 0; s_far_equal = 0; s_far_pairs = 0; }
  __syncthreads();
  const int64_t M = p.B * p.E;
  // four windows of 256 neighbouring pairs, and for each first entry a partner 1021 entries further on;
  // all twelve loads of a thread are independent
  int64_t x[4], y[4], z[4];
  bool ok[4], far_ok[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    const int64_t i = (M / 4) * w + threadIdx.x;
    ok[w] = i + 1 < M;
    far_ok[w] = i + 1021 < M;
    x[w] = y[w] = z[w] = 0;
    if (ok[w]) {
      const int64_t b0 = (p.B == 1) ? 0 : i / p.E, b1 = (p.B == 1) ? 0 : (i + 1) / p.E;
      x[w] = p.index[b0 * p.sb + (i - b0 * p.E) * p.se];
      y[w] = p.index[b1 * p.sb + (i + 1 - b1 * p.E) * p.se];
      ok[w] = b0 == b1;
      if (far_ok[w]) {
        const int64_t b2 = (p.B == 1) ? 0 : (i + 1021) / p.E;
        z[w] = p.index[b2 * p.sb + (i + 1021 - b2 * p.E) * p.se];
        far_ok[w] = b0 == b2;
      }
    } else {
      far_ok[w] = false;
    }
  }
  int equal = 0, pairs = 0, far_equal = 0, far_pairs = 0;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    if (ok[w]) {
      pairs += 1;
      equal += (x[w] == y[w]) ? 1 : 0;
    }
    if (far_ok[w]) {
      far_pairs += 1;
      far_equal += (x[w] == z[w]) ? 1 : 0;
    }
  }
  atomicAdd(&s_equal, equal);
  atomicAdd(&s_pairs, pairs);
  atomicAdd(&s_far_equal, far_equal);
  atomicAdd(&s_far_pairs, far_pairs);
  __syncthreads();
  if (threadIdx.x == 0) {
    // test hooks: the caller may dictate either verdict
    clustered[0] = forced >= 0 ? forced : ((s_pairs > 0 && s_equal * 8 >= s_pairs) ? 1 : 0);
    // two entries far apart name the same row with probability sum p_k^2: about 5 % for Zipf(1.2) over 100,000 rows,
    // 0.0015 % for a uniform index over 65,536; the cache pays from about 1 %
    clustered[1] = forced_skew >= 0 ? forced_skew : ((s_far_pairs >= 64 && s_far_equal * 100 >= s_far_pairs) ? 1 : 0);
  }
}

// ---- direct row kernels: one update per entry ---------------------------------------------------
// L lanes own one entry and move its K values in 16-byte packs; the index is read once per entry.
// The second kernel is the same restricted to the target rows [lo, hi) (rows counted over all batches):
// when the output is larger than L2 the launcher runs one such pass per slice of the output, so that
// the slice being accumulated stays L2-resident.  Every pass re-reads the whole index (8 bytes per
// entry) but only the source rows whose target lies in the slice.
template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(kThreads) scatter_rows_direct_kernel(ScatterParams p) {
  using U = acc_t<T>;
  const T *__restrict__ src = static_cast<const T *>(p.src);
  if (p.clustered[0] != 0) return;                       // the run-combining kernel takes clustered indices
  if (p.binned && p.clustered[1] != 0) return;           // the tile kernel takes skewed ones
  U *target = static_cast<U *>(p.target);
  if (p.replicas > 1) target += (blockIdx.x % p.replicas) * (p.B * p.N * p.K);
  const int L = 1 << p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int col = threadIdx.x & (L - 1);
  const int64_t per_cta = kThreads >> p.l_log2;
  const int64_t M = p.B * p.E;
  // The grid is capped (see direct_grid): a CTA walks the entry blocks blockIdx.x, blockIdx.x + gridDim.x, ... so that
  // a launch whose index the flags hand to another kernel costs a few thousand CTAs, not one per 256 lanes of work.
  for (int64_t first = (int64_t)blockIdx.x * per_cta; first < M; first += (int64_t)gridDim.x * per_cta) {
    const int64_t entry = first + (threadIdx.x >> p.l_log2);
    if (entry >= M) continue;
    const int64_t b = entry / p.E, e = entry - b * p.E;
    const int64_t idx = p.index[b * p.sb + e * p.se];
    if (idx < 0 || idx >= p.N) continue;
    const T *srow = src + entry * p.K;
    U *trow = target + (b * p.N + idx) * p.K;
    for (int64_t c = col; c < Kv; c += L) apply_pack<OP, T, VEC>(trow + c * VEC, ld_stream<T, VEC>(srow + c * VEC));
    // one count per row of the index itself: a batch-broadcast index is counted for b == 0 only
    if (p.count != nullptr && col == 0 && (p.sb != 0 || b == 0)) atomicAdd(p.count + (p.sb ? b : 0) * p.N + idx, 1);
  }
}

constexpr int kRangeBatches = 4;  // 32-entry batches per group: a group is 128 consecutive entries
constexpr int kRangeGroups = 8;   // consecutive groups a warp walks through

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
  const int64_t first = ((int64_t)blockIdx.x * kWarps + warp) * (kCap * kRangeGroups);
  if (first >= M || *p.clustered != 0) return;  // warp-uniform

  // target rows (over all batches) of the 128 entries starting at `gbase`; -1: none / out of range
  auto load_targets = [&](int64_t gbase, int64_t (&t)[kRangeBatches]) {
#pragma unroll
    for (int q = 0; q < kRangeBatches; ++q) {
      const int64_t ent = gbase + q * 32 + lane;
      t[q] = -1;
      if (ent < M) {
        const int64_t b = (p.B == 1) ? 0 : ent / p.E;
        const int64_t idx = p.index[b * p.sb + (ent - b * p.E) * p.se];
        if (idx >= 0 && idx < p.N) t[q] = b * p.N + idx;
      }
    }
  };

  int64_t next[kRangeBatches];
  load_targets(first, next);
  for (int g = 0; g < kRangeGroups; ++g) {
    const int64_t gbase = first + (int64_t)g * kCap;
    if (gbase >= M) break;  // warp-uniform
    int64_t trow[kRangeBatches];
#pragma unroll
    for (int q = 0; q < kRangeBatches; ++q) trow[q] = next[q];
    // the next group's index loads stay in flight while this group's rows are moved: with few matches
    // per group (many slices) a warp would otherwise spend most of its time waiting for indices
    if (g + 1 < kRangeGroups && gbase + kCap < M) load_targets(gbase + kCap, next);

    int n = 0;
#pragma unroll
    for (int q = 0; q < kRangeBatches; ++q) {
      const bool match = trow[q] >= lo && trow[q] < hi;
      const unsigned mask = __ballot_sync(kFullMask, match);
      if (match) {
        const int r = n + __popc(mask & ((1u << lane) - 1u));
        s_ent[warp][r] = gbase + q * 32 + lane;
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
    __syncwarp();  // the list is rebuilt by the next group
  }
}

// ---- row kernel: index constant along k ---------------------------------------------------------
// A warp owns 128 consecutive entries.  It loads their 128 targets with four coalesced loads, keeps
// the ones that fall into the target-row range [lo, hi) of this pass and streams them 32/L rows per
// step, the rows arriving through a shared-memory ring eight steps deep.  If neighbouring entries share a target (an edge list
// sorted by destination, or any clustered index), a segmented scan over the step's lane groups plus a
// carry from step to step combines each run of equal targets, so that ONE update goes to global
// memory per run instead of one per entry; a list without such neighbours takes a direct path.
// (Sorting the warp's entries by target to also combine scattered duplicates was tried: the hardware
// match instruction used to detect duplicates costs more than it saves on duplicate-free indices.)
// With `replicas` > 1 (small outputs under heavy contention) warps spread their updates over several
// copies of the output; the finalize pass folds the copies.
constexpr int kBatches = 4;               // 32-entry batches per warp
constexpr int kWarpEntries = 32 * kBatches;

template <int OP, typename U> __device__ __forceinline__ U combine(U a, U b) {
  if (OP == kSum) return a + b;
  if (OP == kMul) return a * b;
  if (OP == kMin) return b < a ? b : a;
  return b > a ? b : a;
}

template <int OP, typename U, int VEC> __device__ __forceinline__ void apply_acc(U *addr, const U *v) {
  if constexpr (OP == kSum && std::is_same<U, float>::value && (VEC % 4 == 0)) {
#pragma unroll
    for (int i = 0; i < VEC; i += 4) red_add_v4(addr + i, v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) apply_one<OP, U>(addr + i, v[i]);
  }
}

template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(kThreads, 4) scatter_rows_runs_kernel(ScatterParams p, int64_t lo, int64_t hi, int replicas) {
  using U = acc_t<T>;
  constexpr int kWarps = kThreads / 32;
  constexpr int kRing = 8;                         // ring depth in steps (power of two)
  __shared__ int64_t s_key[kWarps][kWarpEntries];  // (target row << 7) | entry position within the warp's 128
  __shared__ Pack<T, VEC> s_ring[kWarps][kRing][32];
  const T *__restrict__ src = static_cast<const T *>(p.src);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = 1 << p.l_log2;
  const int col = lane & (L - 1);
  const int sub = lane >> p.l_log2;
  const int eps = 32 >> p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t M = p.B * p.E;
  const int64_t warp_id = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t base = warp_id * kWarpEntries;
  if (base >= M || *p.clustered == 0) return;  // warp-uniform; the direct kernels take unclustered indices
  U *target = static_cast<U *>(p.target) + (replicas > 1 ? (warp_id % replicas) * (p.B * p.N * p.K) : 0);

  // ---- targets of the warp's entries; all index loads are in flight before any is used
  int64_t trow[kBatches];
#pragma unroll
  for (int q = 0; q < kBatches; ++q) {
    const int64_t ent = base + q * 32 + lane;
    trow[q] = -1;
    if (ent < M) {
      const int64_t b = (p.B == 1) ? 0 : ent / p.E;
      const int64_t idx = p.index[b * p.sb + (ent - b * p.E) * p.se];
      if (idx >= 0 && idx < p.N) {
        const int64_t r = b * p.N + idx;
        if (r >= lo && r < hi) trow[q] = r;
      }
    }
  }
  // ---- compact the kept entries into shared memory, in entry order
  int n = 0;
#pragma unroll
  for (int q = 0; q < kBatches; ++q) {
    const bool keep = trow[q] >= 0;
    const unsigned mask = __ballot_sync(kFullMask, keep);
    if (keep) s_key[warp][n + __popc(mask & ((1u << lane) - 1u))] = (trow[q] << 7) | (int64_t)(q * 32 + lane);
    n += __popc(mask);
  }
  __syncwarp();
  if (n == 0) return;

  // do neighbouring entries of the list share a target?
  bool adjacent_equal = false;
  for (int m = lane; m + 1 < n; m += 32) adjacent_equal = adjacent_equal || (s_key[warp][m] >> 7) == (s_key[warp][m + 1] >> 7);
  const bool combine_runs = __any_sync(kFullMask, adjacent_equal);

  // Source rows travel through a per-warp shared-memory ring filled by per-lane cp.async copies, kRing
  // steps (kRing * 512 bytes) ahead of their use; a lane reads back only what it copied itself.
  const int nsteps = (n + eps - 1) / eps;
  const int64_t all_rows = p.B * p.N;
  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;
    auto issue = [&](int step, int slot) {
      const int m = step * eps + sub;
      if (step < nsteps && m < n && col_ok) {
        const int64_t ent = base + (s_key[warp][m] & 127);
        if (ent < M) async_copy_pack<T, VEC>(&s_ring[warp][slot][lane], src + ent * p.K + c * VEC);
      }
      async_commit();
    };
    auto flush = [&](int64_t key, const U *v, int cnt) {  // one update for an entry or a finished run
      if (key < 0 || key >= all_rows) return;  // cannot happen; keeps a logic error from becoming a fault
      if (col_ok) apply_acc<OP, U, VEC>(target + key * p.K + c * VEC, v);
      if (p.count != nullptr && c == 0) {
        const int64_t b = key / p.N;
        if (p.sb != 0 || b == 0) atomicAdd(p.count + (p.sb ? key : key - b * p.N), cnt);
      }
    };
#pragma unroll
    for (int j = 0; j < kRing; ++j) issue(j, j);

    int64_t carry_key = -1;
    int carry_cnt = 0;
    U carry[VEC];
#pragma unroll
    for (int k = 0; k < VEC; ++k) carry[k] = reduce_identity<T, OP>();

    int slot = 0;
    for (int step = 0; step < nsteps; ++step) {
      async_wait_all_but<kRing - 1>();
      const int m = step * eps + sub;
      const int64_t key = (m < n) ? (s_key[warp][m] >> 7) : -1;
      U val[VEC];
      {
        const Pack<T, VEC> v = s_ring[warp][slot][lane];
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          val[k] = (key >= 0 && col_ok) ? to_acc<T>(v.v[k]) : reduce_identity<T, OP>();
          if ((OP == kMin || OP == kMax) && is_nan(val[k])) val[k] = reduce_identity<T, OP>();
        }
      }
      issue(step + kRing, slot);
      slot = (slot + 1) & (kRing - 1);

      if (!combine_runs) {  // warp-uniform: every entry goes straight to global memory
        if (key >= 0) flush(key, val, 1);
        continue;
      }
      int cnt = key >= 0 ? 1 : 0;
      const int nvalid = (n - step * eps) < eps ? (n - step * eps) : eps;  // lane groups with an entry
      // the run carried over from the previous step continues in lane group 0, or is finished
      if (carry_key >= 0) {
        const int64_t first_key = __shfl_sync(kFullMask, (long long)key, 0);
        if (carry_key == first_key) {
          if (sub == 0) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) val[k] = combine<OP, U>(carry[k], val[k]);
            cnt += carry_cnt;
          }
        } else if (sub == 0) {
          flush(carry_key, carry, carry_cnt);
        }
        carry_key = -1;
      }
      // inclusive segmented scan over the lane groups: only ADJACENT groups with the same target
      // merge (`head` = a run starts in this group)
      const int64_t prev_key = __shfl_up_sync(kFullMask, (long long)key, L);
      int head = (sub == 0 || prev_key != key || key < 0) ? 1 : 0;
      for (int d = 1; d < eps; d <<= 1) {
        const int ohead = __shfl_up_sync(kFullMask, head, d << p.l_log2);
        const int ocnt = __shfl_up_sync(kFullMask, cnt, d << p.l_log2);
        const bool take = sub >= d && !head;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const U o = __shfl_up_sync(kFullMask, val[k], d << p.l_log2);
          if (take) val[k] = combine<OP, U>(o, val[k]);
        }
        if (take) {
          cnt += ocnt;
          head = ohead;
        }
      }
      // a lane group ends a run when its successor has another target; the last group's run may go on
      const int64_t next_key = __shfl_down_sync(kFullMask, (long long)key, L);
      const int last = nvalid - 1;
      if (key >= 0 && sub < last && next_key != key) flush(key, val, cnt);
      carry_key = __shfl_sync(kFullMask, (long long)key, last << p.l_log2);
      carry_cnt = __shfl_sync(kFullMask, cnt, last << p.l_log2);
#pragma unroll
      for (int k = 0; k < VEC; ++k) carry[k] = __shfl_sync(kFullMask, val[k], (last << p.l_log2) + col);
    }
    async_wait_all_but<0>();
    if (carry_key >= 0 && sub == 0) flush(carry_key, carry, carry_cnt);
  }
}

// ---- skewed index, small output: group a tile's entries by target inside the CTA, then walk runs ----------------
// An index where a few targets take most of the entries (a Zipf-like degree distribution) makes every per-entry
// update scheme pay for same-address atomics: in L2 for the direct kernels, in shared memory for a row cache (sixteen
// scalar shared-memory atomics per 64-byte entry kept the SMs busy 72 % of the time with DRAM at a quarter of its
// rate).  Here a CTA takes a tile of kBinTile consecutive entries and
//   1. bins them by a hash of the target row: one shared-memory counter update per ENTRY (not per value) gives the
//      entry's rank inside its bin,
//   2. scans the bin counts and writes (target, entry) pairs into bin order: entries of one target are now
//      neighbours, up to the few other targets that share its bin,
//   3. cuts that list into one contiguous piece per lane group (L lanes, one 16-byte pack of the row each); a lane
//      group walks its piece entry by entry, source rows arriving through a cp.async ring, and keeps accumulating in
//      registers while the target stays the same: ONE global update per run, no shuffle and no shared-memory atomic
//      on values.  (A first version combined the runs of a warp step with a segmented scan over the lane groups:
//      219 warp instructions per 8 entries, issue-bound at 1.49 ms on the Zipf workload.)
// A tile of 4096 Zipf(1.2) entries over 100,000 targets holds about 1200 distinct targets, so 3-4 times fewer updates
// reach L2 and the hottest target receives one update per lane group and tile instead of one per entry.  MIN/MAX keep
// value and entry id per run and settle both with one packed 64-bit atomic per value (see below), ties towards the
// smaller entry id.  The kernel runs only when the probe flags the index as skewed and not clustered.
constexpr int kBinTile = 4096;        // entries per CTA
constexpr int kBinBins = 4096;        // hash bins (power of two)
constexpr int kBinItems = kBinTile / kThreads;
constexpr int kBinRing = 8;           // cp.async ring depth in entries per lane group

template <typename T, int VEC> constexpr size_t binned_smem_bytes() {
  // (target, entry) pairs, then the ring; the bin counters live in the ring's space until the walk starts
  constexpr size_t ring = sizeof(Pack<T, VEC>) * kThreads * kBinRing;
  constexpr size_t cnt = sizeof(int) * (kBinBins + kThreads / 32);
  return sizeof(int2) * kBinTile + (ring > cnt ? ring : cnt);
}

template <int OP> __device__ __forceinline__ uint64_t pack_minmax(int32_t key, uint64_t slot);
template <int OP> __device__ __forceinline__ void atom_packed(uint64_t *addr, uint64_t v);

template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(kThreads, 3) scatter_rows_binned_kernel(ScatterParams p) {
  using U = acc_t<T>;
  constexpr int kWarps = kThreads / 32;
  constexpr bool kMinMax = (OP == kMin || OP == kMax);
  extern __shared__ __align__(16) unsigned char s_binned[];
  int2 *s_pair = reinterpret_cast<int2 *>(s_binned);            // x: target row over all batches, y: entry within the tile
  unsigned char *s_rest = s_binned + sizeof(int2) * kBinTile;
  auto s_ring = reinterpret_cast<Pack<T, VEC>(*)[kThreads]>(s_rest);   // [kBinRing][kThreads]
  int *s_cnt = reinterpret_cast<int *>(s_rest);                 // bins, until the walk starts
  int *s_warp_sum = s_cnt + kBinBins;
  const int64_t tile0 = (int64_t)blockIdx.x * kBinTile;
  // not skewed: the one-update-per-entry kernels; sums of a clustered index: the runs kernel
  if (p.clustered[1] == 0 || (!kMinMax && p.clustered[0] != 0)) return;
  const T *__restrict__ src = static_cast<const T *>(p.src);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t M = p.B * p.E;

  for (int i = tid; i < kBinBins; i += kThreads) s_cnt[i] = 0;
  __syncthreads();
  // The bin is a multiplicative hash of the target, salted with the tile: two hot targets that share a bin (their
  // entries then alternate inside it and every switch costs an update) do so in one tile out of kBinBins, not in all.
  const unsigned salt = (unsigned)blockIdx.x * 0x9e3779b9u;
  auto bin_of = [](int row, unsigned salt) -> unsigned { return (((unsigned)row ^ salt) * 2654435761u) >> 20; };
  // 1. targets of this thread's entries (coalesced loads, all in flight), rank inside the bin
  int row[kBinItems], rank[kBinItems];
#pragma unroll
  for (int j = 0; j < kBinItems; ++j) {
    const int64_t ent = tile0 + j * kThreads + tid;
    row[j] = -1;
    if (ent < M) {
      const int64_t b = (p.B == 1) ? 0 : ent / p.E;
      const int64_t idx = p.index[b * p.sb + (ent - b * p.E) * p.se];
      if (idx >= 0 && idx < p.N) row[j] = (int)(b * p.N + idx);   // B * N < 2^31 (checked by the launcher)
    }
  }
#pragma unroll
  for (int j = 0; j < kBinItems; ++j) {
    rank[j] = 0;
    if (row[j] >= 0) rank[j] = atomicAdd(&s_cnt[bin_of(row[j], salt)], 1);
  }
  __syncthreads();
  // 2. exclusive scan of the bin counts (kBinBins / kThreads consecutive bins per thread)
  {
    constexpr int kPer = kBinBins / kThreads;
    int c[kPer], v = 0;
#pragma unroll
    for (int i = 0; i < kPer; ++i) { c[i] = s_cnt[tid * kPer + i]; v += c[i]; }
    int incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(kFullMask, incl, off);
      if (lane >= off) incl += o;
    }
    if (lane == 31) s_warp_sum[warp] = incl;
    __syncthreads();
    int before = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) before += (w < warp) ? s_warp_sum[w] : 0;
    int run = before + incl - v;
#pragma unroll
    for (int i = 0; i < kPer; ++i) { s_cnt[tid * kPer + i] = run; run += c[i]; }
  }
  __syncthreads();
  int n = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) n += s_warp_sum[w];
#pragma unroll
  for (int j = 0; j < kBinItems; ++j)
    if (row[j] >= 0) s_pair[s_cnt[bin_of(row[j], salt)] + rank[j]] = make_int2(row[j], j * kThreads + tid);
  __syncthreads();  // the list is complete and the bin counters are dead: their space becomes the ring
  if (n == 0) return;

  // 3. every lane group walks its piece of the list
  const int L = 1 << p.l_log2;
  const int col = lane & (L - 1);
  const int groups = kThreads >> p.l_log2;
  const int gid = tid >> p.l_log2;
  const int64_t Kv = p.K / VEC;
  // an odd piece length keeps the groups' list reads on different shared-memory banks
  const int piece = ((n + groups - 1) / groups) | 1;
  const int start = gid * piece;
  const int my_n = start >= n ? 0 : (n - start < piece ? n - start : piece);
  const int2 *list = s_pair + start;
  const int64_t all_rows = p.B * p.N;
  U *target = nullptr;
  uint64_t *packed = nullptr;
  if constexpr (kMinMax) packed = reinterpret_cast<uint64_t *>(p.arg_out);
  else target = static_cast<U *>(p.target) + (p.replicas > 1 ? (blockIdx.x % p.replicas) * (p.B * p.N * p.K) : 0);
  constexpr uint32_t kNone = 0xffffffffu;

  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;
    auto issue = [&](int step, int slot) {
      if (step < my_n && col_ok) {
        const int64_t ent = tile0 + list[step].y;
        async_copy_pack<T, VEC>(&s_ring[slot][tid], src + ent * p.K + c * VEC);
      }
      async_commit();
    };
    U val[VEC];
    uint32_t arg[kMinMax ? VEC : 1];
    uint64_t seen[kMinMax ? VEC : 1];   // MIN/MAX: the target's packed words as they were when the run started
    int cur = -1, cnt = 0;
    auto restart = [&]() {
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        val[k] = reduce_identity<T, OP>();
        if (kMinMax) arg[k] = kNone;
      }
      cnt = 0;
      if constexpr (kMinMax) {
        // Fetched now, used when the run ends: the load has the whole run to arrive, so the walk never waits for L2.
        // The words only ever move towards the winner, so an old copy filters conservatively: an update it lets
        // through may turn out to be unnecessary, one it stops can never have won.
        if (cur >= 0 && cur < all_rows && col_ok) {
          const uint64_t *addr = packed + (int64_t)cur * p.K + c * VEC;
#pragma unroll
          for (int k = 0; k < VEC; ++k) seen[k] = *reinterpret_cast<const volatile uint64_t *>(addr + k);
        }
      }
    };
    auto flush = [&]() {  // one update for the finished run of target `cur`
      if (cur < 0 || cur >= all_rows || !col_ok) return;
      if constexpr (kMinMax) {
        uint64_t *addr = packed + (int64_t)cur * p.K + c * VEC;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          if (arg[k] == kNone) continue;
          const uint64_t w = pack_minmax<OP>(enc_key(val[k]), (uint64_t)arg[k] + 1);
          if (OP == kMax) {
            if (w > seen[k]) atomicMax(reinterpret_cast<unsigned long long *>(addr + k), (unsigned long long)w);
          } else {
            if (w < seen[k]) atomicMin(reinterpret_cast<unsigned long long *>(addr + k), (unsigned long long)w);
          }
        }
      } else {
        apply_acc<OP, U, VEC>(target + (int64_t)cur * p.K + c * VEC, val);
        if (p.count != nullptr && c == 0) {
          const int64_t b = cur / p.N;
          if (p.sb != 0 || b == 0) atomicAdd(p.count + (p.sb ? cur : cur - b * p.N), cnt);
        }
      }
    };
#pragma unroll
    for (int j = 0; j < kBinRing; ++j) issue(j, j);
    restart();
    int slot = 0;
    for (int step = 0; step < piece; ++step) {   // CTA-uniform trip count: one commit group per step and thread
      async_wait_all_but<kBinRing - 1>();
      if (step < my_n) {
        const int2 pr = list[step];
        if (pr.x != cur) {
          flush();
          cur = pr.x;
          restart();
        }
        const Pack<T, VEC> v = s_ring[slot][tid];
        cnt += 1;
        if (col_ok) {
          if constexpr (kMinMax) {
            const int64_t ent = tile0 + pr.y;
            const uint32_t e = (uint32_t)(p.B == 1 ? ent : ent % p.E);
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
              const U x = to_acc<T>(v.v[k]);
              if (is_nan(x)) continue;
              const bool better = (OP == kMin) ? (x < val[k]) : (x > val[k]);
              // the identity is a legal value: a first winner equal to it must still be recorded
              if (better || (x == val[k] && e < arg[k])) { val[k] = x; arg[k] = e; }
            }
          } else {
#pragma unroll
            for (int k = 0; k < VEC; ++k) val[k] = combine<OP, U>(val[k], to_acc<T>(v.v[k]));
          }
        }
      }
      issue(step + kBinRing, slot);
      slot = (slot + 1) & (kBinRing - 1);
    }
    async_wait_all_but<0>();
    flush();
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
// target[r][i] for r < replicas: copy 0 starts from `out` when accumulating into it, everything else
// from the identity (as an ordered key for MIN/MAX).
template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
scatter_init_kernel(const T *out, acc_t<T> *target, int64_t total, int fresh, int replicas) {
  using U = acc_t<T>;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total * replicas) return;
  const U v = (fresh || i >= total) ? reduce_identity<T, OP>() : to_acc<T>(out[i]);
  if (OP == kMin || OP == kMax) reinterpret_cast<key_t<U> *>(target)[i] = enc_key(v);
  else target[i] = v;
}

// floats divide; integers round toward -inf (torch_scatter/scatter.py:65, div_ with rounding_mode='floor')
template <typename T> __device__ __forceinline__ T mean_div(T v, int32_t c) {
  if constexpr (std::is_integral<T>::value) {
    using W = typename std::conditional<sizeof(T) == 8, int64_t, int32_t>::type;
    const W a = (W)v, b = (W)c;
    W q = a / b;
    if ((a % b != 0) && (a < 0)) --q;
    return (T)q;
  } else {
    return v / (T)c;
  }
}
template <> __device__ __forceinline__ __half mean_div<__half>(__half v, int32_t c) {
  return __float2half_rn(__half2float(v) / __half2float(__int2half_rn(c)));
}
template <> __device__ __forceinline__ __nv_bfloat16 mean_div<__nv_bfloat16>(__nv_bfloat16 v, int32_t c) {
  return __float2bfloat16_rn(__bfloat162float(v) / __bfloat162float(__int2bfloat16_rn(c)));
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
scatter_finalize_kernel(T *out, const acc_t<T> *target, const int32_t *count, int64_t total, int64_t N, int64_t K,
                        int fresh, int count_b, int count_k, int replicas) {
  using U = acc_t<T>;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  U v;
  if (OP == kMin || OP == kMax) {
    const key_t<U> *keys = reinterpret_cast<const key_t<U> *>(target);
    key_t<U> best = keys[i];
    for (int r = 1; r < replicas; ++r) {
      const key_t<U> o = keys[(int64_t)r * total + i];
      if ((OP == kMin) ? (o < best) : (o > best)) best = o;
    }
    v = dec_key<U>(best);
    if (fresh && v == reduce_identity<T, OP>()) v = (U)0;
  } else {
    v = target[i];
    for (int r = 1; r < replicas; ++r) v = combine<OP, U>(v, target[(int64_t)r * total + i]);
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

// ---- MIN / MAX with arg in ONE pass for 4-byte accumulation types --------------------------------
// For fp32 / int32 values (fp16 / bf16 compare as fp32) the value's order-preserving 32-bit key and the
// element's position are packed into one 64-bit word, so a single native 64-bit atomicMax / atomicMin
// settles value and arg together.  The low word holds the position plus one ("slot"; 0 = no element):
// MAX keeps (key << 32 | ~slot), MIN keeps (key << 32 | slot).  On equal values the smaller slot wins,
// and slot 0 - the value `out` held before the call, or the identity - beats every element: the rule of
// the CPU loop, whose strict comparison keeps what it already has (csrc/cpu/reducer.h:63-67), so a
// source value equal to the one already in `out` leaves the arg at "none".  The int64 arg_out tensor
// itself holds the packed words until the finalize kernel splits them, so the source is read once and
// no extra memory is needed.  Requires E < 2^32 - 1; 8-byte types keep the two-pass scheme further down.
constexpr uint64_t kNoPos = 0xffffffffull;

template <int OP> __device__ __forceinline__ uint64_t pack_minmax(int32_t key, uint64_t slot) {
  const uint64_t ukey = (uint32_t)key ^ 0x80000000u;  // signed order -> unsigned order
  return (ukey << 32) | (OP == kMax ? (kNoPos - slot) : slot);
}
template <int OP> __device__ __forceinline__ void atom_packed(uint64_t *addr, uint64_t v) {
  const uint64_t cur = *reinterpret_cast<volatile uint64_t *>(addr);  // filters updates that cannot win
  if (OP == kMax) {
    if (v > cur) atomicMax(reinterpret_cast<unsigned long long *>(addr), (unsigned long long)v);
  } else {
    if (v < cur) atomicMin(reinterpret_cast<unsigned long long *>(addr), (unsigned long long)v);
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) packed_init_kernel(const T *out, uint64_t *packed, int64_t total, int fresh) {
  using U = acc_t<T>;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const U v = fresh ? reduce_identity<T, OP>() : to_acc<T>(out[i]);
  packed[i] = pack_minmax<OP>(enc_key(v), 0);  // slot 0: no element
}

// One element: NaN never wins; a value equal to the identity (fresh output) or to the value already in
// `out` never wins either, because slot 0 beats its slot on the equal key.
template <typename T, int OP>
__device__ __forceinline__ void packed_update(uint64_t *addr, T x, int64_t e, int fresh) {
  using U = acc_t<T>;
  (void)fresh;
  const U v = to_acc<T>(x);
  if (is_nan(v)) return;
  atom_packed<OP>(addr, pack_minmax<OP>(enc_key(v), (uint64_t)e + 1));
}

template <typename T, int OP, int VEC>
__global__ void __launch_bounds__(kThreads) packed_rows_kernel(ScatterParams p) {
  if (p.binned && p.clustered[1] != 0) return;  // a skewed index: scatter_rows_binned_kernel takes it
  const T *__restrict__ src = static_cast<const T *>(p.src);
  uint64_t *packed = reinterpret_cast<uint64_t *>(p.arg_out);
  const int L = 1 << p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int col = threadIdx.x & (L - 1);
  const int64_t per_cta = kThreads >> p.l_log2;
  const int64_t M = p.B * p.E;
  for (int64_t first = (int64_t)blockIdx.x * per_cta; first < M; first += (int64_t)gridDim.x * per_cta) {  // capped grid
    const int64_t entry = first + (threadIdx.x >> p.l_log2);
    if (entry >= M) continue;
    const int64_t b = entry / p.E, e = entry - b * p.E;
    const int64_t idx = p.index[b * p.sb + e * p.se];
    if (idx < 0 || idx >= p.N) continue;
    const int64_t obase = (b * p.N + idx) * p.K;
    for (int64_t c = col; c < Kv; c += L) {
      const Pack<T, VEC> v = ld_stream<T, VEC>(src + entry * p.K + c * VEC);
#pragma unroll
      for (int i = 0; i < VEC; ++i) packed_update<T, OP>(packed + obase + c * VEC + i, v.v[i], e, p.fresh);
    }
  }
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads) packed_elems_kernel(ScatterParams p) {
  const T *__restrict__ src = static_cast<const T *>(p.src);
  uint64_t *packed = reinterpret_cast<uint64_t *>(p.arg_out);
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= p.B * p.E * p.K) return;
  const int64_t k = i % p.K, be = i / p.K;
  const int64_t b = be / p.E, e = be - b * p.E;
  const int64_t idx = p.index[b * p.sb + e * p.se + k * p.sk];
  if (idx < 0 || idx >= p.N) return;
  packed_update<T, OP>(packed + (b * p.N + idx) * p.K + k, src[i], e, p.fresh);
}

template <typename T, int OP>
__global__ void __launch_bounds__(kThreads)
packed_finalize_kernel(T *out, int64_t *arg_out, int64_t total, int64_t E, int fresh) {
  using U = acc_t<T>;
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const uint64_t w = reinterpret_cast<const uint64_t *>(arg_out)[i];
  const int32_t key = (int32_t)((uint32_t)(w >> 32) ^ 0x80000000u);
  U v = dec_key<U>(key);
  uint64_t slot = w & kNoPos;
  if (OP == kMax) slot = kNoPos - slot;
  if (slot == 0) {  // no element won: a fresh output's identity is masked to 0, a seeded one keeps its value
    if (fresh) out[i] = from_acc<T>((U)0);
    arg_out[i] = E;
    return;
  }
  out[i] = from_acc<T>(v);
  arg_out[i] = (int64_t)slot - 1;
}

// ---- arg pass ----------------------------------------------------------------------------------
__device__ __forceinline__ void arg_min(int64_t *a, int64_t e) {
  if (e < *reinterpret_cast<volatile int64_t *>(a)) atomicMin(reinterpret_cast<long long *>(a), (long long)e);
}

// Seeded MIN/MAX (the caller passed `out`): the CPU loop's strict comparison lets the value already in `out` win a
// tie and leaves its arg at "none" (csrc/cpu/reducer.h:63-67).  The seeds are kept in arg_out (as raw bits) while
// the values are reduced; afterwards every target whose result equals its seed is closed to the arg pass with a
// marker below every position, and a last pass turns the markers into "none".
constexpr int64_t kSeedWon = -1;

template <typename T>
__global__ void __launch_bounds__(kThreads) seed_stash_kernel(const T *out, int64_t *arg_out, int64_t total) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  int64_t bits = 0;
  const T v = out[i];
  memcpy(&bits, &v, sizeof(T));
  arg_out[i] = bits;
}
template <typename T>
__global__ void __launch_bounds__(kThreads) seed_compare_kernel(const T *out, int64_t *arg_out, int64_t total, int64_t E) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const int64_t bits = arg_out[i];
  T seed;
  memcpy(&seed, &bits, sizeof(T));
  arg_out[i] = (to_acc<T>(out[i]) == to_acc<T>(seed)) ? kSeedWon : E;
}
__global__ void __launch_bounds__(kThreads) seed_close_kernel(int64_t *arg_out, int64_t total, int64_t E) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i < total && arg_out[i] == kSeedWon) arg_out[i] = E;
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
  if (idx < 0 || idx >= p.N) {  // the forward dropped this entry: its gradient is zero
    Pack<T, VEC> zero;
#pragma unroll
    for (int i = 0; i < VEC; ++i) zero.v[i] = from_acc<T>((acc_t<T>)0);
    for (int64_t c = col; c < Kv; c += L) st_stream<T, VEC>(gi + entry * p.K + c * VEC, zero);
    return;
  }
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
  if (idx < 0 || idx >= p.N) { gi[i] = from_acc<T>((acc_t<T>)0); return; }
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

// Grid of the one-update-per-entry row kernels, which walk the entries with a grid stride: enough CTAs to fill the
// device many times over (dynamic balance), few enough that a launch which turns out to have nothing to do is cheap.
inline unsigned direct_grid(int64_t entries, int l_log2) {
  const int64_t per_cta = kThreads >> l_log2;
  const int64_t need = (entries + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)sm_count() * 64;
  return (unsigned)(need < 1 ? 1 : (need < cap ? need : cap));
}

inline bool grid_for(int64_t threads, unsigned *blocks) {
  const int64_t nb = (threads + kThreads - 1) / kThreads;
  if (nb > 2147483647LL) return false;
  *blocks = (unsigned)nb;
  return true;
}

// Copies of the output that warps spread their updates over.  Only small outputs are replicated
// (the copies stay L2-resident); they are the ones where many entries pile onto few addresses.
inline int replicas_for(int64_t target_bytes) {
  if (target_bytes <= 0 || target_bytes > (8ll << 20)) return 1;
  const int64_t r = (64ll << 20) / target_bytes;
  return (int)(r > 16 ? 16 : (r < 1 ? 1 : r));
}

template <typename T, int OP>
int run_scatter(ScatterParams p, int reduce, void *workspace, cudaStream_t stream) {
  using U = acc_t<T>;
  constexpr bool k16 = !std::is_same<T, acc_t<T>>::value;   // accumulates in a wider workspace: fp16 / bf16 -> fp32, narrow ints -> int32
  constexpr bool kMinMax = (OP == kMin || OP == kMax);
  constexpr bool kKeyed = kMinMax && !std::is_same<key_t<U>, U>::value;
  constexpr int kFull = full_vec<T>();
  const int64_t total = p.B * p.N * p.K;
  const bool mean = reduce == TSB_MEAN;
  const bool rows = p.sk == 0;
  unsigned blocks = 0;

  // Replicated accumulation: small output, index constant along the features, enough entries to matter.
  int replicas = replicas_for(total * (int64_t)sizeof(U));
  if (!rows || p.B * p.E < (1 << 16)) replicas = 1;
  const bool small_output = replicas > 1;   // "small" as in: could be contended, several copies would fit in L2
  // fp32 accumulators: a skewed index is taken by the tile kernel that walks runs, which needs no copies, and for any
  // other index the copies only cost their initialisation and the fold (1 M entries into 65,536 rows x 32 floats:
  // 0.136 ms with seven copies, 0.082 ms without)
  if (OP == kSum && std::is_same<U, float>::value) replicas = 1;
  replicas = (int)env_bytes("TSB_SCATTER_REPLICAS", replicas);  // test hook
  if (replicas > replicas_for(total * (int64_t)sizeof(U))) replicas = replicas_for(total * (int64_t)sizeof(U));
  int *flag = static_cast<int *>(workspace);                       // first 256 bytes: the probe's verdict
  void *scratch = static_cast<unsigned char *>(workspace) + 256;  // then accumulators / replicas
  p.target = (k16 || replicas > 1) ? scratch : p.out;
  p.replicas = replicas;
  p.clustered = flag;

  // An output larger than L2 is accumulated slice by slice when the index is constant along the
  // features and a source row is big enough to pay for re-reading the index once per slice.
  const int64_t slice_bytes = env_bytes("TSB_SCATTER_SLICE_BYTES", 128ll << 20);  // test / tuning hook
  const int64_t target_row_bytes = p.K * (int64_t)sizeof(U);
  int64_t slice_rows = target_row_bytes > 0 ? slice_bytes / target_row_bytes : 0;
  if (slice_rows < 1) slice_rows = 1;
  const bool sliced = OP == kSum && rows && replicas == 1 && p.E > 0 && p.B * p.N > slice_rows + slice_rows / 2 &&
                      p.K * (int64_t)sizeof(T) >= 128;

  // MIN / MAX on 4-byte accumulation types: value and arg in one pass through packed 64-bit atomics
  if constexpr (kMinMax && sizeof(U) == 4) {
    // Small outputs (the ones other types replicate): the tile kernel, which walks runs of equal targets with one
    // packed update per run when the probe calls the index skewed and sends one packed update per element otherwise
    // (1 M entries into 65,536 rows x 32: 0.17 ms against 0.31 ms for the replicated two-pass scheme below; 33.5 M
    // Zipf entries into 100,000 rows x 16: 2.65 ms before).  TSB_SCATTER_CACHED=0 (test hook) keeps the two-pass scheme.
    const char *skew_env = std::getenv("TSB_SCATTER_CACHED");  // test hook: "0" / "1" dictate the skew verdict
    const int forced_skew_mm = (skew_env != nullptr && (*skew_env == '0' || *skew_env == '1')) ? (*skew_env - '0') : -1;
    const bool vec_rows = rows && (p.K % kFull == 0) && aligned16(p.src);
    const bool binned = replicas > 1 && forced_skew_mm != 0 && vec_rows && p.B * p.N < (1ll << 31) && p.E > 0;
    if (p.E < 0xfffffffell && (replicas == 1 || binned)) {
      if (total == 0) return TSB_OK;
      if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
      packed_init_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(static_cast<const T *>(p.out),
                                                                  reinterpret_cast<uint64_t *>(p.arg_out), total, p.fresh);
      if (p.E > 0) {
        const bool vec_ok = vec_rows;
        const int64_t Kv = p.K / (vec_ok ? kFull : 1);
        p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
        p.clustered = nullptr;
        p.binned = 0;
        if (binned) {
          p.binned = 1;
          const int64_t bin_tiles = (p.B * p.E + kBinTile - 1) / kBinTile;
          if (bin_tiles > 2147483647LL) return TSB_ERR_TOO_LARGE;
          p.clustered = flag;
          scatter_probe_kernel<<<1, kThreads, 0, stream>>>(p, flag, -1, forced_skew_mm);
          constexpr size_t smem = binned_smem_bytes<T, kFull>();
          static std::atomic<bool> allowed[64];  // per device; setting the attribute twice is harmless
          int dev = 0;
          if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !allowed[dev]) {
            if (cudaFuncSetAttribute(scatter_rows_binned_kernel<T, OP, kFull>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem) != cudaSuccess)
              return TSB_ERR_LAUNCH;
            allowed[dev] = true;
          }
          scatter_rows_binned_kernel<T, OP, kFull><<<(unsigned)bin_tiles, kThreads, smem, stream>>>(p);
        }
        if (rows) {
          blocks = direct_grid(p.B * p.E, p.l_log2);
          if (vec_ok) packed_rows_kernel<T, OP, kFull><<<blocks, kThreads, 0, stream>>>(p);
          else packed_rows_kernel<T, OP, 1><<<blocks, kThreads, 0, stream>>>(p);
        } else {
          if (!grid_for(p.B * p.E * p.K, &blocks)) return TSB_ERR_TOO_LARGE;
          packed_elems_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(p);
        }
      }
      if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
      packed_finalize_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(static_cast<T *>(p.out), p.arg_out, total, p.E, p.fresh);
      return launch_status();
    }
  }

  // 1. bring the target to its starting state
  const bool seeded_minmax = kMinMax && !p.fresh && total > 0;
  if (seeded_minmax) {
    if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
    seed_stash_kernel<T><<<blocks, kThreads, 0, stream>>>(static_cast<const T *>(p.out), p.arg_out, total);
  }
  if (total > 0) {
    const bool need_init = k16 || kKeyed || p.fresh || replicas > 1;
    if (need_init) {
      if (!k16 && OP == kSum && replicas == 1) {
        // sliced passes zero each slice right before accumulating into it (it then never leaves L2)
        if (!sliced && cudaMemsetAsync(p.target, 0, (size_t)total * sizeof(U), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
      } else {
        if (!grid_for(total * replicas, &blocks)) return TSB_ERR_TOO_LARGE;
        scatter_init_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(static_cast<const T *>(p.out),
                                                                     static_cast<U *>(p.target), total, p.fresh, replicas);
      }
    }
    if (mean) {
      const int64_t cn = (p.sb ? p.B : 1) * p.N * (p.sk ? p.K : 1);
      if (cudaMemsetAsync(p.count, 0, (size_t)cn * sizeof(int32_t), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
    }
  }

  // 2. the accumulation pass(es)
  const bool vec_ok = rows && (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.target) && aligned16(p.out);
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);
  p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  if (total > 0 && p.E > 0) {
    if (rows) {
      // A probe over a few windows of the index sets a device flag; the direct kernels and the
      // run-combining kernel are both launched and the one the flag does not select exits at once.
      const char *force_env = std::getenv("TSB_SCATTER_CLUSTERED");  // test hook: "0" / "1"
      const int forced = (force_env != nullptr && (*force_env == '0' || *force_env == '1')) ? (*force_env - '0') : -1;
      const char *cache_env = std::getenv("TSB_SCATTER_CACHED");  // test / tuning hook: "0" / "1" dictate the skew verdict
      const int forced_skew = (cache_env != nullptr && (*cache_env == '0' || *cache_env == '1')) ? (*cache_env - '0') : -1;
      scatter_probe_kernel<<<1, kThreads, 0, stream>>>(p, flag, forced, forced_skew);
      unsigned blocks_direct = 0, blocks_batched = 0, blocks_range = 0;
      if (!grid_for((p.B * p.E + kRangeBatches * kRangeGroups - 1) / (kRangeBatches * kRangeGroups), &blocks_range)) return TSB_ERR_TOO_LARGE;  // 1024 entries per warp
      blocks_direct = direct_grid(p.B * p.E, p.l_log2);                                                      // L lanes per entry, grid stride
      if (!grid_for((p.B * p.E + kBatches - 1) / kBatches, &blocks_batched)) return TSB_ERR_TOO_LARGE;  // 128 entries per warp
      const bool zero_slices = sliced && !k16 && p.fresh;
      const int64_t all_rows = p.B * p.N;
      const int64_t step = sliced ? slice_rows : all_rows;
      for (int64_t lo = 0; lo < all_rows; lo += step) {
        const int64_t hi = lo + step < all_rows ? lo + step : all_rows;
        if (zero_slices && cudaMemsetAsync(static_cast<U *>(p.target) + lo * p.K, 0,
                                           (size_t)((hi - lo) * p.K) * sizeof(U), stream) != cudaSuccess)
          return TSB_ERR_LAUNCH;
        if constexpr (OP == kSum && std::is_same<U, float>::value) {
          // small (= possibly contended) output: a skewed index goes through scatter_rows_binned_kernel, any other
          // through the kernels below, which then leave skewed indices alone (device-side choice, ScatterParams::binned)
          const bool want = forced_skew == 1 || (forced_skew != 0 && small_output);
          const int64_t bin_tiles = (p.B * p.E + kBinTile - 1) / kBinTile;
          if (want && vec_ok && !sliced && all_rows < (1ll << 31) && bin_tiles <= 2147483647LL) {
            constexpr size_t smem = binned_smem_bytes<T, kFull>();
            static std::atomic<bool> allowed[64];  // per device; setting the attribute twice is harmless
            int dev = 0;
            if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && !allowed[dev]) {
              if (cudaFuncSetAttribute(scatter_rows_binned_kernel<T, kSum, kFull>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem) != cudaSuccess)
                return TSB_ERR_LAUNCH;
              allowed[dev] = true;
            }
            p.binned = 1;
            scatter_rows_binned_kernel<T, kSum, kFull><<<(unsigned)bin_tiles, kThreads, smem, stream>>>(p);
          }
        }
        if (vec_ok) {
          bool ranged = false;
          if constexpr (OP == kSum) {  // only sums are ever sliced
            if (sliced) { scatter_rows_range_kernel<T, OP, kFull><<<blocks_range, kThreads, 0, stream>>>(p, lo, hi); ranged = true; }
          }
          if (!ranged) scatter_rows_direct_kernel<T, OP, kFull><<<blocks_direct, kThreads, 0, stream>>>(p);
          scatter_rows_runs_kernel<T, OP, kFull><<<blocks_batched, kThreads, 0, stream>>>(p, lo, hi, replicas);
        } else {
          bool ranged = false;
          if constexpr (OP == kSum) {
            if (sliced) { scatter_rows_range_kernel<T, OP, 1><<<blocks_range, kThreads, 0, stream>>>(p, lo, hi); ranged = true; }
          }
          if (!ranged) scatter_rows_direct_kernel<T, OP, 1><<<blocks_direct, kThreads, 0, stream>>>(p);
          scatter_rows_runs_kernel<T, OP, 1><<<blocks_batched, kThreads, 0, stream>>>(p, lo, hi, replicas);
        }
      }
    } else {
      if (!grid_for(p.B * p.E * p.K, &blocks)) return TSB_ERR_TOO_LARGE;
      scatter_elems_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(p);
    }
  }

  // 3. finalize: fold replicas, decode keys, mask untouched MIN/MAX slots, round fp32 accumulators, divide for MEAN
  if (total > 0 && (k16 || kMinMax || mean || replicas > 1)) {
    if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
    scatter_finalize_kernel<T, OP><<<blocks, kThreads, 0, stream>>>(
        static_cast<T *>(p.out), static_cast<const U *>(p.target), mean ? p.count : nullptr, total, p.N, p.K,
        p.fresh, p.sb != 0, p.sk != 0, replicas);
  }

  // 4. arg pass
  if (kMinMax && total > 0) {
    if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
    if (seeded_minmax) seed_compare_kernel<T><<<blocks, kThreads, 0, stream>>>(static_cast<const T *>(p.out), p.arg_out, total, p.E);
    else fill_i64_kernel<<<blocks, kThreads, 0, stream>>>(p.arg_out, total, p.E);
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
    if (seeded_minmax) {
      if (!grid_for(total, &blocks)) return TSB_ERR_TOO_LARGE;
      seed_close_kernel<<<blocks, kThreads, 0, stream>>>(p.arg_out, total, p.E);
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

namespace {
// The atomics-free path pays about 12 bytes of scratch traffic per entry to group the entries by row;
// it wins once the accumulation target no longer stays in L2 (the reductions then re-fetch output
// lines or re-read the index per slice), for MIN/MAX earlier because value+arg targets are twice as big.
bool prefer_grouped(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  const int64_t acc = (int64_t)tsb::dtype_acc_bytes(dtype);
  const int64_t elem = (int64_t)tsb::dtype_elem_bytes(dtype);
  const int64_t target_bytes = B * N * K * acc;
  // products have no native atomic (compare-and-swap loops): grouping wins as soon as there is work to speak of
  if (reduce == TSB_MUL) return B * E * K >= (1ll << 18) && E < (1ll << 30);
  if (K * elem < 32) return false;
  const bool minmax = reduce == TSB_MIN || reduce == TSB_MAX;
  return target_bytes > (minmax ? (48ll << 20) : (192ll << 20));
}
int grouped_override() {  // test / tuning hook: "0" never, "1" whenever the shapes allow it
  const char *v = std::getenv("TSB_SCATTER_GROUPED");
  return (v != nullptr && (*v == '0' || *v == '1')) ? (*v - '0') : -1;
}
}  // namespace

extern "C" size_t tsb_scatter_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  if (B < 0 || E < 0 || N < 0 || K < 0) return 0;
  const bool k16 = tsb::dtype_accumulates_wider(dtype);
  const size_t acc = tsb::dtype_acc_bytes(dtype);
  const size_t target = (size_t)B * (size_t)N * (size_t)K * acc;
  const int replicas = tsb::replicas_for((int64_t)target);
  size_t scratch = (k16 || replicas > 1) ? target * (size_t)replicas : 0;
  // the index strides are not known here: cover both paths
  const int forced = grouped_override();
  if (forced == 1 || (forced != 0 && prefer_grouped(B, E, K, N, dtype, reduce))) {
    const size_t grouped = tsb::scatter_grouped_workspace_bytes(B, E, K, N, dtype, reduce);
    if (grouped > scratch) scratch = grouped;
  }
  return 256 + scratch;  // 256: the index probe's flag
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
  const size_t need = tsb_scatter_workspace_bytes(B, E, K, N, dtype, reduce);
  if (workspace == nullptr || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return TSB_ERR_WORKSPACE;
  {
    const int forced = grouped_override();
    if ((forced == 1 || (forced != 0 && prefer_grouped(B, E, K, N, dtype, reduce))) &&
        scatter_grouped_possible(B, E, K, N, idx_stride_b, idx_stride_e, idx_stride_k, dtype, reduce))
      return run_scatter_grouped(src, index, out, arg_out, count_out, B, E, K, N, dtype, reduce, out_seeded,
                                 static_cast<unsigned char *>(workspace) + 256, workspace_bytes - 256, stream);
  }
  ScatterParams p;
  p.src = src; p.index = index; p.out = out;
  p.target = out;  // run_scatter redirects it to the workspace where that is used
  p.arg_out = arg_out;
  p.count = reduce == TSB_MEAN ? count_out : nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.sb = idx_stride_b; p.se = idx_stride_e; p.sk = idx_stride_k;
  p.l_log2 = 0;
  p.fresh = out_seeded ? 0 : 1;
  p.replicas = 1;
  p.binned = 0;
  p.clustered = nullptr;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    switch (reduce) {
      case TSB_SUM:
      case TSB_MEAN: return run_scatter<scalar_t, kSum>(p, reduce, workspace, stream);
      case TSB_MIN: return run_scatter<scalar_t, kMin>(p, reduce, workspace, stream);
      case TSB_MAX: return run_scatter<scalar_t, kMax>(p, reduce, workspace, stream);
      case TSB_MUL: return run_scatter<scalar_t, kMul>(p, reduce, workspace, stream);
      default: return TSB_ERR_REDUCE;
    }
  });
}

namespace tsb {
namespace {
// Sums of one edge shard into the target rows [row_lo, row_hi) of a partial held in accumulation
// precision: zero the slice, then the probe and the row kernels restricted to the slice.
template <typename T>
int run_scatter_sum_slice(ScatterParams p, int64_t row_lo, int64_t row_hi, int *flag, cudaStream_t stream) {
  using U = acc_t<T>;
  constexpr int kFull = full_vec<T>();
  if (row_hi <= row_lo || p.K == 0) return TSB_OK;
  if (cudaMemsetAsync(static_cast<U *>(p.target) + row_lo * p.K, 0, (size_t)((row_hi - row_lo) * p.K) * sizeof(U),
                      stream) != cudaSuccess)
    return TSB_ERR_LAUNCH;
  if (p.E == 0) return TSB_OK;
  const bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.target);
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);
  p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  p.clustered = flag;
  unsigned blocks = 0, blocks_range = 0;
  if (!grid_for((p.E + kBatches - 1) / kBatches, &blocks)) return TSB_ERR_TOO_LARGE;
  if (!grid_for((p.E + kRangeBatches * kRangeGroups - 1) / (kRangeBatches * kRangeGroups), &blocks_range)) return TSB_ERR_TOO_LARGE;
  scatter_probe_kernel<<<1, kThreads, 0, stream>>>(p, flag, -1, -1);
  if (vec_ok) {
    scatter_rows_range_kernel<T, kSum, kFull><<<blocks_range, kThreads, 0, stream>>>(p, row_lo, row_hi);
    scatter_rows_runs_kernel<T, kSum, kFull><<<blocks, kThreads, 0, stream>>>(p, row_lo, row_hi, 1);
  } else {
    scatter_rows_range_kernel<T, kSum, 1><<<blocks_range, kThreads, 0, stream>>>(p, row_lo, row_hi);
    scatter_rows_runs_kernel<T, kSum, 1><<<blocks, kThreads, 0, stream>>>(p, row_lo, row_hi, 1);
  }
  return launch_status();
}
}  // namespace
}  // namespace tsb

extern "C" int tsb_scatter_sum_slice(const void *src, const int64_t *index, void *partial, int64_t E, int64_t K,
                                     int64_t N, int dtype, int64_t row_lo, int64_t row_hi, void *workspace,
                                     size_t workspace_bytes, tsb_stream_t stream) {
  using namespace tsb;
  if (E < 0 || K < 0 || N < 0 || row_lo < 0 || row_hi > N) return TSB_ERR_ARG;
  if (N * K == 0 || row_hi <= row_lo) return TSB_OK;
  if (partial == nullptr || (E > 0 && (src == nullptr || index == nullptr))) return TSB_ERR_ARG;
  if (workspace == nullptr || workspace_bytes < 256 || (reinterpret_cast<uintptr_t>(workspace) & 255u)) return TSB_ERR_WORKSPACE;
  ScatterParams p;
  p.src = src; p.index = index; p.out = partial; p.target = partial;
  p.arg_out = nullptr; p.count = nullptr;
  p.B = 1; p.E = E; p.K = K; p.N = N;
  p.sb = 0; p.se = 1; p.sk = 0;
  p.l_log2 = 0; p.fresh = 1; p.replicas = 1; p.binned = 0; p.clustered = nullptr;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    return run_scatter_sum_slice<scalar_t>(p, row_lo, row_hi, static_cast<int *>(workspace),
                                           reinterpret_cast<cudaStream_t>(stream));
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
  // Rows named by a unit-stride index, no divide: the warp-batched streaming copy of tsb_gather_coo
  // (it does not need the index to be sorted) is the fastest kernel for it.
  if (count == nullptr && idx_stride_k == 0 && (idx_stride_e == 1 || E == 1) && (B == 1 || idx_stride_b == 0 || idx_stride_b == E))
    return tsb_gather_coo(grad_out, index, grad_in, nullptr, B, E, K, N, B == 1 ? 0 : idx_stride_b, dtype, stream);
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    return run_scatter_backward<scalar_t>(p, reinterpret_cast<cudaStream_t>(stream));
  });
}

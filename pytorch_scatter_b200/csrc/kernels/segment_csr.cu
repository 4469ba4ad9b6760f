// segment_csr for sm_100a: row-pointer segmented reduction of src [B,E,K] into out [B,N,K].
//
// The rows of a CSR matrix are contiguous in src, so a run of consecutive rows is one contiguous
// byte stream.  Each warp owns a chunk of up to 31 consecutive rows and STREAMS their entries in
// order, independent of where the row boundaries fall:
//   * an entry (K contiguous elements) is covered by L lanes holding one 16-byte pack each, so a warp
//     consumes 32/L entries (512 contiguous bytes for 16-byte packs) per step;
//   * loads run D steps ahead of consumption through a register ring, so every warp keeps D*512
//     bytes in flight no matter how short its rows are;
//   * the row boundaries of the chunk live in registers (lane j holds indptr[first_row + j]); all
//     control flow that depends on them is warp-uniform.  When one or more rows end inside a step,
//     the lanes whose entry belongs to the closing row contribute to a shuffle butterfly and the
//     row is written; the remaining lanes start the next row.
// Rows of at least `long_len` entries (128 KiB of source) are cut out of the stream and reduced by a
// second kernel whose 1024-thread CTAs scan the row pointers for them and put all 32 warps on one
// row at a time, partials combined through shared memory in a fixed order.
// Nothing is atomic: results depend only on the shapes, never on scheduling.
//
// Replaces segment_csr_kernel / segment_csr_broadcast_kernel of the upstream project
// (csrc/cuda/segment_csr_cuda.cu:15-95), which walk each row with a single thread per feature.
#include <cstdlib>

#include "csr_reduce.cuh"

namespace tsb {

namespace {

constexpr int kMaxRowsPerWarp = 31;  // lane j holds boundary j, so rows+1 <= 32

struct CsrGeom {
  int l_log2;         // lanes per entry
  int rows_per_warp;  // consecutive rows streamed by one warp (<= 31)
  int64_t long_len;   // rows at least this long are reduced by the whole CTA
};

template <typename T, int REDUCE, int VEC> struct RowAcc {
  using A = acc_t<T>;
  static constexpr bool kArg = (REDUCE == kMin || REDUCE == kMax);
  A val[VEC];
  int64_t arg[kArg ? VEC : 1];

  __device__ __forceinline__ void init(int64_t sentinel) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      val[i] = reduce_identity<T, REDUCE>();
      if (kArg) arg[i] = sentinel;
    }
  }
  // Entries arrive in increasing e within a lane, so strict comparisons keep the first winner
  // (csrc/cpu/reducer.h:63-67).
  __device__ __forceinline__ void update(const Pack<T, VEC> &v, int64_t e) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const A x = to_acc<T>(v.v[i]);
      if (REDUCE == kSum || REDUCE == kMean) {
        val[i] += x;
      } else if (REDUCE == kMin) {
        if (x < val[i]) { val[i] = x; arg[i] = e; }
      } else {
        if (x > val[i]) { val[i] = x; arg[i] = e; }
      }
    }
  }
  // Merge another lane's partial; on equal values the smaller position wins so that the final
  // arg is the first occurrence over the whole row.
  __device__ __forceinline__ void merge(const A *oval, const int64_t *oarg) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (REDUCE == kSum || REDUCE == kMean) {
        val[i] += oval[i];
      } else {
        const bool better = (REDUCE == kMin) ? (oval[i] < val[i]) : (oval[i] > val[i]);
        if (better || (oval[i] == val[i] && oarg[i] < arg[i])) { val[i] = oval[i]; arg[i] = oarg[i]; }
      }
    }
  }
  __device__ __forceinline__ void butterfly(int from, int to) {
    for (int off = from; off < to; off <<= 1) {
      A oval[VEC];
      int64_t oarg[kArg ? VEC : 1];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        oval[i] = shfl_xor<A>(val[i], off);
        if (kArg) oarg[i] = shfl_xor<int64_t>(arg[i], off);
      }
      merge(oval, oarg);
    }
  }
};

// value / count in the arithmetic of T, count converted the way the upstream writer does
// (csrc/cpu/reducer.h:74-75: `val / (scalar_t)(count > 0 ? count : 1)` with an int count).
template <typename T> __device__ __forceinline__ T div_by_count(T v, int64_t count) { return v / (T)(int)count; }
template <> __device__ __forceinline__ __half div_by_count<__half>(__half v, int64_t count) {
  return __float2half_rn(__half2float(v) / __half2float(__int2half_rn((int)count)));
}
template <> __device__ __forceinline__ __nv_bfloat16 div_by_count<__nv_bfloat16>(__nv_bfloat16 v, int64_t count) {
  return __float2bfloat16_rn(__bfloat162float(v) / __bfloat162float(__int2bfloat16_rn((int)count)));
}

// Writes one finished row (this lane's VEC columns of it).  `acc` is the reduction over the row's
// source entries only; in kCooSeeded mode the row's previous value of `out` joins here.
template <typename T, int REDUCE, int VEC>
__device__ __forceinline__ void write_row(const RowAcc<T, REDUCE, VEC> &acc, T *out_p, int64_t *arg_p,
                                          int64_t len, int mode, int64_t sentinel) {
  using A = acc_t<T>;
  constexpr bool kArg = RowAcc<T, REDUCE, VEC>::kArg;
  if (mode == kCooSeeded && len == 0) {  // a row the index never names keeps its value
    if (kArg) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) arg_p[i] = sentinel;
    }
    return;
  }
  Pack<T, VEC> seed;
  if (mode == kCooSeeded) seed = ld_pack<T, VEC>(out_p);
  Pack<T, VEC> o;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    A v = acc.val[i];
    if (!kArg) {
      if (mode == kCooSeeded) v += to_acc<T>(seed.v[i]);
      T r = from_acc<T>(v);
      if (REDUCE == kMean) r = div_by_count<T>(r, len > 0 ? len : 1);
      o.v[i] = r;
    } else {
      int64_t a = acc.arg[i];
      if (mode == kCsr) {
        if (len == 0) { v = (A)0; a = sentinel; }
      } else if (mode == kCooFresh) {
        if (v == reduce_identity<T, REDUCE>()) v = (A)0;
      } else {
        const A s = to_acc<T>(seed.v[i]);
        const bool seed_wins = (REDUCE == kMin) ? (s < v) : (s > v);
        if (seed_wins) { v = s; a = sentinel; }
      }
      o.v[i] = from_acc<T>(v);
      arg_p[i] = a;
    }
  }
  st_pack<T, VEC>(out_p, o);
}

// Kernel A: one warp per CTA streams a chunk of consecutive rows (long rows are skipped here).
// Single-warp CTAs let the hardware scheduler balance chunks of very different sizes: a warp that
// finishes early frees its slot at once instead of idling until its CTA's slowest warp is done.
template <typename T, int REDUCE, int VEC, int D>
__global__ void __launch_bounds__(32) csr_stream_kernel(CsrParams p, CsrGeom g) {
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC>;
  constexpr bool kArg = Acc::kArg;

  const T *__restrict__ src = static_cast<const T *>(p.src);
  T *__restrict__ out = static_cast<T *>(p.out);

  const int L = 1 << g.l_log2;
  const int lane = threadIdx.x;
  const int col = lane & (L - 1);
  const int sub = lane >> g.l_log2;
  const int eps = 32 >> g.l_log2;
  const int64_t Kv = p.K / VEC;

  const int RW = g.rows_per_warp;
  const int64_t chunks_per_batch = (p.N + RW - 1) / RW;
  const int64_t chunk = blockIdx.x;
  const int64_t b = chunk / chunks_per_batch;
  const int64_t n0 = (chunk - b * chunks_per_batch) * RW;
  const int nrows = (int)((p.N - n0) < RW ? (p.N - n0) : RW);
  const int64_t *ip = p.indptr + b * p.bstride + n0;

  // lane j holds boundary j of the chunk (clamped and made monotone, so that bad row pointers can
  // never take a load or a store out of bounds); lanes past nrows repeat the last boundary
  int64_t bnd = (lane <= nrows) ? clamp64(ip[lane], 0, p.E) : 0;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int64_t o = (int64_t)__shfl_up_sync(kFullMask, (long long)bnd, off);
    if (lane >= off && o > bnd) bnd = o;
  }
  const int64_t next_bnd = (int64_t)__shfl_down_sync(kFullMask, (long long)bnd, 1);
  const unsigned long_mask = __ballot_sync(kFullMask, lane < nrows && (next_bnd - bnd) >= g.long_len);

  const T *bsrc = src + (b * p.E) * p.K;
  const int64_t row0 = b * p.N + n0;
  const int64_t step_stride = (int64_t)eps * p.K;  // elements between consecutive steps of a lane

  Pack<T, VEC> fill;  // what a lane without an entry holds: the identity, so that it never matters
#pragma unroll
  for (int i = 0; i < VEC; ++i) fill.v[i] = from_acc<T>(reduce_identity<T, REDUCE>());

  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;
    T *obase = out + row0 * p.K + c * VEC;
    int64_t *abase = kArg ? p.arg_out + row0 * p.K + c * VEC : nullptr;

    int ra = 0;
    while (ra < nrows) {  // one iteration per maximal run of non-long rows
      const unsigned rest = long_mask >> ra;
      if (rest & 1u) { ++ra; continue; }
      const int rb = rest ? ra + (__ffs((int)rest) - 1) : nrows;
      const int64_t s = (int64_t)__shfl_sync(kFullMask, (long long)bnd, ra);
      // boundaries of this run relative to its first entry: < 31 * long_len, fits 32 bits
      const int64_t rel64 = bnd - s;
      const int rel = rel64 < 0 ? 0 : (rel64 > 0x3fffffff ? 0x3fffffff : (int)rel64);
      const int t = __shfl_sync(kFullMask, rel, rb);

      int cur = ra;
      int cur_start = 0;
      int cur_end = __shfl_sync(kFullMask, rel, ra + 1);
      Acc acc;
      acc.init(p.E);

      // Closes every row that ends at or before `step_end`; `v` is this lane's entry `e` of the step.
      auto close_rows = [&](const Pack<T, VEC> &v, int e, int step_end) {
        while (cur < rb && cur_end <= step_end) {
          Acc tot = acc;
          if (e >= cur_start && e < cur_end) tot.update(v, s + e);
          tot.butterfly(L, 32);
          if (sub == 0 && col_ok) {
            write_row<T, REDUCE, VEC>(tot, obase + (int64_t)cur * p.K, kArg ? abase + (int64_t)cur * p.K : nullptr,
                                      (int64_t)(cur_end - cur_start), p.mode, p.E);
          }
          if (lane == 0 && cb == 0 && p.count_out != nullptr) {
            const int len = cur_end - cur_start;
            static_cast<T *>(p.count_out)[row0 + cur] = from_acc<T>((A)(len > 0 ? len : 1));
          }
          acc.init(p.E);
          ++cur;
          cur_start = cur_end;
          cur_end = __shfl_sync(kFullMask, rel, cur + 1 <= nrows ? cur + 1 : nrows);
        }
      };

      const T *next_ptr = bsrc + (s + sub) * p.K + c * VEC;
      int next_rel = sub;
      Pack<T, VEC> ring[D];
#pragma unroll
      for (int j = 0; j < D; ++j) {
        ring[j] = (col_ok && next_rel < t) ? ld_stream<T, VEC>(next_ptr) : fill;
        next_ptr += step_stride;
        next_rel += eps;
      }
      for (int pos0 = 0; pos0 < t; pos0 += D * eps) {
#pragma unroll
        for (int j = 0; j < D; ++j) {
          const int pos = pos0 + j * eps;
          if (pos < t) {  // warp-uniform
            const Pack<T, VEC> v = ring[j];
            ring[j] = (col_ok && next_rel < t) ? ld_stream<T, VEC>(next_ptr) : fill;
            next_ptr += step_stride;
            next_rel += eps;
            const int e = pos + sub;
            const int step_end = (pos + eps < t) ? pos + eps : t;
            if (cur_end <= step_end) {
              close_rows(v, e, step_end);
              if (e >= cur_start) acc.update(v, s + e);  // the row still open after this step
            } else {
              acc.update(v, s + e);
            }
          }
        }
      }
      // rows without any entry at the end of the run (or a run with no entries at all)
      close_rows(fill, t, t);
      ra = rb;
    }
  }
}

// Kernel B: rows of at least long_len entries, skipped by kernel A.  Every CTA scans a block of rows
// for long ones (the row pointers are L2-resident after kernel A) and reduces each with all its
// warps striding over the row; per-warp partials are folded through shared memory in warp order.
constexpr int kLongThreads = 1024;
constexpr int kLongWarps = kLongThreads / 32;

template <typename T, int REDUCE, int VEC, int U>
__global__ void __launch_bounds__(kLongThreads) csr_long_rows_kernel(CsrParams p, CsrGeom g) {
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC>;
  constexpr bool kArg = Acc::kArg;

  const T *__restrict__ src = static_cast<const T *>(p.src);
  T *__restrict__ out = static_cast<T *>(p.out);

  const int L = 1 << g.l_log2;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int col = lane & (L - 1);
  const int sub = lane >> g.l_log2;
  const int eps = 32 >> g.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t total_rows = p.B * p.N;

  __shared__ int64_t s_long[kLongThreads];
  __shared__ int s_nlong;
  extern __shared__ __align__(16) unsigned char s_dyn[];
  A *s_val = reinterpret_cast<A *>(s_dyn);                                                  // [kLongWarps][32*VEC]
  int64_t *s_arg = reinterpret_cast<int64_t *>(s_dyn + sizeof(A) * kLongWarps * 32 * VEC);  // same shape, kArg only

  if (tid == 0) s_nlong = 0;
  __syncthreads();
  const int64_t row = (int64_t)blockIdx.x * kLongThreads + tid;
  if (row < total_rows) {
    const int64_t b = row / p.N;
    const int64_t *ip = p.indptr + b * p.bstride + (row - b * p.N);
    const int64_t rs = clamp64(ip[0], 0, p.E);
    const int64_t re = clamp64(ip[1], rs, p.E);
    if (re - rs >= g.long_len) s_long[atomicAdd(&s_nlong, 1)] = row;
  }
  __syncthreads();
  const int nlong = s_nlong;
  if (nlong == 0) return;

  const int64_t stride = (int64_t)kLongWarps * eps;
  for (int i = 0; i < nlong; ++i) {
    const int64_t lrow = s_long[i];
    const int64_t lb = lrow / p.N;
    const int64_t *ip = p.indptr + lb * p.bstride + (lrow - lb * p.N);
    const int64_t lrs = clamp64(ip[0], 0, p.E);
    const int64_t lre = clamp64(ip[1], lrs, p.E);
    const int64_t llen = lre - lrs;
    for (int64_t cb = 0; cb < Kv; cb += L) {
      const int64_t c = cb + col;
      const bool col_ok = c < Kv;
      Acc acc;
      acc.init(p.E);
      const T *base = src + (lb * p.E) * p.K + c * VEC;
      if (col_ok) {
        int64_t e = lrs + (int64_t)warp * eps + sub;
        for (; e + (U - 1) * stride < lre; e += U * stride) {
          Pack<T, VEC> v[U];
#pragma unroll
          for (int u = 0; u < U; ++u) v[u] = ld_stream<T, VEC>(base + (e + u * stride) * p.K);
#pragma unroll
          for (int u = 0; u < U; ++u) acc.update(v[u], e + u * stride);
        }
        for (; e < lre; e += stride) acc.update(ld_stream<T, VEC>(base + e * p.K), e);
      }
      acc.butterfly(L, 32);
      if (sub == 0) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          s_val[warp * 32 * VEC + col * VEC + k] = acc.val[k];
          if (kArg) s_arg[warp * 32 * VEC + col * VEC + k] = acc.arg[k];
        }
      }
      __syncthreads();
      if (warp == 0 && sub == 0) {
        // warp 0 already holds its own partial in acc; fold in the other warps in order
        for (int w = 1; w < kLongWarps; ++w) {
          A oval[VEC];
          int64_t oarg[kArg ? VEC : 1];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            oval[k] = s_val[w * 32 * VEC + col * VEC + k];
            if (kArg) oarg[k] = s_arg[w * 32 * VEC + col * VEC + k];
          }
          acc.merge(oval, oarg);
        }
        if (col_ok) {
          write_row<T, REDUCE, VEC>(acc, out + lrow * p.K + c * VEC,
                                    kArg ? p.arg_out + lrow * p.K + c * VEC : nullptr, llen, p.mode, p.E);
        }
      }
      __syncthreads();
    }
    if (tid == 0 && p.count_out != nullptr) {
      static_cast<T *>(p.count_out)[lrow] = from_acc<T>((A)(llen > 0 ? llen : 1));
    }
  }
}

int64_t env_int(const char *name, int64_t fallback) {
  const char *s = std::getenv(name);
  if (s == nullptr || *s == '\0') return fallback;
  char *end = nullptr;
  const long long v = std::strtoll(s, &end, 10);
  return (end != nullptr && *end == '\0') ? (int64_t)v : fallback;
}

template <typename T, int REDUCE, int VEC>
int launch_vec(const CsrParams &p, cudaStream_t stream) {
  using A = acc_t<T>;
  constexpr bool kArg = (REDUCE == kMin || REDUCE == kMax);
  constexpr int kDepth = kArg ? 4 : 8;   // load ring depth: 8 steps (4 KiB per warp) in flight for sums
  constexpr int kUnroll = kArg ? 2 : 4;  // loads in flight per thread in the long-row kernel
  const int64_t Kv = p.K / VEC;

  CsrGeom g;
  g.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  // Chunk size: rows holding about 128 KiB of source on average, between 4 and 31 rows.
  const int64_t avg = p.N > 0 ? (p.E + p.N - 1) / p.N : 1;
  const int64_t row_bytes = (avg > 0 ? avg : 1) * p.K * (int64_t)sizeof(T);
  int64_t rw = (128 * 1024) / row_bytes;
  if (rw < 4) rw = 4;
  rw = env_int("TSB_CSR_ROWS_PER_WARP", rw);  // test hook
  if (rw < 1) rw = 1;
  if (rw > kMaxRowsPerWarp) rw = kMaxRowsPerWarp;
  g.rows_per_warp = (int)rw;
  // A row leaves the stream for the whole-CTA kernel once it holds 128 KiB of source data.
  const int64_t long_bytes = env_int("TSB_CSR_LONG_BYTES", 128 * 1024);  // test hook
  const int64_t long_len = long_bytes / (p.K * (int64_t)sizeof(T));
  g.long_len = long_len < 1 ? 1 : long_len;

  const int64_t chunks = p.B * ((p.N + g.rows_per_warp - 1) / g.rows_per_warp);
  if (chunks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  csr_stream_kernel<T, REDUCE, VEC, kDepth><<<(unsigned)chunks, 32, 0, stream>>>(p, g);

  // no row can reach long_len when the whole reduced dimension is shorter
  if (p.E >= g.long_len) {
    const size_t dyn = (size_t)kLongWarps * 32 * VEC * (sizeof(A) + (kArg ? sizeof(int64_t) : 0));
    static bool attr_set = false;  // per instantiation; the value never changes
    if (dyn > 48 * 1024 && !attr_set) {
      if (cudaFuncSetAttribute(csr_long_rows_kernel<T, REDUCE, VEC, kUnroll>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)dyn) != cudaSuccess)
        return TSB_ERR_LAUNCH;
      attr_set = true;
    }
    const int64_t blocks = (p.B * p.N + kLongThreads - 1) / kLongThreads;
    csr_long_rows_kernel<T, REDUCE, VEC, kUnroll><<<(unsigned)blocks, kLongThreads, dyn, stream>>>(p, g);
  }
  return launch_status();
}

template <typename T, int REDUCE>
int launch_typed(const CsrParams &p, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  if (p.B * p.N == 0) return TSB_OK;
  const bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out);
  return vec_ok ? launch_vec<T, REDUCE, kFull>(p, stream) : launch_vec<T, REDUCE, 1>(p, stream);
}

}  // namespace

int launch_csr_reduce(const CsrParams &p, int dtype, int reduce, cudaStream_t stream) {
  if (p.B < 0 || p.E < 0 || p.K < 0 || p.N < 0) return TSB_ERR_ARG;
  if (p.B * p.N * p.K == 0) return TSB_OK;
  if (p.src == nullptr && p.E > 0) return TSB_ERR_ARG;
  if (p.indptr == nullptr || p.out == nullptr) return TSB_ERR_ARG;
  if ((reduce == TSB_MIN || reduce == TSB_MAX) && p.arg_out == nullptr) return TSB_ERR_ARG;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    switch (reduce) {
      case TSB_SUM: return launch_typed<scalar_t, kSum>(p, stream);
      case TSB_MEAN: return launch_typed<scalar_t, kMean>(p, stream);
      case TSB_MIN: return launch_typed<scalar_t, kMin>(p, stream);
      case TSB_MAX: return launch_typed<scalar_t, kMax>(p, stream);
      default: return TSB_ERR_REDUCE;
    }
  });
}

}  // namespace tsb

extern "C" int tsb_segment_csr(const void *src, const int64_t *indptr, void *out, int64_t *arg_out,
                               int64_t B, int64_t E, int64_t K, int64_t N, int64_t indptr_batch_stride,
                               int dtype, int reduce, tsb_stream_t stream) {
  tsb::CsrParams p;
  p.src = src;
  p.indptr = indptr;
  p.out = out;
  p.arg_out = arg_out;
  p.count_out = nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.bstride = indptr_batch_stride;
  p.mode = tsb::kCsr;
  return tsb::launch_csr_reduce(p, dtype, reduce, reinterpret_cast<cudaStream_t>(stream));
}

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
// Rows of at least `long_len` entries (64 KiB of source) are cut out of the stream, queued in shared
// memory and reduced afterwards by the whole CTA (eight warps striding over the row, partials
// combined through shared memory in a fixed order).
// Nothing is atomic: results depend only on the shapes, never on scheduling.
//
// Replaces segment_csr_kernel / segment_csr_broadcast_kernel of the upstream project
// (csrc/cuda/segment_csr_cuda.cu:15-95), which walk each row with a single thread per feature.
#include <cstdlib>

#include "csr_reduce.cuh"

namespace tsb {

namespace {

constexpr int kWarpsPerCta = kThreads / 32;
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

template <typename T, int REDUCE, int VEC, int D>
__global__ void __launch_bounds__(kThreads) csr_stream_kernel(CsrParams p, CsrGeom g) {
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

  __shared__ int64_t s_long[kWarpsPerCta * kMaxRowsPerWarp];
  __shared__ int s_nlong;
  __shared__ A s_val[kWarpsPerCta][32 * VEC];
  __shared__ int64_t s_arg[kArg ? kWarpsPerCta : 1][kArg ? 32 * VEC : 1];

  if (tid == 0) s_nlong = 0;
  __syncthreads();

  // ---------------- phase 1: every warp streams its chunk of consecutive rows ----------------
  const int RW = g.rows_per_warp;
  const int64_t chunks_per_batch = (p.N + RW - 1) / RW;
  const int64_t chunk = (int64_t)blockIdx.x * kWarpsPerCta + warp;
  if (chunk < p.B * chunks_per_batch) {  // warp-uniform
    const int64_t b = chunk / chunks_per_batch;
    const int64_t n0 = (chunk - b * chunks_per_batch) * RW;
    const int nrows = (int)((p.N - n0) < RW ? (p.N - n0) : RW);
    const int64_t *ip = p.indptr + b * p.bstride + n0;

    // lane j holds boundary j of the chunk (clamped and made monotone, so that bad row pointers
    // can never take a load or a store out of bounds); lanes past nrows repeat the last boundary
    int64_t bnd = (lane <= nrows) ? clamp64(ip[lane], 0, p.E) : 0;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int64_t o = (int64_t)__shfl_up_sync(kFullMask, (long long)bnd, off);
      if (lane >= off && o > bnd) bnd = o;
    }
    auto boundary = [&](int i) -> int64_t { return (int64_t)__shfl_sync(kFullMask, (long long)bnd, i); };

    const int64_t next_bnd = (int64_t)__shfl_down_sync(kFullMask, (long long)bnd, 1);
    const unsigned long_mask = __ballot_sync(kFullMask, lane < nrows && (next_bnd - bnd) >= g.long_len);
    if (lane < nrows && ((long_mask >> lane) & 1u)) s_long[atomicAdd(&s_nlong, 1)] = b * p.N + n0 + lane;

    const T *bsrc = src + (b * p.E) * p.K;
    const int64_t row0 = b * p.N + n0;

    for (int64_t cb = 0; cb < Kv; cb += L) {
      const int64_t c = cb + col;
      const bool col_ok = c < Kv;
      const T *base = bsrc + c * VEC;
      T *obase = out + row0 * p.K + c * VEC;
      int64_t *abase = kArg ? p.arg_out + row0 * p.K + c * VEC : nullptr;

      int ra = 0;
      while (ra < nrows) {  // one iteration per maximal run of non-long rows
        const unsigned rest = long_mask >> ra;
        if (rest & 1u) { ++ra; continue; }
        const int rb = rest ? ra + (__ffs((int)rest) - 1) : nrows;
        const int64_t s = boundary(ra), t = boundary(rb);
        const int64_t nsteps = (t - s + eps - 1) / eps;

        int cur = ra;
        int64_t cur_start = s;
        int64_t cur_end = boundary(ra + 1);
        Acc acc;
        acc.init(p.E);

        // Closes every row that ends at or before `step_end`.  `v` holds this lane's entry `e` of
        // the current step (valid == false when there is none).
        auto close_rows = [&](const Pack<T, VEC> &v, int64_t e, bool valid, int64_t step_end) {
          while (cur < rb && cur_end <= step_end) {
            Acc tot = acc;
            if (valid && e >= cur_start && e < cur_end) tot.update(v, e);
            tot.butterfly(L, 32);
            if (sub == 0 && col_ok) {
              write_row<T, REDUCE, VEC>(tot, obase + (int64_t)cur * p.K, kArg ? abase + (int64_t)cur * p.K : nullptr,
                                        cur_end - cur_start, p.mode, p.E);
            }
            if (lane == 0 && cb == 0 && p.count_out != nullptr) {
              const int64_t len = cur_end - cur_start;
              static_cast<T *>(p.count_out)[row0 + cur] = from_acc<T>((A)(len > 0 ? len : 1));
            }
            acc.init(p.E);
            ++cur;
            cur_start = cur_end;
            cur_end = boundary(cur + 1 <= nrows ? cur + 1 : nrows);
          }
        };

        Pack<T, VEC> ring[D];
        Pack<T, VEC> zero;
#pragma unroll
        for (int i = 0; i < VEC; ++i) zero.v[i] = from_acc<T>((A)0);
#pragma unroll
        for (int j = 0; j < D; ++j) {
          const int64_t e = s + (int64_t)j * eps + sub;
          ring[j] = (col_ok && e < t) ? ld_stream<T, VEC>(base + e * p.K) : zero;
        }
        for (int64_t step0 = 0; step0 < nsteps; step0 += D) {
#pragma unroll
          for (int j = 0; j < D; ++j) {
            const int64_t step = step0 + j;
            if (step < nsteps) {  // warp-uniform
              const Pack<T, VEC> v = ring[j];
              const int64_t e_next = s + (step + D) * eps + sub;
              ring[j] = (col_ok && e_next < t) ? ld_stream<T, VEC>(base + e_next * p.K) : zero;
              const int64_t pos = s + step * eps;
              const int64_t e = pos + sub;
              const bool valid = e < t;
              const int64_t step_end = (pos + eps < t) ? pos + eps : t;
              if (cur_end <= step_end) close_rows(v, e, valid, step_end);
              if (valid && e >= cur_start) acc.update(v, e);  // the row still open after this step
            }
          }
        }
        // rows without any entry at the end of the run (or a run with no entries at all)
        close_rows(zero, t, false, t);
        ra = rb;
      }
    }
  }

  // ---------------- phase 2: queued long rows, whole CTA per row ----------------
  __syncthreads();
  const int nlong = s_nlong;
  if (nlong == 0) return;
  const int64_t stride = (int64_t)kWarpsPerCta * eps;
  for (int i = 0; i < nlong; ++i) {
    const int64_t lrow = s_long[i];
    const int64_t lb = lrow / p.N;
    const int64_t ln = lrow - lb * p.N;
    const int64_t *ip = p.indptr + lb * p.bstride + ln;
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
        for (; e + 3 * stride < lre; e += 4 * stride) {
          const Pack<T, VEC> v0 = ld_stream<T, VEC>(base + e * p.K);
          const Pack<T, VEC> v1 = ld_stream<T, VEC>(base + (e + stride) * p.K);
          const Pack<T, VEC> v2 = ld_stream<T, VEC>(base + (e + 2 * stride) * p.K);
          const Pack<T, VEC> v3 = ld_stream<T, VEC>(base + (e + 3 * stride) * p.K);
          acc.update(v0, e);
          acc.update(v1, e + stride);
          acc.update(v2, e + 2 * stride);
          acc.update(v3, e + 3 * stride);
        }
        for (; e < lre; e += stride) acc.update(ld_stream<T, VEC>(base + e * p.K), e);
      }
      acc.butterfly(L, 32);
      if (sub == 0) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          s_val[warp][col * VEC + k] = acc.val[k];
          if (kArg) s_arg[warp][col * VEC + k] = acc.arg[k];
        }
      }
      __syncthreads();
      if (warp == 0 && sub == 0) {
        // warp 0 already holds its own partial in acc; fold in warps 1..7 in order
        for (int w = 1; w < kWarpsPerCta; ++w) {
          A oval[VEC];
          int64_t oarg[kArg ? VEC : 1];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            oval[k] = s_val[w][col * VEC + k];
            if (kArg) oarg[k] = s_arg[w][col * VEC + k];
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

template <typename T, int REDUCE>
int launch_typed(const CsrParams &p, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  constexpr bool kArg = (REDUCE == kMin || REDUCE == kMax);
  constexpr int kDepth = kArg ? 4 : 8;  // ring depth: 8 steps (4 KiB per warp) in flight for sums
  if (p.B * p.N == 0) return TSB_OK;
  const bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out);
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);

  CsrGeom g;
  g.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  // Chunk size: enough rows that an average chunk spans a few ring refills, at most 31.
  const int eps = 32 >> g.l_log2;
  const int64_t avg = p.N > 0 ? (p.E + p.N - 1) / p.N : 1;
  int64_t rw = (int64_t)eps * kDepth * 4 / (avg > 0 ? avg : 1);
  if (rw < 8) rw = 8;
  if (rw > kMaxRowsPerWarp) rw = kMaxRowsPerWarp;
  rw = env_int("TSB_CSR_ROWS_PER_WARP", rw);  // test hook
  if (rw < 1) rw = 1;
  if (rw > kMaxRowsPerWarp) rw = kMaxRowsPerWarp;
  g.rows_per_warp = (int)rw;
  // A row goes to the whole CTA once it holds 64 KiB of source data.
  const int64_t long_bytes = env_int("TSB_CSR_LONG_BYTES", 64 * 1024);  // test hook
  const int64_t long_len = long_bytes / (p.K * (int64_t)sizeof(T));
  g.long_len = long_len < 1 ? 1 : long_len;

  const int64_t chunks = p.B * ((p.N + g.rows_per_warp - 1) / g.rows_per_warp);
  const int64_t blocks = (chunks + kWarpsPerCta - 1) / kWarpsPerCta;
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  if (vec_ok) {
    csr_stream_kernel<T, REDUCE, kFull, kDepth><<<(unsigned)blocks, kThreads, 0, stream>>>(p, g);
  } else {
    csr_stream_kernel<T, REDUCE, 1, kDepth><<<(unsigned)blocks, kThreads, 0, stream>>>(p, g);
  }
  return launch_status();
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

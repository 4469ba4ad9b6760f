// Shared pieces of the row-pointer reduction's kernels (segment_csr.cu: streaming, staged and fix-up kernels;
// segment_csr_walk.cu: the walking kernel; segment_csr_rows.cu: the row-parallel kernel): chunk geometry, per-lane row
// accumulators, the row writer and the cooperative row searches.  Split over translation units so that they compile
// side by side.
#pragma once

#include <cstdlib>

#include "csr_reduce.cuh"

namespace tsb {
namespace {


// Resident single-warp CTAs per SM the streaming kernel is compiled for (caps its registers at 80),
// and the depth of its shared-memory load ring (a power of two): 16 steps of 512 bytes = 8 KiB in
// flight per warp, 192 KiB per SM.
constexpr int kMinCtasPerSm = 24;
constexpr int kRingDepth = 16;
constexpr int kWindowRows = 31;          // lane j holds row pointer j of the window, so rows+1 <= 32
constexpr int kEmptyRun = 31;            // a warp closes at least this many rows without entries in a row before it searches for the run's end
constexpr int kRelInf = 0x3fffffff;      // "never ends inside this chunk"
constexpr int64_t kChunkBytes = 128 * 1024;
constexpr int64_t kFlatTileBytes = 32 * 1024;  // K == 1: a chunk is staged whole in shared memory (csr_flat_kernel)
constexpr int kFlatThreads = 128;
constexpr int64_t kFlatRowBytes = 0;           // widest entry (besides K == 1) that goes through csr_flat_kernel: none.
                                               // Measured at 64 / 128 / 256 bytes per entry: 0.45 vs 0.26 ms (fp32 F=16),
                                               // 1.07 vs 0.55 ms (bf16 F=64), 1.54 vs 0.73 ms (fp32 F=64) against the stream.
constexpr int kFlatLongRow = 64;               // entries inside the chunk from which a warp, not a thread, reduces a row

struct CsrGeom {
  int l_log2;            // lanes per entry
  int chunk_entries;     // C: entries per chunk (a power of two >= 32)
  int64_t chunks;        // chunks per batch = max(1, ceil(E / C))
  // workspace: per chunk two partial rows (HEAD, TAIL) of K accumulators, the same of int64 arg
  // indices for MIN/MAX, and the id of the row whose HEAD partial the chunk stored (-1: none)
  void *carry_val;
  int64_t *carry_arg;
  int64_t *head_row;
  // the fix-up kernel writes the rows without entries that follow kEmptyRun or more such rows (the streaming and the
  // walking kernel stop closing a run there; the staged kernel hands rows to lane groups anyway and writes its own)
  bool fill_empty = false;
};

// Chunk length: a power of two holding about kChunkBytes of source, shortened (down to one full
// warp step) when the whole reduced dimension would otherwise give too few chunks to occupy the GPU.
// Entries narrow enough for csr_flat_kernel: K == 1; the test hook TSB_CSR_FORCE_FLAT=1 sends every entry of up
// to 64 bytes through it.
inline bool flat_rows(int64_t K, size_t elem) {
  int64_t limit = kFlatRowBytes;
  if (const char *v = std::getenv("TSB_CSR_FORCE_FLAT")) limit = (*v == '1') ? 64 : limit;
  return K == 1 || K * (int64_t)elem <= limit;
}

inline int chunk_entries_for(int64_t K, size_t elem, int64_t E) {
  const bool flat = flat_rows(K, elem);
  int64_t c = (flat ? kFlatTileBytes : kChunkBytes) / (K * (int64_t)elem);
  // ~7 single-warp CTAs per resident slot of a 148-SM part; flat kernel: 128-thread CTAs that pay two row searches each
  const int64_t want_chunks = flat ? 4096 : 16384;
  if (E / want_chunks < c) c = E / want_chunks;
  if (const char *forced = std::getenv("TSB_CSR_CHUNK_ENTRIES")) {  // test hook: force short chunks
    const long long v = std::atoll(forced);
    if (v >= 32) c = v;
  }
  int64_t pow2 = 32;
  while (pow2 * 2 <= c && pow2 < (1 << 20)) pow2 *= 2;
  return (int)pow2;
}

// Per-lane accumulators of one row: VEC values and, for the reductions that need it, a second word per
// value - the arg index for MIN/MAX, the bits of the running sum for LSE.
// LSE is the online log-sum-exp: `val` holds the running maximum m, the second word the running sum
// s = sum exp(x - m); two partials combine as m = max(m1, m2), s = s1 exp(m1 - m) + s2 exp(m2 - m), and
// the row result is m + log s.  It exists for fp32 accumulators only (fp32 / fp16 / bf16 sources).
template <typename T, int REDUCE, int VEC, typename ArgT = int64_t> struct RowAcc {
  using A = acc_t<T>;
  static constexpr bool kArg = (REDUCE == kMin || REDUCE == kMax);
  static constexpr bool kLseAcc = (REDUCE == kLse);
  static constexpr bool kPair = kArg || kLseAcc;
  A val[VEC];
  ArgT arg[kPair ? VEC : 1];

  static __device__ __forceinline__ float sum_of(ArgT word) { return __int_as_float((int)word); }
  static __device__ __forceinline__ ArgT word_of(float s) { return (ArgT)__float_as_int(s); }

  __device__ __forceinline__ void init(ArgT sentinel) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      val[i] = reduce_identity<T, REDUCE>();
      if (kArg) arg[i] = sentinel;
      if (kLseAcc) arg[i] = word_of(0.0f);
    }
  }
  // Entries arrive in increasing e within a lane, so strict comparisons keep the first winner
  // (csrc/cpu/reducer.h:63-67).
  // TIES (entries arrive in no particular order): an equal value wins if its id is smaller.
  template <bool TIES = false> __device__ __forceinline__ void update(const Pack<T, VEC> &v, ArgT e, ArgT none = 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const A x = to_acc<T>(v.v[i]);
      if (REDUCE == kSum || REDUCE == kMean) {
        val[i] += x;
      } else if (REDUCE == kMul) {
        val[i] *= x;
      } else if (REDUCE == kMin) {
        if (x < val[i] || (TIES && x == val[i] && e < arg[i] && arg[i] != none)) { val[i] = x; arg[i] = e; }
      } else if (REDUCE == kMax) {
        if (x > val[i] || (TIES && x == val[i] && e < arg[i] && arg[i] != none)) { val[i] = x; arg[i] = e; }
      } else {
        // One exponential, no branch: whichever of the running maximum and x is larger becomes the
        // reference, the other side is scaled by exp(-|x - m|).  The identity is the lowest finite float,
        // so the first entry gives exp(-huge) = 0 for the empty sum, and an entry of -inf adds 0.
        const float m = (float)val[i], xf = (float)x;
        const float d = xf == m ? 0.0f : xf - m;  // equal infinities: inf - inf would be NaN, upstream gives +inf
        const float e = __expf(-fabsf(d));
        const float sum = sum_of(arg[i]);
        arg[i] = word_of(d > 0.0f ? fmaf(sum, e, 1.0f) : sum + e);
        val[i] = (A)fmaxf(m, xf);
      }
    }
  }
  // Merge another lane's partial; for MIN/MAX the smaller position wins on equal values so that the
  // final arg is the first occurrence over the whole row.
  __device__ __forceinline__ void merge(const A *oval, const ArgT *oarg) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      if (REDUCE == kSum || REDUCE == kMean) {
        val[i] += oval[i];
      } else if (REDUCE == kMul) {
        val[i] *= oval[i];
      } else if (kArg) {
        const bool better = (REDUCE == kMin) ? (oval[i] < val[i]) : (oval[i] > val[i]);
        if (better || (oval[i] == val[i] && oarg[i] < arg[i])) { val[i] = oval[i]; arg[i] = oarg[i]; }
      } else {
        const float m1 = (float)val[i], m2 = (float)oval[i];
        const float d = m2 == m1 ? 0.0f : m2 - m1;
        const float e = __expf(-fabsf(d));
        const float s1 = sum_of(arg[i]), s2 = sum_of(oarg[i]);
        arg[i] = word_of(d > 0.0f ? fmaf(s1, e, s2) : fmaf(s2, e, s1));
        val[i] = (A)fmaxf(m1, m2);
      }
    }
  }
  __device__ __forceinline__ void butterfly(int from, int to) {
    for (int off = from; off < to; off <<= 1) {
      A oval[VEC];
      ArgT oarg[kPair ? VEC : 1];
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        oval[i] = shfl_xor<A>(val[i], off);
        if (kPair) oarg[i] = shfl_xor<ArgT>(arg[i], off);
      }
      merge(oval, oarg);
    }
  }
};

// MEAN: the row total times 1/count (count as upstream's writer converts it: an int, at least 1;
// csrc/cpu/reducer.h:74-75).  For floating types one reciprocal per row replaces VEC divisions; the
// result differs from a true division by at most one ulp, far inside the 1e-5 tolerance.  Integer
// types divide exactly (truncating, as the CPU loop does).
template <typename T, bool INTEGER = std::is_integral<T>::value> struct MeanScale {
  acc_t<T> inv;
  __device__ __forceinline__ explicit MeanScale(int64_t count) : inv((acc_t<T>)1 / (acc_t<T>)(int)count) {}
  __device__ __forceinline__ T apply(acc_t<T> v) const { return from_acc<T>(v * inv); }
};
// integers: the (narrowed) total divided by the count, truncating
template <typename T> struct MeanScale<T, true> {
  int c;
  __device__ __forceinline__ explicit MeanScale(int64_t count) : c((int)count) {}
  __device__ __forceinline__ T apply(acc_t<T> v) const {
    if constexpr (sizeof(T) == 8) return (T)(v / (int64_t)c);
    else return (T)((int32_t)from_acc<T>(v) / c);
  }
};

// Address of element `off` of the output: T everywhere except the LSE table, which is fp32.
template <typename T, int REDUCE, bool EXTRAS>
__device__ __forceinline__ T *row_address(const CsrParams &p, int64_t grow, int64_t col) {
  if constexpr (REDUCE == kLse) {
    return reinterpret_cast<T *>(static_cast<float *>(p.out) + grow * p.K + col);
  } else {
    if (EXTRAS && p.route_world > 0) {  // sharded scatter: the row goes to its owner's staging buffer (maybe over NVLink)
      const int64_t q = grow / p.route_rows;
      const int64_t local = grow - q * p.route_rows;
      return static_cast<T *>(p.route_base[q]) + ((int64_t)p.route_rank * p.route_rows + local) * p.K + col;
    }
    return static_cast<T *>(p.out) + grow * p.K + col;
  }
}

// A routed row of a 16-bit source kept in fp32 (CsrParams::route_wide): this lane's VEC sums go to the owner's
// fp32 staging buffer as they are.  True if the row was stored.
template <typename T, int REDUCE, int VEC, bool EXTRAS, typename ArgT>
__device__ __forceinline__ bool store_wide_routed(const CsrParams &p, const RowAcc<T, REDUCE, VEC, ArgT> &acc,
                                                  int64_t grow, int64_t col) {
  if constexpr (EXTRAS && sizeof(T) == 2 && REDUCE == kSum) {
    if (p.route_world > 0 && p.route_wide) {
      const int64_t q = grow / p.route_rows;
      const int64_t local = grow - q * p.route_rows;
      float *dst = static_cast<float *>(p.route_base[q]) + ((int64_t)p.route_rank * p.route_rows + local) * p.K + col;
      if constexpr (VEC % 4 == 0) {
#pragma unroll
        for (int i = 0; i < VEC; i += 4)
          *reinterpret_cast<float4 *>(dst + i) = make_float4(acc.val[i], acc.val[i + 1], acc.val[i + 2], acc.val[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) dst[i] = acc.val[i];
      }
      return true;
    }
  }
  return false;
}

// Writes one finished row (this lane's VEC columns of it).  `acc` is the reduction over the row's
// source entries only; in kCooSeeded mode the row's previous value of `out` joins here.  Arg indices
// in `acc` are relative to `arg_base`; `arg_none` marks "no element won" and becomes `sentinel`.
template <typename T, int REDUCE, int VEC, typename ArgT>
__device__ __forceinline__ void write_row(const RowAcc<T, REDUCE, VEC, ArgT> &acc, T *out_p, int64_t *arg_p,
                                          int64_t len, int mode, int64_t sentinel, int64_t arg_base, ArgT arg_none) {
  using A = acc_t<T>;
  constexpr bool kArg = RowAcc<T, REDUCE, VEC, ArgT>::kArg;
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
  if constexpr (REDUCE == kLse) {
    // m + log s, fp32 whatever T is (a 16-bit table would cost the softmax its accuracy): `out_p` is the
    // fp32 address.  A row without (finite) entries gives -inf.
    float *o = reinterpret_cast<float *>(out_p);
    float r[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const float sum = RowAcc<T, REDUCE, VEC, ArgT>::sum_of(acc.arg[i]);
      r[i] = sum == 0.0f ? -INFINITY : (float)acc.val[i] + __logf(sum);
    }
    if constexpr (VEC % 4 == 0) {
#pragma unroll
      for (int i = 0; i < VEC; i += 4) *reinterpret_cast<float4 *>(o + i) = make_float4(r[i], r[i + 1], r[i + 2], r[i + 3]);
    } else {
#pragma unroll
      for (int i = 0; i < VEC; ++i) o[i] = r[i];
    }
    return;
  }
  const MeanScale<T> scale(REDUCE == kMean && len > 0 ? len : 1);
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    A v = acc.val[i];
    if (!kArg) {
      if (mode == kCooSeeded) v = (REDUCE == kMul) ? v * to_acc<T>(seed.v[i]) : v + to_acc<T>(seed.v[i]);
      o.v[i] = (REDUCE == kMean) ? scale.apply(v) : from_acc<T>(v);
    } else {
      int64_t a = (acc.arg[i] == arg_none) ? sentinel : arg_base + (int64_t)acc.arg[i];
      if (mode == kCsr) {
        if (len == 0) { v = (A)0; a = sentinel; }
      } else if (mode == kCooFresh) {
        if (v == reduce_identity<T, REDUCE>()) v = (A)0;
      } else {
        const A s = to_acc<T>(seed.v[i]);
        const bool seed_wins = (REDUCE == kMin) ? (s <= v) : (s >= v);
        if (seed_wins) { v = s; a = sentinel; }
      }
      o.v[i] = from_acc<T>(v);
      arg_p[i] = a;
    }
  }
  st_pack<T, VEC>(out_p, o);
}

// First row whose end (indptr[r + 1]) lies after `pos`, by a cooperative 32-ary search of one warp; N if none.
__device__ __forceinline__ int64_t first_row_ending_after(const int64_t *ip, int64_t N, int64_t pos, int lane) {
  int64_t lo = 0, hi = N;  // answer in [lo, hi]; hi == N means "no such row"
  while (hi - lo > 32) {
    const int64_t step = (hi - lo + 31) / 32;
    int64_t probe = lo + (lane + 1) * step - 1;
    if (probe > hi - 1) probe = hi - 1;
    const unsigned gt = __ballot_sync(kFullMask, ip[probe + 1] > pos);
    if (gt == 0) { lo = hi; break; }
    const int f = __ffs((int)gt) - 1;
    const int64_t new_hi = lo + (int64_t)(f + 1) * step - 1;
    lo = lo + (int64_t)f * step;
    hi = new_hi < hi - 1 ? new_hi : hi - 1;  // ends[hi] > pos is known: the answer is <= hi
    if (hi < lo) hi = lo;
  }
  if (lo >= N) return N;
  const bool in = lo + lane <= hi && lo + lane < N;
  const unsigned gt = __ballot_sync(kFullMask, in && ip[lo + lane + 1] > pos);
  return gt ? lo + (__ffs((int)gt) - 1) : hi;
}

// The same, not inlined, for call sites that run once per long run of empty rows inside issue-bound loops.
__device__ __noinline__ int64_t first_row_ending_after_cold(const int64_t *ip, int64_t N, int64_t pos, int lane) {
  return first_row_ending_after(ip, N, pos, lane);
}

// The same search by one group of L lanes (`gmask`: the group's lanes, `gbase`: its first lane, `col`: the lane inside
// the group), over rows [from, N): every group of a warp may be in a search of its own.
// Not inlined: it runs once per long run of empty rows, and the row-closing code it is called from is inlined twice
// into kernels that are bound by instruction issue.
__device__ __noinline__ int64_t first_row_ending_after_group(const int64_t *ip, int64_t from, int64_t N, int64_t pos, int col,
                                                             int L, unsigned gmask, int gbase) {
  int64_t lo = from < N ? from : N, hi = N;
  while (hi - lo > L) {
    const int64_t step = (hi - lo + L - 1) / L;
    int64_t probe = lo + (col + 1) * step - 1;
    if (probe > hi - 1) probe = hi - 1;
    const unsigned gt = (__ballot_sync(gmask, ip[probe + 1] > pos) & gmask) >> gbase;
    if (gt == 0) { lo = hi; break; }
    const int f = __ffs((int)gt) - 1;
    const int64_t new_hi = lo + (int64_t)(f + 1) * step - 1;
    lo = lo + (int64_t)f * step;
    hi = new_hi < hi - 1 ? new_hi : hi - 1;
    if (hi < lo) hi = lo;
  }
  if (lo >= N) return N;
  const bool in = lo + col <= hi && lo + col < N;
  const unsigned gt = (__ballot_sync(gmask, in && ip[lo + col + 1] > pos) & gmask) >> gbase;
  return gt ? lo + (__ffs((int)gt) - 1) : hi;
}

}  // namespace

// Launches csr_walk_kernel (segment_csr_walk.cu) for `dtype` / `reduce`; `wide`: two 16-byte packs per lane (built for
// fp32 sum / mean over a contiguous source only); mode 0: contiguous source, 1: through CsrParams::perm, 2: perm plus the
// sharded-scatter features.  Returns false if that combination is not built (the caller then streams).
bool launch_csr_walk(const CsrParams &p, const void *geom, unsigned total_chunks, int dtype, int reduce, bool wide, int mode,
                     cudaStream_t stream);

// Launches csr_rows_kernel (segment_csr_rows.cu): a lane group per row, for problems whose rows hold only a few
// entries.  `vec`: 16-byte packs (K a multiple of the pack, aligned pointers); mode as above.  Returns false if that
// combination is not built.
bool launch_csr_short_rows(const CsrParams &p, int dtype, int reduce, bool vec, int mode, cudaStream_t stream);

}  // namespace tsb

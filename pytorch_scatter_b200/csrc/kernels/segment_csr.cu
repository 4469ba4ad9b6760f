// segment_csr for sm_100a: row-pointer segmented reduction of src [B,E,K] into out [B,N,K].
//
// Geometry.  One entry (b,e) is K contiguous elements; it is covered by L lanes that each own one
// 16-byte pack (VEC elements).  A row is reduced by a group of G >= L lanes, so G/L entries are
// loaded per step and a warp holds 32/G rows.  G grows with the average row length, L with K, so
// that for K = 64 fp32 a whole warp walks one row two entries (512 contiguous bytes) per step.
// Rows of at least `long_len` entries are not walked by their group: they are queued in shared
// memory and afterwards reduced by the whole CTA, eight warps striding over the row, partials
// combined through shared memory in a fixed order.  Nothing is atomic; the result depends only on
// the shapes, never on scheduling.
//
// Replaces segment_csr_kernel / segment_csr_broadcast_kernel of the upstream project
// (csrc/cuda/segment_csr_cuda.cu:15-95), which walk a row with a single thread per feature.
#include <cstdlib>

#include "csr_reduce.cuh"

namespace tsb {

namespace {

constexpr int kWarpsPerCta = kThreads / 32;

struct CsrGeom {
  int l_log2;        // lanes per entry
  int g_log2;        // lanes per row group
  int64_t long_len;  // rows at least this long are reduced by the whole CTA
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

template <typename T, int REDUCE, int VEC>
__device__ __forceinline__ void write_row(const RowAcc<T, REDUCE, VEC> &acc, T *out_p, int64_t *arg_p,
                                          int64_t len, int mode, int64_t sentinel) {
  using A = acc_t<T>;
  constexpr bool kArg = RowAcc<T, REDUCE, VEC>::kArg;
  Pack<T, VEC> o;
  if (!kArg) {
    if (mode == kCooSeeded && len == 0) return;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      T r = from_acc<T>(acc.val[i]);
      if (REDUCE == kMean) r = div_by_count<T>(r, len > 0 ? len : 1);
      o.v[i] = r;
    }
    st_pack<T, VEC>(out_p, o);
  } else {
    bool write_val = true;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const A ident = reduce_identity<T, REDUCE>();
      T r = from_acc<T>(acc.val[i]);
      int64_t a = acc.arg[i];
      if (mode == kCsr) {
        if (len == 0) { r = from_acc<T>((A)0); a = sentinel; }
      } else if (mode == kCooFresh) {
        if (acc.val[i] == ident) r = from_acc<T>((A)0);
      } else {
        if (len == 0) { write_val = false; a = sentinel; }
      }
      o.v[i] = r;
      arg_p[i] = a;
    }
    if (write_val) st_pack<T, VEC>(out_p, o);
  }
}

template <typename T, int REDUCE, int VEC>
__global__ void __launch_bounds__(kThreads) csr_reduce_kernel(CsrParams p, CsrGeom g) {
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC>;
  constexpr bool kArg = Acc::kArg;

  const T *__restrict__ src = static_cast<const T *>(p.src);
  T *__restrict__ out = static_cast<T *>(p.out);

  const int G = 1 << g.g_log2, L = 1 << g.l_log2;
  const int tid = threadIdx.x;
  const int grp = tid >> g.g_log2;
  const int gl = tid & (G - 1);
  const int col = gl & (L - 1);
  const int sub = gl >> g.l_log2;
  const int eps = G >> g.l_log2;
  const int rows_per_cta = kThreads >> g.g_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t total_rows = p.B * p.N;

  __shared__ int64_t s_long[kThreads];
  __shared__ int s_nlong;
  __shared__ A s_val[kWarpsPerCta][32 * VEC];
  __shared__ int64_t s_arg[kArg ? kWarpsPerCta : 1][kArg ? 32 * VEC : 1];

  if (tid == 0) s_nlong = 0;
  __syncthreads();

  // ---------------- phase 1: one row per lane group ----------------
  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + grp;
  int64_t b = 0, rs = 0, re = 0;
  bool active = false;
  if (row < total_rows) {
    b = row / p.N;
    const int64_t n = row - b * p.N;
    const int64_t *ip = p.indptr + b * p.bstride + n;
    rs = clamp64(ip[0], 0, p.E);
    re = clamp64(ip[1], rs, p.E);
    if (re - rs >= g.long_len) {
      if (gl == 0) s_long[atomicAdd(&s_nlong, 1)] = row;
    } else {
      active = true;
    }
  }
  const int64_t len = re - rs;
  const int64_t e_end = active ? re : rs;

  for (int64_t cb = 0; cb < Kv; cb += L) {
    const int64_t c = cb + col;
    const bool col_ok = c < Kv;
    Acc acc;
    acc.init(p.E);
    const T *base = src + (b * p.E) * p.K + c * VEC;
    if (col_ok) {
      if (p.mode == kCooSeeded && sub == 0 && active && len > 0) {
        const Pack<T, VEC> seed = ld_pack<T, VEC>(out + row * p.K + c * VEC);
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc.val[i] = to_acc<T>(seed.v[i]);
      }
      int64_t e = rs + sub;
      for (; e + 3 * (int64_t)eps < e_end; e += 4 * (int64_t)eps) {
        const Pack<T, VEC> v0 = ld_stream<T, VEC>(base + e * p.K);
        const Pack<T, VEC> v1 = ld_stream<T, VEC>(base + (e + eps) * p.K);
        const Pack<T, VEC> v2 = ld_stream<T, VEC>(base + (e + 2 * eps) * p.K);
        const Pack<T, VEC> v3 = ld_stream<T, VEC>(base + (e + 3 * eps) * p.K);
        acc.update(v0, e);
        acc.update(v1, e + eps);
        acc.update(v2, e + 2 * eps);
        acc.update(v3, e + 3 * eps);
      }
      for (; e < e_end; e += eps) acc.update(ld_stream<T, VEC>(base + e * p.K), e);
    }
    acc.butterfly(L, G);
    if (active && col_ok && sub == 0) {
      write_row<T, REDUCE, VEC>(acc, out + row * p.K + c * VEC, kArg ? p.arg_out + row * p.K + c * VEC : nullptr,
                                len, p.mode, p.E);
    }
  }
  if (active && gl == 0 && p.count_out != nullptr) {
    static_cast<T *>(p.count_out)[row] = from_acc<T>((A)(len > 0 ? len : 1));
  }

  // ---------------- phase 2: queued long rows, whole CTA per row ----------------
  __syncthreads();
  const int nlong = s_nlong;
  if (nlong == 0) return;
  const int warp = tid >> 5, lane = tid & 31;
  const int wcol = lane & (L - 1);
  const int wsub = lane >> g.l_log2;
  const int weps = 32 >> g.l_log2;
  const int64_t stride = (int64_t)kWarpsPerCta * weps;
  for (int i = 0; i < nlong; ++i) {
    const int64_t lrow = s_long[i];
    const int64_t lb = lrow / p.N;
    const int64_t ln = lrow - lb * p.N;
    const int64_t *ip = p.indptr + lb * p.bstride + ln;
    const int64_t lrs = clamp64(ip[0], 0, p.E);
    const int64_t lre = clamp64(ip[1], lrs, p.E);
    const int64_t llen = lre - lrs;
    for (int64_t cb = 0; cb < Kv; cb += L) {
      const int64_t c = cb + wcol;
      const bool col_ok = c < Kv;
      Acc acc;
      acc.init(p.E);
      const T *base = src + (lb * p.E) * p.K + c * VEC;
      if (col_ok) {
        if (p.mode == kCooSeeded && warp == 0 && wsub == 0) {
          const Pack<T, VEC> seed = ld_pack<T, VEC>(out + lrow * p.K + c * VEC);
#pragma unroll
          for (int k = 0; k < VEC; ++k) acc.val[k] = to_acc<T>(seed.v[k]);
        }
        int64_t e = lrs + (int64_t)warp * weps + wsub;
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
      if (wsub == 0) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          s_val[warp][wcol * VEC + k] = acc.val[k];
          if (kArg) s_arg[warp][wcol * VEC + k] = acc.arg[k];
        }
      }
      __syncthreads();
      if (warp == 0 && wsub == 0) {
        // warp 0 already holds its own partial in acc; fold in warps 1..7 in order
        for (int w = 1; w < kWarpsPerCta; ++w) {
          A oval[VEC];
          int64_t oarg[kArg ? VEC : 1];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            oval[k] = s_val[w][wcol * VEC + k];
            if (kArg) oarg[k] = s_arg[w][wcol * VEC + k];
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
  const int64_t total_rows = p.B * p.N;
  if (total_rows == 0) return TSB_OK;
  const bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out);
  const int vec = vec_ok ? kFull : 1;
  const int64_t Kv = p.K / vec;

  CsrGeom g;
  g.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  // Aim at about four steps for an average row: entries per step = avg/4, rounded up to a power of two.
  const int64_t avg = p.N > 0 ? p.E / p.N : 0;
  int g_log2 = g.l_log2 + ilog2_ceil(avg / 4 > 1 ? avg / 4 : 1);
  const int64_t forced = env_int("TSB_CSR_GROUP_LOG2", -1);  // test hook: force the group width
  if (forced >= 0) g_log2 = (int)forced;
  if (g_log2 < g.l_log2) g_log2 = g.l_log2;
  if (g_log2 > 5) g_log2 = 5;
  g.g_log2 = g_log2;
  // A row goes to the whole CTA once it holds 64 KiB of source data.
  const int64_t long_bytes = env_int("TSB_CSR_LONG_BYTES", 64 * 1024);  // test hook
  int64_t long_len = long_bytes / (p.K * (int64_t)sizeof(T));
  g.long_len = long_len < 1 ? 1 : long_len;

  const int rows_per_cta = kThreads >> g.g_log2;
  const int64_t blocks = (total_rows + rows_per_cta - 1) / rows_per_cta;
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  if (vec_ok) {
    csr_reduce_kernel<T, REDUCE, kFull><<<(unsigned)blocks, kThreads, 0, stream>>>(p, g);
  } else {
    csr_reduce_kernel<T, REDUCE, 1><<<(unsigned)blocks, kThreads, 0, stream>>>(p, g);
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

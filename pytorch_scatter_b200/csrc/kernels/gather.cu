// gather_csr, gather_coo and the MIN/MAX backward for sm_100a: pure streaming kernels.
//
// gather_csr is row driven with the lane geometry of the forward reduction (L lanes hold one row
// of K values in 16-byte packs, a group of G lanes writes G/L entries per step); rows holding 64 KiB
// or more are queued in shared memory and written by the whole CTA.  gather_coo is entry driven:
// L lanes copy one entry, the index is read once per entry instead of once per element.
//
// Replaces gather_csr_kernel / gather_csr_broadcast_kernel (csrc/cuda/segment_csr_cuda.cu:170-217)
// and gather_coo_kernel / gather_coo_broadcast_kernel (csrc/cuda/segment_coo_cuda.cu:285-325) of the
// upstream project.
#include "common.cuh"

namespace tsb {
namespace {

template <typename T> __device__ __forceinline__ T div_t(T a, T b) { return a / b; }
template <> __device__ __forceinline__ __half div_t<__half>(__half a, __half b) {
  return __float2half_rn(__half2float(a) / __half2float(b));
}
template <> __device__ __forceinline__ __nv_bfloat16 div_t<__nv_bfloat16>(__nv_bfloat16 a, __nv_bfloat16 b) {
  return __float2bfloat16_rn(__bfloat162float(a) / __bfloat162float(b));
}
// int64 -> T the way Tensor.to(dtype) converts
template <typename T> __device__ __forceinline__ T count_to_t(int64_t c) { return (T)c; }
template <> __device__ __forceinline__ __half count_to_t<__half>(int64_t c) { return __ll2half_rn(c); }
template <> __device__ __forceinline__ __nv_bfloat16 count_to_t<__nv_bfloat16>(int64_t c) { return __ll2bfloat16_rn(c); }

struct GatherCsrParams {
  const void *src;
  const int64_t *indptr;
  void *out;
  int64_t B, E, K, N, bstride;
  int l_log2, g_log2;
  int64_t long_len;
  int divide;
};

template <typename T, int VEC>
__global__ void __launch_bounds__(kThreads) gather_csr_kernel(GatherCsrParams p) {
  const T *__restrict__ src = static_cast<const T *>(p.src);
  T *__restrict__ out = static_cast<T *>(p.out);
  const int G = 1 << p.g_log2, L = 1 << p.l_log2;
  const int tid = threadIdx.x;
  const int grp = tid >> p.g_log2;
  const int gl = tid & (G - 1);
  const int col = gl & (L - 1);
  const int sub = gl >> p.l_log2;
  const int eps = G >> p.l_log2;
  const int rows_per_cta = kThreads >> p.g_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t total_rows = p.B * p.N;

  __shared__ int64_t s_long[kThreads];
  __shared__ int s_nlong;
  if (tid == 0) s_nlong = 0;
  __syncthreads();

  const int64_t row = (int64_t)blockIdx.x * rows_per_cta + grp;
  if (row < total_rows) {
    const int64_t b = row / p.N;
    const int64_t n = row - b * p.N;
    const int64_t *ip = p.indptr + b * p.bstride + n;
    const int64_t rs = clamp64(ip[0], 0, p.E);
    const int64_t re = clamp64(ip[1], rs, p.E);
    if (re - rs >= p.long_len) {
      if (gl == 0) s_long[atomicAdd(&s_nlong, 1)] = row;
    } else if (re > rs) {
      for (int64_t c = col; c < Kv; c += L) {
        Pack<T, VEC> v = ld_pack<T, VEC>(src + row * p.K + c * VEC);
        if (p.divide) {
          const T cnt = count_to_t<T>(re - rs);
#pragma unroll
          for (int i = 0; i < VEC; ++i) v.v[i] = div_t<T>(v.v[i], cnt);
        }
        T *base = out + (b * p.E) * p.K + c * VEC;
        for (int64_t e = rs + sub; e < re; e += eps) st_stream<T, VEC>(base + e * p.K, v);
      }
    }
  }
  __syncthreads();
  const int nlong = s_nlong;
  if (nlong == 0) return;
  const int tcol = tid & (L - 1);
  const int tsub = tid >> p.l_log2;
  const int teps = kThreads >> p.l_log2;
  for (int i = 0; i < nlong; ++i) {
    const int64_t lrow = s_long[i];
    const int64_t b = lrow / p.N;
    const int64_t n = lrow - b * p.N;
    const int64_t *ip = p.indptr + b * p.bstride + n;
    const int64_t rs = clamp64(ip[0], 0, p.E);
    const int64_t re = clamp64(ip[1], rs, p.E);
    for (int64_t c = tcol; c < Kv; c += L) {
      Pack<T, VEC> v = ld_pack<T, VEC>(src + lrow * p.K + c * VEC);
      if (p.divide) {
        const T cnt = count_to_t<T>(re - rs);
#pragma unroll
        for (int k = 0; k < VEC; ++k) v.v[k] = div_t<T>(v.v[k], cnt);
      }
      T *base = out + (b * p.E) * p.K + c * VEC;
      for (int64_t e = rs + tsub; e < re; e += teps) st_stream<T, VEC>(base + e * p.K, v);
    }
  }
}

template <typename T>
int launch_gather_csr(GatherCsrParams p, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  const int64_t total_rows = p.B * p.N;
  if (total_rows == 0 || p.E == 0 || p.K == 0) return TSB_OK;
  const bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out);
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);
  p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  const int64_t avg = p.E / p.N;
  int g_log2 = p.l_log2 + ilog2_ceil(avg / 4 > 1 ? avg / 4 : 1);
  p.g_log2 = g_log2 > 5 ? 5 : g_log2;
  int64_t long_len = (64 * 1024) / (p.K * (int64_t)sizeof(T));
  p.long_len = long_len < 1 ? 1 : long_len;
  const int rows_per_cta = kThreads >> p.g_log2;
  const int64_t blocks = (total_rows + rows_per_cta - 1) / rows_per_cta;
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  if (vec_ok) gather_csr_kernel<T, kFull><<<(unsigned)blocks, kThreads, 0, stream>>>(p);
  else gather_csr_kernel<T, 1><<<(unsigned)blocks, kThreads, 0, stream>>>(p);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
struct GatherCooParams {
  const void *src;
  const int64_t *index;
  void *out;
  const void *count;
  const void *x;  // optional per-entry operand [B,E,K]: out = op(x, gathered row)
  int op;         // 1: exp(x - row), 2: x - row (the second passes of softmax / log_softmax), 3: (x - row)^2
  const float *scale;  // optional second fp32 table [B,N,K]: the result is multiplied by its gathered row
  int64_t B, E, K, N, bstride;
  int l_log2;
};

// A warp owns 128 consecutive entries: it loads their indices with four coalesced loads, then copies
// 32/L rows per step (index broadcast by shuffle), four steps of loads in flight before the stores.
// With a sorted index neighbouring entries name the same source row, which then comes from L1/L2.
constexpr int kGatherBatches = 4;

// A row piece of the fp32 table of the APPLY form: VEC floats fetched 16 bytes at a time.
template <int VEC> struct FloatRow { float v[VEC]; };
template <int VEC> __device__ __forceinline__ FloatRow<VEC> ld_float_row(const float *p) {
  FloatRow<VEC> r;
  if constexpr (VEC % 4 == 0) {
#pragma unroll
    for (int i = 0; i < VEC; i += 4) {
      const float4 t = *reinterpret_cast<const float4 *>(p + i);
      r.v[i] = t.x; r.v[i + 1] = t.y; r.v[i + 2] = t.z; r.v[i + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) r.v[i] = p[i];
  }
  return r;
}

// MODE 0: plain gather.  1: src is an fp32 table and out[e] = op(x[e], src[index[e]]) (op 1: exp(x - row),
// 2: x - row, 3: (x - row)^2).  2: the same times the gathered row of a second fp32 table (`scale`); a mode of its
// own because as a run-time branch it cost the softmax passes a fifth of their speed.
template <typename T, int VEC, int MODE>
__global__ void __launch_bounds__(kThreads) gather_coo_kernel(GatherCooParams p) {
  constexpr bool APPLY = MODE >= 1;
  constexpr bool SCALED = MODE == 2;
  using Row = typename std::conditional<APPLY, FloatRow<VEC>, Pack<T, VEC>>::type;
  const T *__restrict__ src = static_cast<const T *>(p.src);
  const float *__restrict__ table = static_cast<const float *>(p.src);
  T *__restrict__ out = static_cast<T *>(p.out);
  const T *__restrict__ count = static_cast<const T *>(p.count);
  const T *__restrict__ xs = static_cast<const T *>(p.x);  // APPLY: second operand at the entry's own position
  constexpr int kWarps = kThreads / 32;
  // entries a lane group has in flight.  The apply modes hold an fp32 table row beside every 16-byte pack (eight
  // values on 16-bit data): with four steps the bf16 kernel needs 115 registers and two CTAs fit an SM, with two steps
  // 64.  Measured, scatter_softmax at F=64 (ms; 1 / 2 / 4 / 8 steps): fp32 2.80 / 2.66 / 2.77 / 3.56; bf16 2.61 -> 2.01
  // from four steps to two.
  constexpr int kSteps = APPLY ? 2 : 4;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = 1 << p.l_log2;
  const int col = lane & (L - 1);
  const int sub = lane >> p.l_log2;
  const int eps = 32 >> p.l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t M = p.B * p.E;
  const int64_t base = ((int64_t)blockIdx.x * kWarps + warp) * (32 * kGatherBatches);
  if (base >= M) return;  // warp-uniform

  int64_t srow[kGatherBatches];  // source row (over all batches) of this lane's entry, -1: skip
  unsigned no_row = 0;           // bit q: this lane's entry of batch q exists but its index lies outside [0, N)
#pragma unroll
  for (int q = 0; q < kGatherBatches; ++q) {
    const int64_t ent = base + q * 32 + lane;
    srow[q] = -1;
    if (ent < M) {
      const int64_t b = (p.B == 1) ? 0 : ent / p.E;
      const int64_t idx = p.index[b * p.bstride + (ent - b * p.E)];
      if (idx >= 0 && idx < p.N) srow[q] = b * p.N + idx;
      else no_row |= 1u << q;
    }
  }
#pragma unroll
  for (int q = 0; q < kGatherBatches; ++q) {
    const int64_t ent0 = base + q * 32;
    if (ent0 >= M) break;  // warp-uniform
    for (int64_t cb = 0; cb < Kv; cb += L) {
      const int64_t c = cb + col;
      const bool col_ok = c < Kv;
      for (int i = 0; i < 32; i += kSteps * eps) {
        Row v[kSteps];
        Pack<T, VEC> xv[APPLY ? kSteps : 1];
        int64_t r[kSteps];
#pragma unroll
        for (int u = 0; u < kSteps; ++u) {
          const int m = i + u * eps + sub;  // entry within the batch handled by this lane group
          r[u] = __shfl_sync(kFullMask, (long long)srow[q], m & 31);
          if (m >= 32 || !col_ok) r[u] = -1;
          if (r[u] >= 0) {
            if constexpr (APPLY) {
              v[u] = ld_float_row<VEC>(table + r[u] * p.K + c * VEC);
              xv[u] = ld_stream<T, VEC>(xs + (ent0 + i + u * eps + sub) * p.K + c * VEC);
            } else {
              v[u] = ld_pack<T, VEC>(src + r[u] * p.K + c * VEC);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kSteps; ++u) {
          if (r[u] >= 0) {
            const int64_t at = (ent0 + i + u * eps + sub) * p.K + c * VEC;
            if constexpr (APPLY) {
              Pack<T, VEC> o;
              FloatRow<VEC> w;
              if constexpr (SCALED) w = ld_float_row<VEC>(p.scale + r[u] * p.K + c * VEC);  // the table row's neighbour in time: L1/L2
#pragma unroll
              for (int k = 0; k < VEC; ++k) {
                const float d = (float)to_acc<T>(xv[u].v[k]) - v[u].v[k];
                float y = p.op == 1 ? __expf(d) : (p.op == 3 ? d * d : d);
                if constexpr (SCALED) y *= w.v[k];
                o.v[k] = from_acc<T>((acc_t<T>)y);
              }
              st_stream<T, VEC>(out + at, o);
            } else {
              if (count != nullptr) {
                const T cnt = count[r[u]];
#pragma unroll
                for (int k = 0; k < VEC; ++k) v[u].v[k] = div_t<T>(v[u].v[k], cnt);
              }
              st_stream<T, VEC>(out + at, v[u]);
            }
          }
        }
      }
    }
  }
  // Entries whose index lies outside [0, N) have no source row: they read as zero rather than as whatever the (possibly
  // uninitialised) output held.  Kept out of the loops above: a store among their loads cost the fp32 kernel 20 %.
#pragma unroll
  for (int q = 0; q < kGatherBatches; ++q) {
    const int64_t ent0 = base + q * 32;
    unsigned bad = __ballot_sync(kFullMask, (no_row >> q) & 1u);
    while (bad != 0) {
      const int m = __ffs((int)bad) - 1;
      bad &= bad - 1;
      Pack<T, VEC> zero;
#pragma unroll
      for (int k = 0; k < VEC; ++k) zero.v[k] = from_acc<T>((acc_t<T>)0);
      for (int64_t c = lane; c < Kv; c += 32) st_stream<T, VEC>(out + (ent0 + m) * p.K + c * VEC, zero);
    }
  }
}

template <typename T, int MODE>
int launch_gather_coo(GatherCooParams p, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  const int64_t entries = p.B * p.E;
  if (entries == 0 || p.K == 0 || p.N == 0) return TSB_OK;
  const bool vec_ok = (p.K % kFull == 0) && aligned16(p.src) && aligned16(p.out) && (p.x == nullptr || aligned16(p.x)) &&
                      (p.scale == nullptr || aligned16(p.scale));
  const int64_t Kv = p.K / (vec_ok ? kFull : 1);
  p.l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  const int64_t per_cta = (int64_t)(kThreads / 32) * 32 * kGatherBatches;
  const int64_t blocks = (entries + per_cta - 1) / per_cta;
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  if (vec_ok) gather_coo_kernel<T, kFull, MODE><<<(unsigned)blocks, kThreads, 0, stream>>>(p);
  else gather_coo_kernel<T, 1, MODE><<<(unsigned)blocks, kThreads, 0, stream>>>(p);
  return launch_status();
}

// ---------------------------------------------------------------------------------------------
// grad_in[b, arg[b,n,k], k] = grad_out[b,n,k] where arg < E (grad_in zeroed beforehand).
template <typename T>
__global__ void __launch_bounds__(kThreads)
arg_backward_kernel(const T *__restrict__ grad_out, const int64_t *__restrict__ arg, T *__restrict__ grad_in,
                    int64_t total, int64_t E, int64_t K, int64_t N) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i >= total) return;
  const int64_t a = arg[i];
  if (a < 0 || a >= E) return;
  const int64_t k = i % K;
  const int64_t b = i / (N * K);
  grad_in[(b * E + a) * K + k] = grad_out[i];
}

}  // namespace
}  // namespace tsb

extern "C" int tsb_gather_csr(const void *src, const int64_t *indptr, void *out, int64_t B, int64_t E,
                              int64_t K, int64_t N, int64_t indptr_batch_stride, int dtype,
                              int divide_by_count, tsb_stream_t stream) {
  using namespace tsb;
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (B * N * K == 0 || E == 0) return TSB_OK;
  if (src == nullptr || indptr == nullptr || out == nullptr) return TSB_ERR_ARG;
  if (divide_by_count && dtype_is_integer(dtype)) return TSB_ERR_DTYPE;
  GatherCsrParams p;
  p.src = src; p.indptr = indptr; p.out = out;
  p.B = B; p.E = E; p.K = K; p.N = N; p.bstride = indptr_batch_stride;
  p.l_log2 = p.g_log2 = 0; p.long_len = 1; p.divide = divide_by_count ? 1 : 0;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    return launch_gather_csr<scalar_t>(p, reinterpret_cast<cudaStream_t>(stream));
  });
}

extern "C" int tsb_gather_coo(const void *src, const int64_t *index, void *out, const void *count,
                              int64_t B, int64_t E, int64_t K, int64_t N, int64_t index_batch_stride,
                              int dtype, tsb_stream_t stream) {
  using namespace tsb;
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (B * E * K == 0 || N == 0) return TSB_OK;
  if (src == nullptr || index == nullptr || out == nullptr) return TSB_ERR_ARG;
  if (count != nullptr && dtype_is_integer(dtype)) return TSB_ERR_DTYPE;
  GatherCooParams p;
  p.src = src; p.index = index; p.out = out; p.count = count;
  p.x = nullptr; p.op = 0; p.scale = nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N; p.bstride = index_batch_stride; p.l_log2 = 0;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    return launch_gather_coo<scalar_t, 0>(p, reinterpret_cast<cudaStream_t>(stream));
  });
}

extern "C" int tsb_gather_coo_apply(const void *x, const void *table, const int64_t *index, void *out, int64_t B,
                                    int64_t E, int64_t K, int64_t N, int64_t index_batch_stride, int dtype, int op,
                                    tsb_stream_t stream) {
  return tsb_gather_coo_apply2(x, table, nullptr, index, out, B, E, K, N, index_batch_stride, dtype, op, stream);
}

extern "C" int tsb_gather_coo_apply2(const void *x, const void *table, const void *scale, const int64_t *index, void *out,
                                     int64_t B, int64_t E, int64_t K, int64_t N, int64_t index_batch_stride, int dtype,
                                     int op, tsb_stream_t stream) {
  using namespace tsb;
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (B * E * K == 0 || N == 0) return TSB_OK;
  if (x == nullptr || table == nullptr || index == nullptr || out == nullptr) return TSB_ERR_ARG;
  if (op < 1 || op > 3) return TSB_ERR_REDUCE;
  if (dtype != TSB_F32 && dtype != TSB_F16 && dtype != TSB_BF16) return TSB_ERR_DTYPE;  // computed in fp32
  GatherCooParams p;
  p.src = table; p.index = index; p.out = out; p.count = nullptr;
  p.x = x; p.op = op; p.scale = static_cast<const float *>(scale);
  p.B = B; p.E = E; p.K = K; p.N = N; p.bstride = index_batch_stride; p.l_log2 = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (scale != nullptr) {
    if (dtype == TSB_F32) return launch_gather_coo<float, 2>(p, s);
    if (dtype == TSB_F16) return launch_gather_coo<__half, 2>(p, s);
    return launch_gather_coo<__nv_bfloat16, 2>(p, s);
  }
  if (dtype == TSB_F32) return launch_gather_coo<float, 1>(p, s);
  if (dtype == TSB_F16) return launch_gather_coo<__half, 1>(p, s);
  return launch_gather_coo<__nv_bfloat16, 1>(p, s);
}

extern "C" int tsb_arg_backward(const void *grad_out, const int64_t *arg, void *grad_in, int64_t B,
                                int64_t E, int64_t K, int64_t N, int dtype, tsb_stream_t stream_) {
  using namespace tsb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    const int64_t in_total = B * E * K;
    if (in_total > 0) {
      if (grad_in == nullptr) return TSB_ERR_ARG;
      if (cudaMemsetAsync(grad_in, 0, (size_t)in_total * sizeof(scalar_t), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
    }
    const int64_t total = B * N * K;
    if (total == 0 || in_total == 0) return TSB_OK;
    if (grad_out == nullptr || arg == nullptr) return TSB_ERR_ARG;
    const int64_t blocks = (total + kThreads - 1) / kThreads;
    if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
    arg_backward_kernel<scalar_t><<<(unsigned)blocks, kThreads, 0, stream>>>(
        static_cast<const scalar_t *>(grad_out), arg, static_cast<scalar_t *>(grad_in), total, E, K, N);
    return launch_status();
  });
}

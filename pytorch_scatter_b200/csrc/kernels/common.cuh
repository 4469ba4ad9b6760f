// Shared device/host helpers for the tsb200 kernel library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cmath>
#include <limits>
#include <type_traits>

#include "../../../include/tsb200.h"

namespace tsb {

constexpr int kSum = TSB_SUM, kMean = TSB_MEAN, kMin = TSB_MIN, kMax = TSB_MAX, kMul = TSB_MUL, kLse = TSB_LSE;
constexpr int kThreads = 256;          // CTA size used by every streaming kernel
constexpr unsigned kFullMask = 0xffffffffu;

// ---------------------------------------------------------------------------------------------
// accumulation type: 16-bit floats accumulate in fp32 (csrc/cpu/segment_csr_cpu.cpp:62 uses
// at::opmath_type the same way); everything else accumulates in its own type.
template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<__half> { using type = float; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };
// narrow integers accumulate in int32 (the same result modulo 2^bits as accumulating in the type itself)
template <> struct AccOf<uint8_t> { using type = int32_t; };
template <> struct AccOf<int8_t> { using type = int32_t; };
template <> struct AccOf<int16_t> { using type = int32_t; };
template <typename T> using acc_t = typename AccOf<T>::type;

template <typename T> __host__ __device__ __forceinline__ acc_t<T> to_acc(T v) { return (acc_t<T>)v; }
template <> __host__ __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }
template <> __host__ __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __host__ __device__ __forceinline__ T from_acc(acc_t<T> v) { return (T)v; }
template <> __host__ __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }
template <> __host__ __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Identity of MIN / MAX in the *storage* type T expressed in the accumulation type: the largest /
// lowest finite value of T, not +-inf (csrc/cpu/reducer.h:44-53).
template <typename T> struct Limits {
  __host__ __device__ static constexpr T max() { return std::numeric_limits<T>::max(); }
  __host__ __device__ static constexpr T lowest() { return std::numeric_limits<T>::lowest(); }
};
template <> struct Limits<float> {
  __host__ __device__ static constexpr float max() { return 3.402823466e+38f; }
  __host__ __device__ static constexpr float lowest() { return -3.402823466e+38f; }
};
template <> struct Limits<double> {
  __host__ __device__ static constexpr double max() { return 1.7976931348623157e+308; }
  __host__ __device__ static constexpr double lowest() { return -1.7976931348623157e+308; }
};
template <> struct Limits<int32_t> {
  __host__ __device__ static constexpr int32_t max() { return 2147483647; }
  __host__ __device__ static constexpr int32_t lowest() { return -2147483647 - 1; }
};
template <> struct Limits<int64_t> {
  __host__ __device__ static constexpr int64_t max() { return 9223372036854775807LL; }
  __host__ __device__ static constexpr int64_t lowest() { return -9223372036854775807LL - 1; }
};
template <> struct Limits<__half> {            // as fp32: +-65504
  __host__ __device__ static constexpr float max() { return 65504.0f; }
  __host__ __device__ static constexpr float lowest() { return -65504.0f; }
};
template <> struct Limits<__nv_bfloat16> {     // as fp32: +-0x7f7f0000
  __host__ __device__ static constexpr float max() { return 3.38953139e+38f; }
  __host__ __device__ static constexpr float lowest() { return -3.38953139e+38f; }
};

template <typename T, int REDUCE> __host__ __device__ __forceinline__ acc_t<T> reduce_identity() {
  if (REDUCE == kMin) return (acc_t<T>)Limits<T>::max();
  if (REDUCE == kMax) return (acc_t<T>)Limits<T>::lowest();
  if (REDUCE == kMul) return (acc_t<T>)1;
  if (REDUCE == kLse) {  // running maximum of the online log-sum-exp (floating accumulators only)
    if constexpr (std::is_floating_point<acc_t<T>>::value) return (acc_t<T>)(-3.402823466e+38f);
    else return (acc_t<T>)0;
  }
  return (acc_t<T>)0;
}

// ---------------------------------------------------------------------------------------------
// Packs: VEC consecutive elements moved with one load/store instruction (16 bytes when VEC is the
// full width of the type).
template <typename T, int VEC> struct alignas(sizeof(T) * VEC) Pack { T v[VEC]; };

// (narrow integers move element by element: rare types, not worth sixteen accumulators per lane)
template <typename T> constexpr int full_vec() {
  return (std::is_integral<T>::value && sizeof(T) < 4) ? 1 : 16 / (int)sizeof(T);
}

// Streaming (evict-first) load of a pack: the reductions read src exactly once.
template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> ld_stream(const T *p) {
  Pack<T, VEC> r;
  constexpr int bytes = sizeof(T) * VEC;
  if constexpr (bytes == 16) {
    int4 t = __ldcs(reinterpret_cast<const int4 *>(p));
    r = *reinterpret_cast<Pack<T, VEC> *>(&t);
  } else if constexpr (bytes == 8) {
    int2 t = __ldcs(reinterpret_cast<const int2 *>(p));
    r = *reinterpret_cast<Pack<T, VEC> *>(&t);
  } else if constexpr (bytes == 4) {
    int t = __ldcs(reinterpret_cast<const int *>(p));
    r = *reinterpret_cast<Pack<T, VEC> *>(&t);
  } else if constexpr (bytes == 2) {
    short t = __ldcs(reinterpret_cast<const short *>(p));
    r = *reinterpret_cast<Pack<T, VEC> *>(&t);
  } else {
    r = *reinterpret_cast<const Pack<T, VEC> *>(p);
  }
  return r;
}

// Cached load of a pack (values re-used by neighbouring threads / later kernels).
template <typename T, int VEC> __device__ __forceinline__ Pack<T, VEC> ld_pack(const T *p) {
  return *reinterpret_cast<const Pack<T, VEC> *>(p);
}
template <typename T, int VEC> __device__ __forceinline__ void st_pack(T *p, const Pack<T, VEC> &v) {
  *reinterpret_cast<Pack<T, VEC> *>(p) = v;
}
// Streaming store: written once, not read again by this kernel.
template <typename T, int VEC> __device__ __forceinline__ void st_stream(T *p, const Pack<T, VEC> &v) {
  constexpr int bytes = sizeof(T) * VEC;
  if constexpr (bytes == 16) {
    __stcs(reinterpret_cast<int4 *>(p), *reinterpret_cast<const int4 *>(&v));
  } else if constexpr (bytes == 8) {
    __stcs(reinterpret_cast<int2 *>(p), *reinterpret_cast<const int2 *>(&v));
  } else if constexpr (bytes == 4) {
    __stcs(reinterpret_cast<int *>(p), *reinterpret_cast<const int *>(&v));
  } else {
    *reinterpret_cast<Pack<T, VEC> *>(p) = v;
  }
}

// Asynchronous global -> shared copy of one pack by the calling lane (cp.async; 16-byte packs bypass
// L1).  Packs of less than 4 bytes have no asynchronous form and are copied through a register.
template <typename T, int VEC> __device__ __forceinline__ void async_copy_pack(Pack<T, VEC> *smem_dst, const T *gsrc) {
  constexpr int bytes = sizeof(T) * VEC;
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  if constexpr (bytes == 32) {  // a double pack: two 16-byte copies
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gsrc) : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16), "l"(reinterpret_cast<const char *>(gsrc) + 16) : "memory");
  } else if constexpr (bytes == 16) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gsrc) : "memory");
  } else if constexpr (bytes == 8) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(gsrc) : "memory");
  } else if constexpr (bytes == 4) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(gsrc) : "memory");
  } else {
    *smem_dst = *reinterpret_cast<const Pack<T, VEC> *>(gsrc);
  }
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void async_wait_all_but() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Shuffles for every accumulator type we use.
template <typename A> __device__ __forceinline__ A shfl_xor(A v, int mask) { return __shfl_xor_sync(kFullMask, v, mask); }
template <> __device__ __forceinline__ int64_t shfl_xor<int64_t>(int64_t v, int mask) {
  return (int64_t)__shfl_xor_sync(kFullMask, (long long)v, mask);
}

__host__ __device__ __forceinline__ int64_t clamp64(int64_t v, int64_t lo, int64_t hi) {
  return v < lo ? lo : (v > hi ? hi : v);
}

// ---------------------------------------------------------------------------------------------
// host helpers
inline int ilog2_ceil(int64_t v) {
  int l = 0;
  while (((int64_t)1 << l) < v) ++l;
  return l;
}
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

// element / accumulator sizes of a tsb_dtype
inline size_t dtype_elem_bytes(int dtype) {
  switch (dtype) {
    case TSB_F64: case TSB_I64: return 8;
    case TSB_F16: case TSB_BF16: case TSB_I16: return 2;
    case TSB_U8: case TSB_I8: return 1;
    default: return 4;
  }
}
inline size_t dtype_acc_bytes(int dtype) { return (dtype == TSB_F64 || dtype == TSB_I64) ? 8 : 4; }
inline bool dtype_is_integer(int dtype) { return dtype == TSB_I32 || dtype == TSB_I64 || dtype == TSB_U8 || dtype == TSB_I8 || dtype == TSB_I16; }
inline bool dtype_accumulates_wider(int dtype) {
  return dtype == TSB_F16 || dtype == TSB_BF16 || dtype == TSB_U8 || dtype == TSB_I8 || dtype == TSB_I16;
}

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? TSB_OK : TSB_ERR_LAUNCH; }

inline int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// Dispatch a generic lambda-like macro body over the nine dtypes.
#define TSB_DISPATCH_DTYPE(dtype, ...)                                              \
  [&]() -> int {                                                                    \
    switch (dtype) {                                                                \
      case TSB_F32: { using scalar_t = float; return __VA_ARGS__(); }               \
      case TSB_F64: { using scalar_t = double; return __VA_ARGS__(); }              \
      case TSB_F16: { using scalar_t = __half; return __VA_ARGS__(); }              \
      case TSB_BF16: { using scalar_t = __nv_bfloat16; return __VA_ARGS__(); }      \
      case TSB_I32: { using scalar_t = int32_t; return __VA_ARGS__(); }             \
      case TSB_I64: { using scalar_t = int64_t; return __VA_ARGS__(); }             \
      case TSB_U8: { using scalar_t = uint8_t; return __VA_ARGS__(); }              \
      case TSB_I8: { using scalar_t = int8_t; return __VA_ARGS__(); }               \
      case TSB_I16: { using scalar_t = int16_t; return __VA_ARGS__(); }             \
      default: return TSB_ERR_DTYPE;                                                \
    }                                                                               \
  }()

}  // namespace tsb

// segment_coo for sm_100a: reduction keyed by a sorted index.
//
// The sorted index is first turned back into row pointers by one streaming pass (each thread looks
// at one index entry and its predecessor; a run boundary writes the row starts it uncovers), then
// the row-pointer reduction of segment_csr.cu does the arithmetic with the COO write rules.  The
// extra traffic is N+1 row pointers written and read once; in exchange the reduction is free of
// atomics, deterministic, balanced over long runs, and MIN/MAX get their arg index in the same pass
// with the first-occurrence tie-break of the CPU loop (csrc/cpu/segment_coo_cpu.cpp:96-128).
//
// Replaces segment_coo_kernel, segment_coo_broadcast_kernel and the two arg kernels of the upstream
// project (csrc/cuda/segment_coo_cuda.cu:14-150), which issue an atomic per run end and per chunk end
// and find arg indices in a second, racy pass.
#include "csr_reduce.cuh"

namespace tsb {
namespace {

// rowptr[r] = first position e with index[e] >= r, for r in [0, N]; equals E when no such e.
// A thread looks at kRowptrItems consecutive entries of one batch (and the entry before them).
constexpr int kRowptrItems = 4;

__global__ void __launch_bounds__(kThreads)
coo_rowptr_kernel(const int64_t *__restrict__ index, int64_t *__restrict__ rowptr, int64_t B, int64_t E,
                  int64_t N, int64_t bstride) {
  const int64_t per_batch = (E + kRowptrItems - 1) / kRowptrItems;  // threads per batch
  const int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (t >= B * per_batch) return;
  const int64_t b = (B == 1) ? 0 : t / per_batch;
  const int64_t e0 = (t - b * per_batch) * kRowptrItems;
  const int64_t *ix = index + b * bstride;
  int64_t *rp = rowptr + b * (N + 1);
  int64_t v[kRowptrItems + 1];
  v[0] = e0 > 0 ? ix[e0 - 1] : -1;
#pragma unroll
  for (int j = 0; j < kRowptrItems; ++j) v[j + 1] = e0 + j < E ? ix[e0 + j] : v[j];  // past the end: no new run
#pragma unroll
  for (int j = 0; j < kRowptrItems; ++j) {
    const int64_t e = e0 + j;
    if (e >= E) break;
    const int64_t cur = v[j + 1], prev = v[j];
    if (cur > prev) {
      const int64_t lo = prev + 1 > 0 ? prev + 1 : 0;
      const int64_t hi = cur < N ? cur : N;
      for (int64_t r = lo; r <= hi; ++r) rp[r] = e;
    }
    if (e == E - 1) {
      const int64_t lo = cur + 1 > 0 ? cur + 1 : 0;
      for (int64_t r = lo; r <= N; ++r) rp[r] = E;
    }
  }
}

// *unsorted = 1 if some entry is smaller than its predecessor (the flag must be zero beforehand)
__global__ void __launch_bounds__(kThreads)
index_unsorted_kernel(const int64_t *__restrict__ index, int64_t n, int *unsorted) {
  const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (i + 1 < n && index[i] > index[i + 1]) *unsorted = 1;
}

}  // namespace
}  // namespace tsb

namespace {
size_t rowptr_bytes(int64_t B, int64_t N) {
  return (((size_t)B * (size_t)(N + 1) * sizeof(int64_t)) + 255) & ~(size_t)255;
}
}  // namespace

extern "C" size_t tsb_segment_coo_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  if (B < 0 || N < 0 || E < 0 || K < 0) return 0;
  return rowptr_bytes(B, N) + tsb::csr_reduce_workspace_bytes(B, E, K, N, dtype, reduce);
}

extern "C" int tsb_segment_coo(const void *src, const int64_t *index, void *out, int64_t *arg_out,
                               void *count_out, int64_t B, int64_t E, int64_t K, int64_t N,
                               int64_t index_batch_stride, int dtype, int reduce, int out_seeded,
                               void *workspace, size_t workspace_bytes, tsb_stream_t stream_) {
  using namespace tsb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (B < 0 || E < 0 || K < 0 || N < 0) return TSB_ERR_ARG;
  if (reduce == TSB_LSE && out_seeded) return TSB_ERR_ARG;
  if (B * N == 0) return TSB_OK;
  if (workspace == nullptr || workspace_bytes < tsb_segment_coo_workspace_bytes(B, E, K, N, dtype, reduce)) return TSB_ERR_WORKSPACE;
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return TSB_ERR_WORKSPACE;
  if (E > 0 && index == nullptr) return TSB_ERR_ARG;
  int64_t *rowptr = static_cast<int64_t *>(workspace);
  if (E == 0) {
    if (cudaMemsetAsync(rowptr, 0, rowptr_bytes(B, N), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
  } else {
    const int64_t blocks = (B * ((E + kRowptrItems - 1) / kRowptrItems) + kThreads - 1) / kThreads;
    if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
    coo_rowptr_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(index, rowptr, B, E, N, index_batch_stride);
    if (launch_status() != TSB_OK) return TSB_ERR_LAUNCH;
  }
  CsrParams p;
  p.src = src;
  p.indptr = rowptr;
  p.out = out;
  p.arg_out = arg_out;
  p.count_out = (reduce == TSB_MEAN) ? count_out : nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.bstride = N + 1;
  p.mode = out_seeded ? kCooSeeded : kCooFresh;
  p.workspace = static_cast<unsigned char *>(workspace) + rowptr_bytes(B, N);
  p.workspace_bytes = workspace_bytes - rowptr_bytes(B, N);
  return launch_csr_reduce(p, dtype, reduce, stream);
}

extern "C" int tsb_index_unsorted(const int64_t *index, int64_t n, int *unsorted_flag, tsb_stream_t stream_) {
  using namespace tsb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (n < 0 || unsorted_flag == nullptr || (n > 0 && index == nullptr)) return TSB_ERR_ARG;
  if (cudaMemsetAsync(unsorted_flag, 0, sizeof(int), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
  if (n < 2) return TSB_OK;
  const int64_t blocks = (n + kThreads - 1) / kThreads;
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  index_unsorted_kernel<<<(unsigned)blocks, kThreads, 0, stream>>>(index, n, unsorted_flag);
  return launch_status();
}

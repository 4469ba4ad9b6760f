// scatter with a large output, without atomics on the output: group the entry ids by target row
// (a counting sort of the index alone: 12 bytes of scratch traffic per entry), then reduce every row
// with the row-pointer streaming kernel reading the source through that permutation.
//
// Why: reductions into an output larger than L2 through red.global pay for every output line twice
// or more (fetched, evicted, fetched again) or re-read the index once per output slice; here the
// source is read once (row-sized random reads), the output is written once, the traffic does not
// depend on the output size, 16-bit sources accumulate in fp32 registers instead of an fp32 copy of
// the output, and MIN/MAX find value and arg in the same single pass.
//
//   1. group_rank_kernel    rank[e] = how many entries naming the same row arrived before e
//                           (atomicAdd on a counter per row; the counters double as MEAN's count)
//   2. three small kernels  exclusive scan of the counters -> row pointers (int64)
//   3. group_place_kernel   perm[rowptr[index[e]] + rank[e]] = e
//   4. launch_csr_reduce    with CsrParams::perm
// The order of the entries inside a row depends on the arrival order of the atomics: float sums are
// as (non-)reproducible as the upstream atomics; MIN/MAX args break ties towards the smaller entry
// id explicitly, as the upstream CPU loop does implicitly (csrc/cpu/scatter_cpu.cpp:63-82).
//
// Replaces, for this regime, scatter_kernel + scatter_arg_kernel of the upstream project
// (csrc/cuda/scatter_cuda.cu:13-56).
#include "scatter_grouped.cuh"

#include <cstdlib>

namespace tsb {
namespace {

constexpr int kScanItems = 8;                       // counters per thread in the scan kernels
constexpr int kScanTile = kThreads * kScanItems;    // counters per CTA

__global__ void __launch_bounds__(kThreads)
group_rank_kernel(const int64_t *__restrict__ index, int64_t E, int64_t N, int32_t *__restrict__ count,
                  int32_t *__restrict__ rank) {
  const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (e >= E) return;
  const int64_t t = __ldcs(index + e);
  rank[e] = (t >= 0 && t < N) ? atomicAdd(count + t, 1) : -1;  // -1: the entry names no row and is dropped
}

__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *total) {
  __shared__ int64_t s_warp[kThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t incl = v;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int64_t o = __shfl_up_sync(kFullMask, incl, off);
    if (lane >= off) incl += o;
  }
  if (lane == 31) s_warp[warp] = incl;
  __syncthreads();
  int64_t before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) {
    if (w < warp) before += s_warp[w];
    all += s_warp[w];
  }
  __syncthreads();  // s_warp may be reused by the caller's next scan
  *total = all;
  return before + incl - v;
}

// tile_sum[b] = sum of the counters of tile b
__global__ void __launch_bounds__(kThreads)
scan_tile_sums_kernel(const int32_t *__restrict__ count, int64_t N, int64_t *__restrict__ tile_sum) {
  const int64_t first = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  int64_t v = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i)
    if (first + i < N) v += count[first + i];
  int64_t total;
  block_exclusive_scan(v, &total);
  if (threadIdx.x == 0) tile_sum[blockIdx.x] = total;
}

// in place: tile_sum[b] = sum of the tiles before b (one CTA walks all tiles, kThreads at a time)
__global__ void __launch_bounds__(kThreads) scan_tile_offsets_kernel(int64_t *tile_sum, int64_t tiles) {
  int64_t carry = 0;
  for (int64_t base = 0; base < tiles; base += kThreads) {
    const int64_t i = base + threadIdx.x;
    const int64_t v = i < tiles ? tile_sum[i] : 0;
    int64_t total;
    const int64_t excl = block_exclusive_scan(v, &total);
    if (i < tiles) tile_sum[i] = carry + excl;
    carry += total;
  }
}

// rowptr[i] = tile offset + exclusive scan inside the tile; rowptr[N] = everything
__global__ void __launch_bounds__(kThreads)
scan_rowptr_kernel(const int32_t *__restrict__ count, int64_t N, const int64_t *__restrict__ tile_off,
                   int64_t *__restrict__ rowptr) {
  const int64_t first = (int64_t)blockIdx.x * kScanTile + (int64_t)threadIdx.x * kScanItems;
  int32_t c[kScanItems];
  int64_t v = 0;
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    c[i] = first + i < N ? count[first + i] : 0;
    v += c[i];
  }
  int64_t total;
  int64_t run = tile_off[blockIdx.x] + block_exclusive_scan(v, &total);
#pragma unroll
  for (int i = 0; i < kScanItems; ++i) {
    if (first + i < N) rowptr[first + i] = run;
    run += c[i];
    if (first + i == N - 1) rowptr[N] = run;
  }
}

__global__ void __launch_bounds__(kThreads)
group_place_kernel(const int64_t *__restrict__ index, int64_t E, const int32_t *__restrict__ rank,
                   const int64_t *__restrict__ rowptr, int32_t *__restrict__ perm) {
  const int64_t e = (int64_t)blockIdx.x * kThreads + threadIdx.x;
  if (e >= E) return;
  const int32_t r = __ldcs(rank + e);
  if (r < 0) return;
  perm[rowptr[__ldcs(index + e)] + r] = (int32_t)e;
}

size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

struct GroupedLayout {
  size_t count, rank, rowptr, perm, tiles, csr, total;
};
GroupedLayout layout_for(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  GroupedLayout l;
  size_t off = 0;
  l.count = off;  off += up256((size_t)N * sizeof(int32_t));
  l.rank = off;   off += up256((size_t)E * sizeof(int32_t));
  l.rowptr = off; off += up256((size_t)(N + 1) * sizeof(int64_t));
  l.perm = off;   off += up256((size_t)E * sizeof(int32_t));
  l.tiles = off;  off += up256((size_t)((N + kScanTile - 1) / kScanTile + 1) * sizeof(int64_t));
  l.csr = off;    off += up256(csr_reduce_workspace_bytes(B, E, K, N, dtype, reduce));
  l.total = off;
  return l;
}

}  // namespace

bool scatter_grouped_possible(int64_t B, int64_t E, int64_t K, int64_t N, int64_t sb, int64_t se, int64_t sk,
                              int dtype, int reduce) {
  if (reduce != TSB_SUM && reduce != TSB_MEAN && reduce != TSB_MIN && reduce != TSB_MAX) return false;
  // the CSR mean truncates integers, upstream's scatter_mean floors them (torch_scatter/scatter.py:65)
  if (reduce == TSB_MEAN && (dtype == TSB_I32 || dtype == TSB_I64)) return false;
  if (sk != 0 || (E > 1 && se != 1) || (B > 1 && sb != 0)) return false;  // one index entry per source row, shared by the batches
  return B >= 1 && K >= 1 && N >= 1 && E >= 1 && E < (1ll << 30) && N < (1ll << 31) - 1;
}

size_t scatter_grouped_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  if (B < 1 || E < 1 || K < 1 || N < 1 || E >= (1ll << 30)) return 0;
  return layout_for(B, E, K, N, dtype, reduce).total;
}

int run_scatter_grouped(const void *src, const int64_t *index, void *out, int64_t *arg_out, int32_t *count_out,
                        int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce, int out_seeded,
                        void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  const GroupedLayout l = layout_for(B, E, K, N, dtype, reduce);
  if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return TSB_ERR_WORKSPACE;
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  int32_t *count = (reduce == TSB_MEAN && count_out != nullptr) ? count_out : reinterpret_cast<int32_t *>(ws + l.count);
  int32_t *rank = reinterpret_cast<int32_t *>(ws + l.rank);
  int64_t *rowptr = reinterpret_cast<int64_t *>(ws + l.rowptr);
  int32_t *perm = reinterpret_cast<int32_t *>(ws + l.perm);
  int64_t *tiles = reinterpret_cast<int64_t *>(ws + l.tiles);

  const int64_t entry_blocks = (E + kThreads - 1) / kThreads;
  const int64_t n_tiles = (N + kScanTile - 1) / kScanTile;
  if (entry_blocks > 2147483647LL || n_tiles > 2147483647LL) return TSB_ERR_TOO_LARGE;
  if (cudaMemsetAsync(count, 0, (size_t)N * sizeof(int32_t), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
  group_rank_kernel<<<(unsigned)entry_blocks, kThreads, 0, stream>>>(index, E, N, count, rank);
  scan_tile_sums_kernel<<<(unsigned)n_tiles, kThreads, 0, stream>>>(count, N, tiles);
  scan_tile_offsets_kernel<<<1, kThreads, 0, stream>>>(tiles, n_tiles);
  scan_rowptr_kernel<<<(unsigned)n_tiles, kThreads, 0, stream>>>(count, N, tiles, rowptr);
  group_place_kernel<<<(unsigned)entry_blocks, kThreads, 0, stream>>>(index, E, rank, rowptr, perm);
  if (launch_status() != TSB_OK) return TSB_ERR_LAUNCH;

  CsrParams p;
  p.src = src;
  p.indptr = rowptr;
  p.out = out;
  p.arg_out = arg_out;
  p.count_out = nullptr;
  p.B = B; p.E = E; p.K = K; p.N = N;
  p.bstride = 0;  // one set of row pointers for every batch
  p.perm = perm;
  p.mode = out_seeded ? kCooSeeded : kCooFresh;
  p.workspace = ws + l.csr;
  p.workspace_bytes = workspace_bytes - l.csr;
  return launch_csr_reduce(p, dtype, reduce, stream);
}

}  // namespace tsb

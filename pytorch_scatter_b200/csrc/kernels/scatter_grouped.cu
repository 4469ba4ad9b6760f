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

#include <atomic>
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

template <int THREADS = kThreads>
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *total) {
  __shared__ int64_t s_warp[THREADS / 32];
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
  for (int w = 0; w < THREADS / 32; ++w) {
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


// ---------------------------------------------------------------------------------------------
// The same grouping with shared-memory counters instead of one global atomic per entry.
// Global atomics on random addresses run at some 100 G/s here, so the three random accesses per entry
// of the kernels above (counter, row pointer, permutation slot) cost more than a third of the whole
// scatter.  Two levels remove them:
//   A  bucket_hist_kernel       rows are cut into P buckets of R = 2^shift rows; per-CTA histogram
//                               of the entries over buckets in shared memory, then P global adds
//   -  bucket_scan_kernel       exclusive scan -> first slot of every bucket
//   B  bucket_partition_kernel  a CTA sorts a tile of 16384 entries by bucket in shared memory (rank
//                               from a shared-memory atomic), reserves its share of every bucket
//                               with one global add per bucket, writes (entry, row) pairs in runs
//   C  bucket_finalize_kernel   one CTA per bucket: row counters and cursors in shared memory,
//                               row pointers out, the bucket's slice of the permutation staged in
//                               shared memory and written coalesced
// Traffic: the index twice, the pairs written once and read twice (mostly from L2), permutation and
// row pointers once.
constexpr int kPartThreads = 1024;   // a tile of the partition kernel is 16 entries per thread: 512 threads (twice the tiles) took twice as long
constexpr int kFinalThreads = 512;   // (1024 threads, full occupancy: 90.6 us against 93)
constexpr int kMaxBuckets = 4096;
constexpr int kMaxBucketRows = 16384;
constexpr int kStageEntries = 49152;  // most permutation slots kernel C stages in shared memory (192 KiB)
constexpr int kFinalSmemInts = 56832; // rows + staged slots of kernel C (222 KiB)

__global__ void __launch_bounds__(kThreads)
bucket_hist_kernel(const int64_t *__restrict__ index, int64_t E, int64_t N, int shift, int P, int32_t *__restrict__ hist) {
  extern __shared__ int s_hist[];
  for (int b = threadIdx.x; b < P; b += kThreads) s_hist[b] = 0;
  __syncthreads();
  const int64_t first = (int64_t)blockIdx.x * (kThreads * 64);
  for (int j0 = 0; j0 < 64; j0 += 8) {  // eight independent loads in flight, then their eight updates
    int64_t t[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int64_t e = first + (int64_t)(j0 + j) * kThreads + threadIdx.x;
      t[j] = e < E ? __ldcs(index + e) : -1;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (t[j] >= 0 && t[j] < N) atomicAdd(&s_hist[(int)(t[j] >> shift)], 1);
  }
  __syncthreads();
  for (int b = threadIdx.x; b < P; b += kThreads)
    if (s_hist[b] != 0) atomicAdd(hist + b, s_hist[b]);
}

// start[q] = entries in the Q buckets before q, start[Q] = all valid entries; cursor[q] = 0.  One CTA: thread t owns a
// run of consecutive buckets.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
bucket_scan_kernel(const int32_t *__restrict__ hist, int Q, int32_t *__restrict__ start, int32_t *__restrict__ cursor) {
  const int per = (Q + kScanThreads - 1) / kScanThreads;
  const int q0 = threadIdx.x * per;
  int64_t v = 0;
  for (int i = 0; i < per; ++i)
    if (q0 + i < Q) v += hist[q0 + i];
  int64_t total;
  int64_t run = block_exclusive_scan<kScanThreads>(v, &total);
  for (int i = 0; i < per; ++i) {
    const int q = q0 + i;
    if (q < Q) {
      start[q] = (int32_t)run;
      cursor[q] = 0;
      run += hist[q];
    }
  }
  if (threadIdx.x == 0) start[Q] = (int32_t)total;
}

template <int kPartItems>  // entries per thread
__global__ void __launch_bounds__(kPartThreads)
bucket_partition_kernel(const int64_t *__restrict__ index, int64_t E, int64_t N, int shift, int P,
                        const int32_t *__restrict__ start, int32_t *__restrict__ cursor, int2 *__restrict__ pairs) {
  extern __shared__ int s_part[];
  int *s_cnt = s_part;            // entries of this tile per bucket
  int *s_off = s_part + P;        // first staging slot of the bucket
  int *s_dst = s_part + 2 * P;    // first global slot this tile got in the bucket
  int2 *s_pairs = reinterpret_cast<int2 *>(s_part + 3 * P + (P & 1));  // 8-byte aligned
  for (int b = threadIdx.x; b < P; b += kPartThreads) s_cnt[b] = 0;
  __syncthreads();
  constexpr int kPartTile = kPartThreads * kPartItems;
  const int64_t first = (int64_t)blockIdx.x * kPartTile;
  int row[kPartItems], rank[kPartItems];
  constexpr int kBatch = kPartItems < 8 ? kPartItems : 8;  // independent loads in flight, then their updates
#pragma unroll
  for (int j0 = 0; j0 < kPartItems; j0 += kBatch) {
    int64_t t[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int64_t e = first + (int64_t)(j0 + j) * kPartThreads + threadIdx.x;
      t[j] = e < E ? __ldcs(index + e) : -1;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const bool ok = t[j] >= 0 && t[j] < N;
      row[j0 + j] = ok ? (int)t[j] : -1;
      rank[j0 + j] = ok ? atomicAdd(&s_cnt[(int)(t[j] >> shift)], 1) : 0;
    }
  }
  __syncthreads();
  {  // exclusive scan of the tile's bucket counts; reserve the tile's slots in every bucket it feeds
    constexpr int kItems = kMaxBuckets / kPartThreads;
    int c[kItems];
    int64_t v = 0;
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
      const int b = threadIdx.x * kItems + i;
      c[i] = b < P ? s_cnt[b] : 0;
      v += c[i];
    }
    int64_t total;
    int run = (int)block_exclusive_scan<kPartThreads>(v, &total);
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
      const int b = threadIdx.x * kItems + i;
      if (b < P) {
        s_off[b] = run;
        // (handing a bucket's slots out through 8 counters instead of one, to shorten the queue of a thousand tiles on
        // every counter, measured no faster: this kernel 104 vs 102 us, the histogram and the scan 18 us slower)
        if (c[i] != 0) s_dst[b] = start[b] + atomicAdd(cursor + b, c[i]);
      }
      run += c[i];
    }
    if (threadIdx.x == 0) s_cnt[0] = (int)total;  // s_cnt is free again: keep the tile's valid count
  }
  __syncthreads();
  const int valid = s_cnt[0];
#pragma unroll
  for (int j = 0; j < kPartItems; ++j) {
    if (row[j] >= 0) {
      const int64_t e = first + (int64_t)j * kPartThreads + threadIdx.x;
      s_pairs[s_off[row[j] >> shift] + rank[j]] = make_int2((int)e, row[j]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < valid; i += kPartThreads) {
    const int2 pr = s_pairs[i];
    const int b = pr.y >> shift;
    pairs[s_dst[b] + (i - s_off[b])] = pr;
  }
}

__global__ void __launch_bounds__(kFinalThreads)
bucket_finalize_kernel(const int2 *__restrict__ pairs, const int32_t *__restrict__ start, int64_t N, int shift, int P,
                       int32_t *__restrict__ perm, int64_t *__restrict__ rowptr, int32_t *__restrict__ count_out,
                       int stage_entries) {
  extern __shared__ int s_fin[];
  const int R = 1 << shift;
  int *s_rows = s_fin;       // per row of the bucket: count, then first slot, then cursor
  int *s_perm = s_fin + R;   // the bucket's slice of the permutation, when it fits
  const int b = blockIdx.x;
  const int lo = start[b];
  const int n = start[b + 1] - lo;
  const int64_t row0 = (int64_t)b << shift;
  for (int j = threadIdx.x; j < R; j += kFinalThreads) s_rows[j] = 0;
  __syncthreads();
  constexpr int kBatch = 8;  // independent loads in flight, then their updates
  for (int i0 = 0; i0 < n; i0 += kBatch * kFinalThreads) {
    int y[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + j * kFinalThreads + threadIdx.x;
      y[j] = i < n ? pairs[lo + i].y : -1;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
      if (y[j] >= 0) atomicAdd(&s_rows[y[j] - (int)row0], 1);
  }
  __syncthreads();
  {  // exclusive scan over the R rows: thread t owns rows [t * per, t * per + per)
    const int per = (R + kFinalThreads - 1) / kFinalThreads;
    const int j0 = threadIdx.x * per;
    int64_t v = 0;
    for (int i = 0; i < per; ++i)
      if (j0 + i < R) v += s_rows[j0 + i];
    int64_t total;
    int run = (int)block_exclusive_scan<kFinalThreads>(v, &total);
    for (int i = 0; i < per; ++i) {
      const int j = j0 + i;
      if (j < R) {
        const int c = s_rows[j];
        s_rows[j] = run;
        if (row0 + j < N) {
          rowptr[row0 + j] = (int64_t)lo + run;
          if (count_out != nullptr) count_out[row0 + j] = c;
        }
        run += c;
      }
    }
    if (b == P - 1 && threadIdx.x == 0) rowptr[N] = (int64_t)lo + n;
  }
  __syncthreads();
  const bool staged = n <= stage_entries;
  for (int i0 = 0; i0 < n; i0 += kBatch * kFinalThreads) {
    int2 pr[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int i = i0 + j * kFinalThreads + threadIdx.x;
      pr[j] = i < n ? pairs[lo + i] : make_int2(0, -1);
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      if (pr[j].y < 0) continue;
      const int slot = atomicAdd(&s_rows[pr[j].y - (int)row0], 1);
      if (staged) s_perm[slot] = pr[j].x;
      else perm[lo + slot] = pr[j].x;
    }
  }
  if (!staged) return;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += kFinalThreads) perm[lo + i] = s_perm[i];
}

// Bucket geometry: 12k to 24k entries per bucket on average, so that nearly every bucket's slice of the
// permutation fits the shared-memory stage.  shift < 0: the shapes do not fit (too many rows for
// kMaxBuckets buckets of kMaxBucketRows rows) and the global-atomic kernels are used.
struct BucketGeom { int shift, P; };
constexpr int kBucketEntries = 12288;  // entries a bucket should hold at least (measured, whole scatter: 3k 1.059 ms, 6k 1.034, 12k 1.026, 24k 1.110)
BucketGeom bucket_geom(int64_t E, int64_t N) {
  const int64_t want = ((int64_t)kBucketEntries * N) / (E > 0 ? E : 1);  // rows holding that many entries
  int shift = 6;
  while ((1ll << shift) < want && (1 << shift) < kMaxBucketRows) ++shift;  // rounded up to a power of two
  while (((N + (1ll << shift) - 1) >> shift) > kMaxBuckets && (1 << shift) < kMaxBucketRows) ++shift;
  const int64_t P = (N + (1ll << shift) - 1) >> shift;
  if (P > kMaxBuckets) return BucketGeom{-1, 0};
  return BucketGeom{shift, (int)P};
}

// Shared memory above the 48 KiB default has to be allowed per kernel and device, once.
int allow_bucket_smem() {
  static std::atomic<bool> done[64];  // per device; setting the attributes twice is harmless
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TSB_ERR_LAUNCH;
  if (done[dev]) return TSB_OK;
  const int part = (3 * kMaxBuckets + 1) * (int)sizeof(int);
  const int fin = kFinalSmemInts * (int)sizeof(int);
  if (cudaFuncSetAttribute(bucket_partition_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, part + 16 * kPartThreads * (int)sizeof(int2)) != cudaSuccess ||
      cudaFuncSetAttribute(bucket_finalize_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fin) != cudaSuccess)
    return TSB_ERR_LAUNCH;
  done[dev] = true;
  return TSB_OK;
}

size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

struct GroupedLayout {
  size_t count, rowptr, perm, group, csr, total;
};
size_t group_scratch_bytes(int64_t E, int64_t N);
GroupedLayout layout_for(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  GroupedLayout l;
  size_t off = 0;
  l.count = off;  off += up256((size_t)N * sizeof(int32_t));
  l.rowptr = off; off += up256((size_t)(N + 1) * sizeof(int64_t));
  l.perm = off;   off += up256((size_t)E * sizeof(int32_t));
  l.group = off;  off += up256(group_scratch_bytes(E, N));
  l.csr = off;    off += up256(csr_reduce_workspace_bytes(B, E, K, N, dtype, reduce));
  l.total = off;
  return l;
}

}  // namespace

bool scatter_grouped_possible(int64_t B, int64_t E, int64_t K, int64_t N, int64_t sb, int64_t se, int64_t sk,
                              int dtype, int reduce) {
  if (reduce != TSB_SUM && reduce != TSB_MEAN && reduce != TSB_MIN && reduce != TSB_MAX && reduce != TSB_MUL) return false;
  // the CSR mean truncates integers, upstream's scatter_mean floors them (torch_scatter/scatter.py:65)
  if (reduce == TSB_MEAN && dtype_is_integer(dtype)) return false;
  if (sk != 0 || (E > 1 && se != 1) || (B > 1 && sb != 0)) return false;  // one index entry per source row, shared by the batches
  return B >= 1 && K >= 1 && N >= 1 && E >= 1 && E < (1ll << 30) && N < (1ll << 31) - 1;
}

size_t scatter_grouped_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  if (B < 1 || E < 1 || K < 1 || N < 1 || E >= (1ll << 30)) return 0;
  return layout_for(B, E, K, N, dtype, reduce).total;
}

namespace {
struct GroupScratch { size_t pairs, tiles, total; };
GroupScratch group_scratch(int64_t E, int64_t N);
size_t group_scratch_bytes(int64_t E, int64_t N) { return group_scratch(E, N).total; }
GroupScratch group_scratch(int64_t E, int64_t N) {
  GroupScratch l;
  size_t off = 0;
  l.pairs = off; off += up256((size_t)E * sizeof(int2));  // ranks (global-atomic kernels) or (entry, row) pairs
  l.tiles = off; off += up256((size_t)((N + kScanTile - 1) / kScanTile + 1) * sizeof(int64_t) + (size_t)(3 * kMaxBuckets + 1) * sizeof(int32_t));
  l.total = off;
  return l;
}
}  // namespace

size_t scatter_group_workspace_bytes(int64_t E, int64_t N) {
  if (E < 1 || N < 1 || E >= (1ll << 30)) return 256;
  return group_scratch(E, N).total;
}

// rowptr [N+1], perm [E] (its first rowptr[N] slots are meaningful), count [N] or null.
int scatter_group(const int64_t *index, int64_t E, int64_t N, int64_t *rowptr, int32_t *perm, int32_t *count,
                  void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  if (E < 1 || N < 1 || E >= (1ll << 30) || N >= (1ll << 31) - 1) return TSB_ERR_TOO_LARGE;
  const GroupScratch l = group_scratch(E, N);
  if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return TSB_ERR_WORKSPACE;
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  int32_t *rank = reinterpret_cast<int32_t *>(ws + l.pairs);
  int64_t *tiles = reinterpret_cast<int64_t *>(ws + l.tiles);

  const char *sort_env = std::getenv("TSB_SCATTER_GROUPED_SORT");  // test hook: "atomic" forces the global-atomic kernels
  BucketGeom geom = (sort_env != nullptr && sort_env[0] == 'a') ? BucketGeom{-1, 0} : bucket_geom(E, N);
  if (geom.shift < 0 && count == nullptr) return TSB_ERR_ARG;  // the global-atomic kernels need a counter per row
  if (geom.shift >= 0) {
    const int st = allow_bucket_smem();
    if (st != TSB_OK) return st;
    int32_t *hist = reinterpret_cast<int32_t *>(tiles);
    int32_t *start = hist + kMaxBuckets;
    int32_t *cursor = start + kMaxBuckets + 1;
    int2 *pairs = reinterpret_cast<int2 *>(rank);
    const int P = geom.P, R = 1 << geom.shift;
    const int64_t hist_blocks = (E + kThreads * 64 - 1) / (kThreads * 64);
    constexpr int part_items = 16;
    const int part_tile = kPartThreads * part_items;   // the histogram kernel's tiles are the same 16384 entries
    const int64_t part_blocks = (E + part_tile - 1) / part_tile;
    if (cudaMemsetAsync(hist, 0, (size_t)P * sizeof(int32_t), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
    bucket_hist_kernel<<<(unsigned)hist_blocks, kThreads, (size_t)P * sizeof(int), stream>>>(index, E, N, geom.shift, P, hist);
    bucket_scan_kernel<<<1, kScanThreads, 0, stream>>>(hist, P, start, cursor);
    const size_t part_smem = (size_t)(3 * P + (P & 1)) * sizeof(int) + (size_t)part_tile * sizeof(int2);
    bucket_partition_kernel<part_items><<<(unsigned)part_blocks, kPartThreads, part_smem, stream>>>(index, E, N, geom.shift, P, start, cursor, pairs);
    // staged permutation slots per bucket: one and a half times the average bucket, so that small buckets leave room for
    // more CTAs per SM (the kernel is a chain of short dependent phases: residency is what hides them)
    int stage = (int)(((E / P) * 3 / 2 + 1023) / 1024) * 1024;
    if (stage < 4096) stage = 4096;
    if (stage > 24576) stage = 24576;
    if (stage > kStageEntries) stage = kStageEntries;
    if (stage > kFinalSmemInts - R) stage = kFinalSmemInts - R;
    const size_t fin_smem = (size_t)(R + stage) * sizeof(int);
    bucket_finalize_kernel<<<(unsigned)P, kFinalThreads, fin_smem, stream>>>(pairs, start, N, geom.shift, P, perm, rowptr, count, stage);
  } else {
    const int64_t entry_blocks = (E + kThreads - 1) / kThreads;
    const int64_t n_tiles = (N + kScanTile - 1) / kScanTile;
    if (entry_blocks > 2147483647LL || n_tiles > 2147483647LL) return TSB_ERR_TOO_LARGE;
    if (cudaMemsetAsync(count, 0, (size_t)N * sizeof(int32_t), stream) != cudaSuccess) return TSB_ERR_LAUNCH;
    group_rank_kernel<<<(unsigned)entry_blocks, kThreads, 0, stream>>>(index, E, N, count, rank);
    scan_tile_sums_kernel<<<(unsigned)n_tiles, kThreads, 0, stream>>>(count, N, tiles);
    scan_tile_offsets_kernel<<<1, kThreads, 0, stream>>>(tiles, n_tiles);
    scan_rowptr_kernel<<<(unsigned)n_tiles, kThreads, 0, stream>>>(count, N, tiles, rowptr);
    group_place_kernel<<<(unsigned)entry_blocks, kThreads, 0, stream>>>(index, E, rank, rowptr, perm);
  }
  return launch_status();
}

int run_scatter_grouped(const void *src, const int64_t *index, void *out, int64_t *arg_out, int32_t *count_out,
                        int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce, int out_seeded,
                        void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  const GroupedLayout l = layout_for(B, E, K, N, dtype, reduce);
  if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255u))
    return TSB_ERR_WORKSPACE;
  unsigned char *ws = static_cast<unsigned char *>(workspace);
  int32_t *count = (reduce == TSB_MEAN && count_out != nullptr) ? count_out : reinterpret_cast<int32_t *>(ws + l.count);
  int64_t *rowptr = reinterpret_cast<int64_t *>(ws + l.rowptr);
  int32_t *perm = reinterpret_cast<int32_t *>(ws + l.perm);
  const int st = scatter_group(index, E, N, rowptr, perm, count, ws + l.group, l.csr - l.group, stream);
  if (st != TSB_OK) return st;

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

namespace tsb {
namespace {
// out[i] = sum over q of slabs[q * elems + i], accumulated in acc_t<T> (fp32 for 16-bit), 16 bytes of slab per thread.
// S is the slabs' element type: T, or acc_t<T> when the partial sums travelled in accumulation precision.
template <typename S, typename T, int VEC>
__global__ void __launch_bounds__(kThreads) sum_slabs_kernel(const S *__restrict__ slabs, T *__restrict__ out, int world, int64_t elems) {
  const int64_t i = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * VEC;
  if (i >= elems) return;
  acc_t<T> acc[VEC];
#pragma unroll
  for (int k = 0; k < VEC; ++k) acc[k] = (acc_t<T>)0;
  for (int q = 0; q < world; ++q) {
    const Pack<S, VEC> v = ld_stream<S, VEC>(slabs + (int64_t)q * elems + i);
#pragma unroll
    for (int k = 0; k < VEC; ++k) acc[k] += (acc_t<T>)to_acc<S>(v.v[k]);
  }
  Pack<T, VEC> o;
#pragma unroll
  for (int k = 0; k < VEC; ++k) o.v[k] = from_acc<T>(acc[k]);
  st_stream<T, VEC>(out + i, o);
}

template <typename S, typename T>
int launch_sum_slabs(const void *slabs, void *out, int world, int64_t elems, cudaStream_t st) {
  constexpr int kFull = full_vec<S>();
  const bool vec_ok = elems % kFull == 0 && aligned16(slabs) && (reinterpret_cast<uintptr_t>(out) % (sizeof(T) * kFull) == 0);
  const int64_t threads = vec_ok ? elems / kFull : elems;
  const int64_t blocks = (threads + kThreads - 1) / kThreads;
  if (blocks > 2147483647LL) return TSB_ERR_TOO_LARGE;
  if (vec_ok) sum_slabs_kernel<S, T, kFull><<<(unsigned)blocks, kThreads, 0, st>>>(static_cast<const S *>(slabs), static_cast<T *>(out), world, elems);
  else sum_slabs_kernel<S, T, 1><<<(unsigned)blocks, kThreads, 0, st>>>(static_cast<const S *>(slabs), static_cast<T *>(out), world, elems);
  return launch_status();
}
}  // namespace
}  // namespace tsb

extern "C" size_t tsb_scatter_group_workspace_bytes(int64_t E, int64_t N) { return tsb::scatter_group_workspace_bytes(E, N); }

extern "C" int tsb_scatter_group(const int64_t *index, int64_t E, int64_t N, int64_t *rowptr, int32_t *perm,
                                 int32_t *count, void *workspace, size_t workspace_bytes, tsb_stream_t stream) {
  if (E < 0 || N < 1 || rowptr == nullptr) return TSB_ERR_ARG;
  if (E == 0) {
    return cudaMemsetAsync(rowptr, 0, (size_t)(N + 1) * sizeof(int64_t), reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess &&
                   (count == nullptr ||
                    cudaMemsetAsync(count, 0, (size_t)N * sizeof(int32_t), reinterpret_cast<cudaStream_t>(stream)) == cudaSuccess)
               ? TSB_OK
               : TSB_ERR_LAUNCH;
  }
  if (index == nullptr || perm == nullptr) return TSB_ERR_ARG;
  return tsb::scatter_group(index, E, N, rowptr, perm, count, workspace, workspace_bytes, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" size_t tsb_segment_csr_perm_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce) {
  return tsb::csr_reduce_workspace_bytes(B, E, K, N, dtype, reduce);
}

extern "C" int tsb_segment_csr_perm(const void *src, const int64_t *rowptr, const int32_t *perm, void *out,
                                    int64_t *arg_out, int64_t B, int64_t E, int64_t K, int64_t N, int64_t row_lo,
                                    int64_t row_hi, int dtype, int reduce, int out_seeded, void *workspace,
                                    size_t workspace_bytes, tsb_stream_t stream) {
  using namespace tsb;
  if (B < 0 || E < 0 || K < 0 || N < 0 || row_lo < 0 || row_hi > N) return TSB_ERR_ARG;
  if (B * K == 0 || row_hi <= row_lo) return TSB_OK;
  if (rowptr == nullptr || out == nullptr || (E > 0 && (src == nullptr || perm == nullptr))) return TSB_ERR_ARG;
  const bool slice = row_lo != 0 || row_hi != N;
  if (slice && B != 1) return TSB_ERR_ARG;
  const size_t elem = dtype_elem_bytes(dtype);
  CsrParams p;
  p.src = src;
  p.indptr = rowptr + row_lo;
  p.out = static_cast<unsigned char *>(out) + (size_t)(row_lo * K) * elem;
  p.arg_out = arg_out != nullptr ? arg_out + row_lo * K : nullptr;
  p.count_out = nullptr;
  p.B = B; p.E = E; p.K = K; p.N = row_hi - row_lo;
  p.bstride = 0;
  p.perm = E > 0 ? perm : nullptr;
  p.skip_outside = slice;
  p.mode = out_seeded ? kCooSeeded : kCooFresh;
  p.workspace = workspace;
  p.workspace_bytes = workspace_bytes;
  return launch_csr_reduce(p, dtype, reduce, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tsb_segment_csr_perm_routed(const void *src, const int64_t *rowptr, const int32_t *perm,
                                           void *const *owner_base, int world, int rank, int64_t rows_per_owner,
                                           int wide_staging, int64_t E, int64_t K, int64_t N, int dtype, int reduce,
                                           void *workspace, size_t workspace_bytes, tsb_stream_t stream) {
  using namespace tsb;
  if (E < 0 || K < 0 || N < 0 || owner_base == nullptr || world < 1 || world > CsrParams::kMaxRoute) return TSB_ERR_ARG;
  if (K == 0 || N == 0) return TSB_OK;
  if (rowptr == nullptr || (E > 0 && (src == nullptr || perm == nullptr))) return TSB_ERR_ARG;
  CsrParams p;
  p.src = src;
  p.indptr = rowptr;
  p.out = nullptr;
  p.arg_out = nullptr;
  p.count_out = nullptr;
  p.B = 1; p.E = E; p.K = K; p.N = N;
  p.bstride = 0;
  p.perm = E > 0 ? perm : nullptr;
  p.mode = kCooFresh;
  for (int q = 0; q < world; ++q) p.route_base[q] = owner_base[q];
  p.route_world = world;
  p.route_rank = rank;
  p.route_rows = rows_per_owner;
  p.route_wide = wide_staging != 0;
  p.workspace = workspace;
  p.workspace_bytes = workspace_bytes;
  return launch_csr_reduce(p, dtype, reduce, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tsb_sum_slabs(const void *slabs, void *out, int world, int64_t elems, int dtype, int wide_slabs,
                             tsb_stream_t stream) {
  using namespace tsb;
  if (world < 1 || elems < 0) return TSB_ERR_ARG;
  if (elems == 0) return TSB_OK;
  if (slabs == nullptr || out == nullptr) return TSB_ERR_ARG;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    if (wide_slabs) return launch_sum_slabs<acc_t<scalar_t>, scalar_t>(slabs, out, world, elems, st);
    return launch_sum_slabs<scalar_t, scalar_t>(slabs, out, world, elems, st);
  });
}

// The row-parallel kernel of the row-pointer reduction, for problems whose rows hold only a few NARROW entries (up to
// 64 bytes; the launcher's rule and the measurements behind it are in segment_csr.cu).  The chunk kernels balance
// entries and pay a fixed price per finished row - window bookkeeping, a shuffle or a diverged lane group, the fix-up of
// border rows - that is amortised over a row's entries; with two or three narrow entries per row that price is what
// bounds them.  Here a lane group (the L lanes of one entry) owns a ROW: two row pointers, up to four source entries in
// flight at a time, one write.  No carries, no fix-up kernel, rows without entries cost a store.  Rows longer than
// kShortRow entries are queued in shared memory and reduced by the whole CTA afterwards (every lane group takes every
// G-th entry, partials are merged over the groups of a warp by a shuffle butterfly and over the warps through shared
// memory, in a fixed order).  With wide entries a CTA holds few rows, each a chain of three dependent loads, and the
// kernel is latency-bound: the chunk kernels keep those shapes.
#include "csr_rows.cuh"

namespace tsb {
namespace {

constexpr int kShortRow = 32;   // entries up to which a lane group reduces a row on its own
constexpr int kRowBatch = 4;    // source entries a lane group has in flight

template <typename T, int REDUCE, int VEC, int MODE>
__global__ void __launch_bounds__(kThreads) csr_rows_kernel(CsrParams p, int l_log2) {
  constexpr bool INDIRECT = MODE >= 1;
  constexpr bool EXTRAS = MODE == 2;
  using A = acc_t<T>;
  using Acc = RowAcc<T, REDUCE, VEC, int64_t>;   // arg: the source entry (its position, or with a permutation its id)
  constexpr bool kArg = Acc::kArg;
  constexpr int kWarps = kThreads / 32;

  const T *__restrict__ src = static_cast<const T *>(p.src);
  const int L = 1 << l_log2;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int col = threadIdx.x & (L - 1);
  const int group = threadIdx.x >> l_log2;          // lane group inside the CTA
  const int groups = kThreads >> l_log2;
  const int64_t Kv = p.K / VEC;
  const int64_t total_rows = p.B * p.N;
  const int64_t none = p.E;                          // "no entry won" (MIN/MAX)

  __shared__ int64_t s_long[kThreads];
  __shared__ int s_nlong;
  __shared__ A s_val[kWarps][32 * VEC];
  __shared__ int64_t s_arg[Acc::kPair ? kWarps : 1][Acc::kPair ? 32 * VEC : 1];
  if (threadIdx.x == 0) s_nlong = 0;
  __syncthreads();

  int64_t row = (int64_t)blockIdx.x * groups + group;
  const bool have_row = row < total_rows;
  if (EXTRAS && p.route_world > 1 && have_row) {
    // routed rows: rank r starts with the rows of owner r + 1, so that at any moment the ranks store to distinct owners
    int64_t first_row = (int64_t)((p.route_rank + 1) % p.route_world) * p.route_rows;
    if (first_row > p.N) first_row = p.N;
    row = (row + first_row) % p.N;   // single batch
  }
  if (have_row) {
    const int64_t b = (p.B == 1) ? 0 : row / p.N;
    const int64_t n = row - b * p.N;
    const int64_t *ip = p.indptr + b * p.bstride + n;
    const int64_t rs = clamp64(__ldg(ip), 0, p.E);
    const int64_t re = clamp64(__ldg(ip + 1), rs, p.E);
    const int64_t len = re - rs;
    if (len > kShortRow) {
      if (col == 0) s_long[atomicAdd(&s_nlong, 1)] = row;
    } else {
      const T *bsrc = src + (b * p.E) * p.K;
      for (int64_t cb = 0; cb < Kv; cb += L) {
        const int64_t c = cb + col;
        if (c >= Kv) continue;
        Acc acc;
        acc.init(none);
        for (int64_t e0 = rs; e0 < re; e0 += kRowBatch) {   // kRowBatch loads in flight, consumed in entry order
          int64_t id[kRowBatch];
          Pack<T, VEC> v[kRowBatch];
#pragma unroll
          for (int j = 0; j < kRowBatch; ++j) {
            id[j] = -1;
            if (e0 + j < re) {
              id[j] = INDIRECT ? (int64_t)__ldg(p.perm + e0 + j) : e0 + j;
              if (id[j] < 0 || id[j] >= p.E) id[j] = -1;   // a stale slot of a permutation must not become an address
            }
          }
#pragma unroll
          for (int j = 0; j < kRowBatch; ++j)
            if (id[j] >= 0) v[j] = ld_pack<T, VEC>(bsrc + id[j] * p.K + c * VEC);
#pragma unroll
          for (int j = 0; j < kRowBatch; ++j)
            if (id[j] >= 0) acc.template update<INDIRECT>(v[j], id[j], none);
        }
        if (!store_wide_routed<T, REDUCE, VEC, EXTRAS, int64_t>(p, acc, row, c * VEC))
          write_row<T, REDUCE, VEC, int64_t>(acc, row_address<T, REDUCE, EXTRAS>(p, row, c * VEC),
                                             kArg ? p.arg_out + row * p.K + c * VEC : nullptr, len, p.mode, p.E, 0, none);
      }
      if (col == 0 && p.count_out != nullptr) static_cast<T *>(p.count_out)[row] = from_acc<T>((A)(len > 0 ? len : 1));
    }
  }
  __syncthreads();

  // ---- rows of more than kShortRow entries: the whole CTA per row ------------------------------------------------
  const int nlong = s_nlong;
  const int sub = lane >> l_log2;                    // lane group inside the warp
  for (int i = 0; i < nlong; ++i) {
    const int64_t lrow = s_long[i];
    const int64_t b = (p.B == 1) ? 0 : lrow / p.N;
    const int64_t n = lrow - b * p.N;
    const int64_t *ip = p.indptr + b * p.bstride + n;
    const int64_t rs = clamp64(__ldg(ip), 0, p.E);
    const int64_t re = clamp64(__ldg(ip + 1), rs, p.E);
    const T *bsrc = src + (b * p.E) * p.K;
    for (int64_t cb = 0; cb < Kv; cb += L) {
      const int64_t c = cb + col;
      const bool col_ok = c < Kv;
      Acc acc;
      acc.init(none);
      if (col_ok) {
        for (int64_t e0 = rs + group; e0 < re; e0 += (int64_t)groups * kRowBatch) {
          int64_t id[kRowBatch];
          Pack<T, VEC> v[kRowBatch];
#pragma unroll
          for (int j = 0; j < kRowBatch; ++j) {
            const int64_t e = e0 + (int64_t)j * groups;
            id[j] = -1;
            if (e < re) {
              id[j] = INDIRECT ? (int64_t)__ldg(p.perm + e) : e;
              if (id[j] < 0 || id[j] >= p.E) id[j] = -1;
            }
          }
#pragma unroll
          for (int j = 0; j < kRowBatch; ++j)
            if (id[j] >= 0) v[j] = ld_pack<T, VEC>(bsrc + id[j] * p.K + c * VEC);
#pragma unroll
          for (int j = 0; j < kRowBatch; ++j)
            if (id[j] >= 0) acc.template update<true>(v[j], id[j], none);   // a group's entries are not its row's first ones
        }
      }
      acc.butterfly(L, 32);                           // over the lane groups of the warp
      if (sub == 0 && col_ok) {
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          s_val[warp][col * VEC + k] = acc.val[k];
          if (Acc::kPair) s_arg[Acc::kPair ? warp : 0][Acc::kPair ? col * VEC + k : 0] = acc.arg[k];
        }
      }
      __syncthreads();
      if (warp == 0 && sub == 0 && col_ok) {          // warp 0 folds the warps' partials in a fixed order
        Acc total;
        total.init(none);
        for (int w = 0; w < kWarps; ++w) {
          A oval[VEC];
          int64_t oarg[Acc::kPair ? VEC : 1];
#pragma unroll
          for (int k = 0; k < VEC; ++k) {
            oval[k] = s_val[w][col * VEC + k];
            if (Acc::kPair) oarg[k] = s_arg[Acc::kPair ? w : 0][Acc::kPair ? col * VEC + k : 0];
          }
          total.merge(oval, oarg);
        }
        if (!store_wide_routed<T, REDUCE, VEC, EXTRAS, int64_t>(p, total, lrow, c * VEC))
          write_row<T, REDUCE, VEC, int64_t>(total, row_address<T, REDUCE, EXTRAS>(p, lrow, c * VEC),
                                             kArg ? p.arg_out + lrow * p.K + c * VEC : nullptr, re - rs, p.mode, p.E, 0, none);
      }
      __syncthreads();
    }
    if (threadIdx.x == 0 && p.count_out != nullptr) static_cast<T *>(p.count_out)[lrow] = from_acc<T>((A)(re - rs));
  }
}

template <typename T, int REDUCE, int VEC>
bool launch_mode(const CsrParams &p, int mode, cudaStream_t stream) {
  const int64_t Kv = p.K / VEC;
  const int l_log2 = (int)(Kv >= 32 ? 5 : ilog2_ceil(Kv));
  const int groups = kThreads >> l_log2;
  const int64_t blocks = (p.B * p.N + groups - 1) / groups;
  if (blocks < 1 || blocks > 2147483647LL) return false;
  if (mode == 0) csr_rows_kernel<T, REDUCE, VEC, 0><<<(unsigned)blocks, kThreads, 0, stream>>>(p, l_log2);
  else if (mode == 1) csr_rows_kernel<T, REDUCE, VEC, 1><<<(unsigned)blocks, kThreads, 0, stream>>>(p, l_log2);
  else csr_rows_kernel<T, REDUCE, VEC, 2><<<(unsigned)blocks, kThreads, 0, stream>>>(p, l_log2);
  return true;
}

template <typename T, int REDUCE>
bool launch_reduce(const CsrParams &p, bool vec, int mode, cudaStream_t stream) {
  constexpr int kFull = full_vec<T>();
  if (REDUCE == kMul && mode != 1) return false;   // products exist for scatter only: through the permutation
  if constexpr (kFull > 1) {
    if (vec) return launch_mode<T, REDUCE, kFull>(p, mode, stream);
  }
  return launch_mode<T, REDUCE, 1>(p, mode, stream);
}

}  // namespace

bool launch_csr_short_rows(const CsrParams &p, int dtype, int reduce, bool vec, int mode, cudaStream_t stream) {
  if (p.B * p.N >= (1ll << 40)) return false;
  return TSB_DISPATCH_DTYPE(dtype, [&]() -> int {
    switch (reduce) {
      case TSB_SUM: return launch_reduce<scalar_t, kSum>(p, vec, mode, stream);
      case TSB_MEAN: return launch_reduce<scalar_t, kMean>(p, vec, mode, stream);
      case TSB_MIN: return launch_reduce<scalar_t, kMin>(p, vec, mode, stream);
      case TSB_MAX: return launch_reduce<scalar_t, kMax>(p, vec, mode, stream);
      case TSB_MUL: return launch_reduce<scalar_t, kMul>(p, vec, mode, stream);
      default: return 0;
    }
  }) > 0;
}

}  // namespace tsb

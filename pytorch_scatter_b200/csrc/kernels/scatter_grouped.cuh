// Internal interface of the atomics-free scatter path (scatter_grouped.cu): entries grouped by target
// row with a counting sort of the index, rows reduced through the permutation.
#pragma once

#include "csr_reduce.cuh"

namespace tsb {

// Structural conditions: one index entry per source row (stride 0 along the features, unit stride
// along the entries), shared by all batches; SUM / MEAN (floats) / MIN / MAX / MUL; E < 2^30.
bool scatter_grouped_possible(int64_t B, int64_t E, int64_t K, int64_t N, int64_t sb, int64_t se, int64_t sk,
                              int dtype, int reduce);

// Scratch: a counter and a row pointer per row, a rank and a permutation slot per entry, and the
// partial-row scratch of the reduction.  0 when the shapes rule the path out.
size_t scatter_grouped_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce);

// The grouping alone: rowptr [N+1], perm [E] (the first rowptr[N] slots are meaningful; entries that name
// no row are dropped), count [N] raw entries per row or null (required beyond 67 M rows).
size_t scatter_group_workspace_bytes(int64_t E, int64_t N);
int scatter_group(const int64_t *index, int64_t E, int64_t N, int64_t *rowptr, int32_t *perm, int32_t *count,
                  void *workspace, size_t workspace_bytes, cudaStream_t stream);

// out_seeded / arg_out / count_out (raw int32 counts per row, MEAN only) as in tsb_scatter.
int run_scatter_grouped(const void *src, const int64_t *index, void *out, int64_t *arg_out, int32_t *count_out,
                        int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce, int out_seeded,
                        void *workspace, size_t workspace_bytes, cudaStream_t stream);

}  // namespace tsb

/*
 * tsb200 - C ABI of the B200 (sm_100a) kernel library behind the torch_scatter operator set.
 *
 * Everything here is plain C: device pointers, 64-bit sizes, enums as int, a CUDA stream handle.
 * No torch types cross this boundary.  Every entry point
 *   - returns 0 (TSB_OK) or a tsb_status error code, never throws,
 *   - launches on the stream it is given and returns without synchronising,
 *   - allocates no memory: scratch comes from the caller (query the *_workspace_bytes twin first),
 *   - is re-entrant.  Global state: per-device attributes cached on first use (SM count, opt-in shared-memory sizes:
 *     idempotent, written through atomics).  The one exception is tsb_segment_csr_noalloc, whose scratch is a single
 *     array inside the library: calls that overlap on one device race on it, and its first call per device (which looks
 *     the array's address up) must come before any stream capture.
 *
 * Canonical flattened shapes (the same B/E/K/N flattening the upstream launchers use,
 * csrc/cuda/scatter_cuda.cu:103-110, segment_csr_cuda.cu:144-146, segment_coo_cuda.cu:207-211):
 *   src  [B, E, K]   B = product of the dims before the reduced dim, E = length of the reduced dim,
 *   out  [B, N, K]   K = product of the trailing (feature) dims, N = output length of the reduced dim.
 * All data tensors are dense row-major in that flattened shape.  Index / indptr tensors are int64.
 *
 * Robustness rule: an index outside [0, N) or an indptr outside [0, E] never faults the GPU; such
 * entries are skipped / clamped (the upstream kernels leave this undefined, scatter_cuda.cu:25-30).
 */
#ifndef TSB200_H
#define TSB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling in cuda_runtime.h */
typedef struct CUstream_st *tsb_stream_t;

/* element types of src/out (the six types the upstream test-suite exercises, torch_scatter/testing.py:7-10) */
/* The narrow integers (upstream dispatches them with AT_DISPATCH_ALL_TYPES_AND2, csrc/cuda/scatter_cuda.cu:114,
 * segment_csr_cuda.cu:150, segment_coo_cuda.cu:217) accumulate in int32 and are narrowed once at the end: identical to
 * accumulating in the narrow type (two's-complement wrap) for SUM / MUL / MIN / MAX; MEAN divides the narrowed sum. */
enum tsb_dtype { TSB_F32 = 0, TSB_F64 = 1, TSB_F16 = 2, TSB_BF16 = 3, TSB_I32 = 4, TSB_I64 = 5,
                 TSB_U8 = 6, TSB_I8 = 7, TSB_I16 = 8 };

/* reductions (csrc/cuda/reducer.cuh:8-13; "div" is unreachable upstream and is not provided) */
enum tsb_reduce { TSB_SUM = 0, TSB_MEAN = 1, TSB_MIN = 2, TSB_MAX = 3, TSB_MUL = 4,
                  /* log-sum-exp per row, segment_csr / segment_coo only, fp32 / fp16 / bf16 only: the per-group
                   * statistic behind upstream's softmax composites (torch_scatter/composite/softmax.py:9-51,
                   * logsumexp.py:8-56), computed online in one pass.  `out` is FP32 [B,N,K] for every source dtype;
                   * rows without entries give -inf; out_seeded must be 0 */
                  TSB_LSE = 5 };

enum tsb_status {
  TSB_OK = 0,
  TSB_ERR_DTYPE = 1,       /* unknown dtype enum */
  TSB_ERR_REDUCE = 2,      /* unknown / unsupported reduction for this entry point */
  TSB_ERR_ARG = 3,         /* null pointer or negative size where one is required */
  TSB_ERR_WORKSPACE = 4,   /* workspace pointer null or smaller than *_workspace_bytes() */
  TSB_ERR_LAUNCH = 5,      /* cudaGetLastError() reported a launch failure */
  TSB_ERR_TOO_LARGE = 6    /* a size exceeds a documented limit of the entry point */
};

/* Human-readable text for a tsb_status value (static storage). */
const char *tsb_status_string(int status);

/* CUDA toolkit version the library was compiled with, e.g. 12090.
 * Replaces scatter::cuda_version(), csrc/version.cpp:27-42. */
int64_t tsb_cuda_version(void);

/* ------------------------------------------------------------------------------------------------
 * segment_csr: out[b,n,:] = reduce over e in [indptr[b,n], indptr[b,n+1]) of src[b,e,:]
 * Replaces segment_csr_cuda + segment_csr_kernel / segment_csr_broadcast_kernel,
 * csrc/cuda/segment_csr_cuda.cu:97-168, :15-60, :62-95 (CPU twin csrc/cpu/segment_csr_cpu.cpp:8-92).
 *   indptr               [*, N+1] int64; row b starts at indptr + b*indptr_batch_stride (0 = one shared row)
 *   out                  [B,N,K]; always overwritten (never accumulated into)
 *   arg_out              [B,N,K] int64, required for MIN/MAX, ignored otherwise; empty rows get E
 *   reduce               SUM, MEAN, MIN or MAX.  MEAN divides by max(count,1); empty rows give 0.
 *   workspace            tsb_segment_csr_workspace_bytes(...) bytes, 256-byte aligned: partial rows at
 *                        the borders of the entry chunks the reduction is balanced over
 * Deterministic: the summation order depends only on the shapes. */
size_t tsb_segment_csr_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce);
int tsb_segment_csr(const void *src, const int64_t *indptr, void *out, int64_t *arg_out,
                    int64_t B, int64_t E, int64_t K, int64_t N, int64_t indptr_batch_stride,
                    int dtype, int reduce, void *workspace, size_t workspace_bytes, tsb_stream_t stream);

/* segment_csr for callers that cannot provide a workspace.  It has no counterpart in the upstream
 * project.  Meant for hosts that cannot allocate device memory at call time: an inference server that
 * handed the whole GPU to its own memory pool at start-up, a real-time loop where cudaMalloc's implicit
 * device synchronisation (and its chance of failing under fragmentation) is not acceptable, or a plug-in
 * that may only launch kernels - and that have no caching allocator to ask for a scratch tensor instead.
 * Same arguments and results as tsb_segment_csr; the scratch is a fixed array of
 * TSB_STATIC_SCRATCH_BYTES inside the library (every GPU that loads the library holds it until the
 * process exits).
 *   - Problems whose tsb_segment_csr_workspace_bytes(...) exceeds TSB_STATIC_SCRATCH_BYTES are rejected
 *     with TSB_ERR_TOO_LARGE before anything is launched (fp32, K = 64: about 8 million entries).
 *   - The call itself allocates nothing (no cudaMalloc / cudaFree, no allocating library routine).
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that
 *     device current); make that first call before starting any stream capture.
 *   - All calls on a device share the one array.  It keeps the previous call's contents, which is harmless:
 *     nothing in it has to start at zero.  Two calls that overlap on the GPU (different streams, or
 *     different host threads) race on it: serialise them, or use tsb_segment_csr with separate workspaces. */
#define TSB_STATIC_SCRATCH_BYTES (8u << 20)
int tsb_segment_csr_noalloc(const void *src, const int64_t *indptr, void *out, int64_t *arg_out,
                            int64_t B, int64_t E, int64_t K, int64_t N, int64_t indptr_batch_stride,
                            int dtype, int reduce, tsb_stream_t stream);

/* gather_csr: out[b,e,:] = src[b,n,:] for e in [indptr[b,n], indptr[b,n+1]); positions no row covers
 * are left untouched.  Replaces gather_csr_cuda + kernels, csrc/cuda/segment_csr_cuda.cu:219-281,
 * :170-217.  Here src is [B,N,K] and out is [B,E,K].
 *   divide_by_count != 0 fuses the backward of segment_mean_csr (csrc/segment_csr.cpp:94-111):
 *   each row's value is divided by its length before it is broadcast (floating dtypes only). */
int tsb_gather_csr(const void *src, const int64_t *indptr, void *out,
                   int64_t B, int64_t E, int64_t K, int64_t N, int64_t indptr_batch_stride,
                   int dtype, int divide_by_count, tsb_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * segment_coo: the same reduction keyed by a SORTED index [*, E] (row b at index + b*index_batch_stride).
 * Replaces segment_coo_cuda + its five kernels, csrc/cuda/segment_coo_cuda.cu:152-283, :14-150
 * (CPU twin csrc/cpu/segment_coo_cpu.cpp:8-141).
 *   out_seeded == 0      out is write-only: rows no index names become 0; MIN/MAX results equal to
 *                        the reduction's identity are replaced by 0 (segment_coo_cpu.cpp:131-132)
 *   out_seeded != 0      accumulate into the caller's out (the `out=` argument): each named row
 *                        starts from its current value; unnamed rows are untouched
 *   arg_out              [B,N,K] int64 for MIN/MAX (always fully written; E where no element won)
 *   count_out            [B,N] of dtype, for MEAN: run length clamped to >= 1 (segment_coo_cpu.cpp:134-136)
 *   workspace            tsb_segment_coo_workspace_bytes(...) bytes, 256-byte aligned: the row pointers
 *                        rebuilt from the sorted index, then the scratch of the row-pointer reduction
 * Deterministic (no atomics). */
size_t tsb_segment_coo_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce);
int tsb_segment_coo(const void *src, const int64_t *index, void *out, int64_t *arg_out, void *count_out,
                    int64_t B, int64_t E, int64_t K, int64_t N, int64_t index_batch_stride,
                    int dtype, int reduce, int out_seeded,
                    void *workspace, size_t workspace_bytes, tsb_stream_t stream);

/* gather_coo: out[b,e,:] = src[b,index[b,e],:].  src [B,N,K], out [B,E,K].
 * Replaces gather_coo_cuda + kernels, csrc/cuda/segment_coo_cuda.cu:327-382, :285-325.
 *   count (may be null)  [B,N] of dtype: when given, each value is divided by count[b,index[b,e]];
 *                        fuses the backward of segment_mean_coo (csrc/segment_coo.cpp:99-112). */
int tsb_gather_coo(const void *src, const int64_t *index, void *out, const void *count,
                   int64_t B, int64_t E, int64_t K, int64_t N, int64_t index_batch_stride,
                   int dtype, tsb_stream_t stream);

/* gather_coo with an element-wise epilogue: out[b,e,:] = op(x[b,e,:], table[b,index[b,e],:]), op 1 = exp(x - row),
 * op 2 = x - row; x and out fp32 / fp16 / bf16, table always FP32 (what TSB_LSE writes).  With table = the TSB_LSE reduction of x these are the second passes of
 * upstream's scatter_softmax / scatter_log_softmax (torch_scatter/composite/softmax.py:9-51) on a sorted index:
 * two passes over the source instead of six. */
int tsb_gather_coo_apply(const void *x, const void *table, const int64_t *index, void *out,
                         int64_t B, int64_t E, int64_t K, int64_t N, int64_t index_batch_stride,
                         int dtype, int op, tsb_stream_t stream);
/* The same with op 3 = (x - row)^2 as well and an optional second FP32 table `scale` [B,N,K] (NULL: none) whose
 * gathered row multiplies the result: with table = the group means these are the second pass of upstream's
 * scatter_std (torch_scatter/composite/std.py:31-33, op 3) and its backward (op 2 with scale = grad / (count * std)). */
int tsb_gather_coo_apply2(const void *x, const void *table, const void *scale, const int64_t *index, void *out,
                          int64_t B, int64_t E, int64_t K, int64_t N, int64_t index_batch_stride,
                          int dtype, int op, tsb_stream_t stream);

/* Sets *unsorted_flag (a device int) to 1 if the n index entries are not ascending, else to 0.  Lets a caller
 * pick the sorted-index kernels for an index of unknown order (upstream asserts sortedness instead,
 * csrc/cuda/segment_coo_cuda.cu:42,111). */
int tsb_index_unsorted(const int64_t *index, int64_t n, int *unsorted_flag, tsb_stream_t stream);

/* ------------------------------------------------------------------------------------------------
 * scatter: out[b, index(b,e,k), k] (+)= src[b,e,k] for an UNSORTED index.
 * Replaces scatter_cuda + scatter_kernel + scatter_arg_kernel, csrc/cuda/scatter_cuda.cu:58-138,
 * :13-56 (CPU twin csrc/cpu/scatter_cpu.cpp:7-87), and for SUM/MEAN the ATen route of
 * torch_scatter/scatter.py:8-25,44-66.
 *   index                int64 view of logical shape [B,E,K] addressed as
 *                        index[b*idx_stride_b + e*idx_stride_e + k*idx_stride_k]; a broadcast 1-D
 *                        index is (0,1,0) and is then read once per row, not once per element
 *   reduce               SUM, MEAN, MIN, MAX or MUL
 *   out_seeded           0: out is write-only (SUM/MEAN/MUL start from the identity; MIN/MAX results
 *                        equal to the identity become 0, scatter_cpu.cpp:80-81); !=0: accumulate into out
 *   arg_out              [B,N,K] int64 for MIN/MAX: smallest e whose value equals the result, else E
 *   count_out            MEAN only: int32 [Bc,N,Kc] with Bc = idx_stride_b ? B : 1 and
 *                        Kc = idx_stride_k ? K : 1; receives the per-target element count
 *   workspace            tsb_scatter_workspace_bytes(...) bytes, 256-byte aligned, always at least 256: a
 *                        flag for the variant choice, fp32 accumulators for 16-bit dtypes, copies of
 *                        small outputs that contended updates are spread over, and - for outputs too
 *                        large to stay in L2 - the scratch of the atomics-free path (entries grouped by
 *                        target row with a counting sort of the index, rows reduced through that
 *                        permutation: 8 bytes per entry + 12 per row)
 * Float SUM/MEAN/MUL: the summation order is not fixed.  MIN/MAX and arg are exact. */
size_t tsb_scatter_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce);
int tsb_scatter(const void *src, const int64_t *index, void *out, int64_t *arg_out, int32_t *count_out,
                int64_t B, int64_t E, int64_t K, int64_t N,
                int64_t idx_stride_b, int64_t idx_stride_e, int64_t idx_stride_k,
                int dtype, int reduce, int out_seeded,
                void *workspace, size_t workspace_bytes, tsb_stream_t stream);

/* The two halves of the atomics-free scatter, for callers that reuse one grouping for several reductions or
 * reduce the rows slice by slice (a sharded scatter hands every finished slice to its collective while the next
 * one is reduced).  No counterpart upstream.
 *   tsb_scatter_group     groups the entry ids 0..E-1 by the row index[e] names: rowptr [N+1] int64 (row n owns
 *                         perm[rowptr[n] .. rowptr[n+1])), perm [E] int32 (entries naming no row are dropped, so
 *                         only the first rowptr[N] slots are meaningful), count [N] int32 entries per row or NULL
 *                         (required above 67 M rows).  E < 2^30.  The order inside a row is not fixed.
 *   tsb_segment_csr_perm  out[b, n, :] = reduce over q in [rowptr[n], rowptr[n+1]) of src[b, perm[q], :] for the rows
 *                         row_lo <= n < row_hi (other rows of out are not touched; a proper slice needs B == 1),
 *                         with scatter's write rules (out_seeded as in tsb_scatter; MIN/MAX args are entry ids,
 *                         ties towards the smaller id).  SUM, MEAN, MIN, MAX, or (whole problem only) MUL. */
size_t tsb_scatter_group_workspace_bytes(int64_t E, int64_t N);
int tsb_scatter_group(const int64_t *index, int64_t E, int64_t N, int64_t *rowptr, int32_t *perm, int32_t *count,
                      void *workspace, size_t workspace_bytes, tsb_stream_t stream);
size_t tsb_segment_csr_perm_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce);
int tsb_segment_csr_perm(const void *src, const int64_t *rowptr, const int32_t *perm, void *out, int64_t *arg_out,
                         int64_t B, int64_t E, int64_t K, int64_t N, int64_t row_lo, int64_t row_hi,
                         int dtype, int reduce, int out_seeded,
                         void *workspace, size_t workspace_bytes, tsb_stream_t stream);

/* tsb_segment_csr_perm for a scatter sharded over `world` <= 8 GPUs (SUM of this rank's entries, write-only):
 * GPU q owns the rows [q*rows_per_owner, (q+1)*rows_per_owner) and holds a staging buffer [world, rows_per_owner, K]
 * at owner_base[q] (a HOST array of `world` device pointers, peers' memory included: anything this GPU may store
 * to).  Every finished row n is stored into slab `rank` of its owner's buffer, so the partial rows cross NVLink as
 * plain stores while the reduction is still running; once all ranks have finished (the caller's barrier), every
 * owner adds its `world` slabs.  rows_per_owner * world >= N.
 *   wide_staging != 0    the staging buffers hold the accumulation type (fp32 for fp16 / bf16 sources, the source type
 *                        otherwise): 16-bit partial sums then cross NVLink unrounded and the sharded result equals
 *                        the single-GPU one up to summation order; 0: staging buffers of the source type (half the
 *                        NVLink bytes for 16-bit sources, every rank's partial rounded once more).
 * No counterpart upstream (its scatter is single-GPU). */
int tsb_segment_csr_perm_routed(const void *src, const int64_t *rowptr, const int32_t *perm,
                                void *const *owner_base, int world, int rank, int64_t rows_per_owner, int wide_staging,
                                int64_t E, int64_t K, int64_t N, int dtype, int reduce,
                                void *workspace, size_t workspace_bytes, tsb_stream_t stream);

/* The owner's last step of the routed scatter: out[i] = sum over q < world of slabs[q * elems + i] (accumulated in fp32
 * for 16-bit dtypes), one streaming pass.  wide_slabs != 0: the slabs hold the accumulation type (see above), out the
 * dtype. */
int tsb_sum_slabs(const void *slabs, void *out, int world, int64_t elems, int dtype, int wide_slabs, tsb_stream_t stream);

/* One slice of an unsorted scatter SUM, for sharded use: adds the E edges of this call (src [E,K], 1-D index [E])
 * into the target rows [row_lo, row_hi) of `partial` [N,K], after zeroing exactly those rows; targets outside the
 * slice are ignored.  `partial` is held in accumulation precision: fp32 for fp32/fp16/bf16 sources, the source
 * type otherwise.  A caller that shards the edge dimension over GPUs runs one call per slice and can hand each
 * finished slice to a collective while the next slice is being accumulated (upstream has no sharded path; this
 * is the building block of the multi-GPU scatter here, built on the kernels of tsb_scatter).
 *   workspace            at least 256 bytes, 256-byte aligned (the index probe's flag). */
int tsb_scatter_sum_slice(const void *src, const int64_t *index, void *partial, int64_t E, int64_t K, int64_t N,
                          int dtype, int64_t row_lo, int64_t row_hi, void *workspace, size_t workspace_bytes,
                          tsb_stream_t stream);

/* Backward of scatter SUM / MEAN: grad_in[b,e,k] = grad_out[b, index(b,e,k), k] (/ max(count,1)).
 * Replaces the torch::gather calls in ScatterSum/ScatterMean::backward, csrc/scatter.cpp:72-80,149-160.
 * count may be null (SUM); otherwise the int32 tensor tsb_scatter filled for MEAN. */
int tsb_scatter_backward(const void *grad_out, const int64_t *index, void *grad_in, const int32_t *count,
                         int64_t B, int64_t E, int64_t K, int64_t N,
                         int64_t idx_stride_b, int64_t idx_stride_e, int64_t idx_stride_k,
                         int dtype, tsb_stream_t stream);

/* Backward of every MIN/MAX op: grad_in [B,E,K] is zeroed, then grad_in[b, arg[b,n,k], k] = grad_out[b,n,k]
 * wherever arg < E.  Replaces the zeros + scatter_ + narrow sequence of csrc/scatter.cpp:184-196,
 * csrc/segment_coo.cpp:132-144 and csrc/segment_csr.cpp:130-142. */
int tsb_arg_backward(const void *grad_out, const int64_t *arg, void *grad_in,
                     int64_t B, int64_t E, int64_t K, int64_t N, int dtype, tsb_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* TSB200_H */

// Internal interface of the row-pointer segmented reduction shared by segment_csr and segment_coo.
#pragma once

#include "common.cuh"

namespace tsb {

// How results are written (the three behaviours of the upstream CPU loops):
//   kCsr        out overwritten; empty row -> 0, arg E          (csrc/cpu/segment_csr_cpu.cpp:69-87)
//   kCooFresh   out write-only; absent row -> 0; MIN/MAX equal to the identity -> 0
//                                                              (csrc/cpu/segment_coo_cpu.cpp:84-85,131-132)
//   kCooSeeded  accumulate into out; absent rows untouched     (csrc/cpu/segment_coo_cpu.cpp:91-92,120);
//               MIN/MAX: the value already in out wins ties and then the arg is E
enum CsrMode { kCsr = 0, kCooFresh = 1, kCooSeeded = 2 };

struct CsrParams {
  const void *src;        // [B,E,K]
  const int64_t *indptr;  // row b at indptr + b*bstride, N+1 entries
  void *out;              // [B,N,K]
  int64_t *arg_out;       // [B,N,K] or null
  void *count_out;        // [B,N] of dtype or null (COO mean)
  int64_t B, E, K, N, bstride;
  // Optional indirection: position q of the reduced dimension reads source entry perm[q] (the same
  // permutation for every batch).  Lets an unsorted scatter run as "group the entry ids by target row,
  // then reduce rows" without moving the source.  MIN/MAX then report perm[q] as the arg and break
  // ties towards the smaller entry id.  Requires E < 2^30.
  const int32_t *perm = nullptr;
  // Row pointers that cover only part of [0, E) (a slice of the rows of a larger problem): chunks that
  // lie entirely before indptr[0] or after indptr[N] return at once instead of streaming entries that
  // belong to no row.  Single batch only.
  bool skip_outside = false;
  // Optional routing of the finished rows to their owners (a sharded scatter over `route_world` GPUs,
  // SUM, single batch): row n belongs to GPU q = n / route_rows and is stored at
  // route_base[q] + ((route_rank * route_rows + n % route_rows) * K) elements, i.e. into the slab this
  // rank owns inside q's staging buffer [route_world, route_rows, K].  route_base[q] may be peer memory:
  // the rows then cross NVLink as plain stores while the reduction is still running.  `out` is unused.
  static constexpr int kMaxRoute = 8;
  void *route_base[kMaxRoute] = {nullptr};
  int route_world = 0, route_rank = 0;
  int64_t route_rows = 0;
  // Staging buffers in accumulation precision: fp16 / bf16 partial sums travel as fp32 and are rounded once, by the
  // owner, after the slabs have been added (twice the bytes over NVLink; without it every rank rounds its partial to
  // 16 bits first).  No difference for the other types, whose accumulators have the source type.
  bool route_wide = false;
  int mode;
  void *workspace;        // csr_reduce_workspace_bytes(...) bytes, 256-byte aligned
  size_t workspace_bytes;
};

// Scratch for the partial rows at chunk borders (see segment_csr.cu).
size_t csr_reduce_workspace_bytes(int64_t B, int64_t E, int64_t K, int64_t N, int dtype, int reduce);

// Picks the vector width / lane geometry from the shapes and launches.  Returns a tsb_status.
int launch_csr_reduce(const CsrParams &p, int dtype, int reduce, cudaStream_t stream);

}  // namespace tsb

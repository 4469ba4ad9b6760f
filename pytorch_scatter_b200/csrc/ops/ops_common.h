// Host side of the torch_scatter operator set: argument checking, shape flattening, output
// allocation and autograd.  All arithmetic happens behind the C ABI declared in tsb200.h; this
// layer only moves torch tensors' device pointers, sizes and the current CUDA stream across it.
#pragma once

#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/script.h>

#include <optional>
#include <string>
#include <tuple>
#include <vector>

#include "../../../include/tsb200.h"

namespace tsb_ops {

// Same wording as the upstream checks (csrc/cuda/utils.cuh:5-7) so callers see familiar errors.
#define TSB_CHECK_CUDA(x) TORCH_CHECK((x).device().is_cuda(), #x " must be CUDA tensor (this build has no CPU path)")
#define TSB_CHECK_INPUT(x) TORCH_CHECK(x, "Input mismatch")

inline int dtype_enum(const torch::Tensor &t) {
  switch (t.scalar_type()) {
    case at::ScalarType::Float: return TSB_F32;
    case at::ScalarType::Double: return TSB_F64;
    case at::ScalarType::Half: return TSB_F16;
    case at::ScalarType::BFloat16: return TSB_BF16;
    case at::ScalarType::Int: return TSB_I32;
    case at::ScalarType::Long: return TSB_I64;
    case at::ScalarType::Byte: return TSB_U8;
    case at::ScalarType::Char: return TSB_I8;
    case at::ScalarType::Short: return TSB_I16;
    default: TORCH_CHECK(false, "torch_scatter (B200 build): unsupported dtype ", t.scalar_type());
  }
}

inline int reduce_enum(const std::string &reduce) {
  if (reduce == "sum" || reduce == "add") return TSB_SUM;
  if (reduce == "mean") return TSB_MEAN;
  if (reduce == "min") return TSB_MIN;
  if (reduce == "max") return TSB_MAX;
  if (reduce == "mul") return TSB_MUL;
  TORCH_CHECK(false, "unknown reduce '", reduce, "'");
}

inline void check_status(int status, const char *what) {
  TORCH_CHECK(status == TSB_OK, what, " failed: ", tsb_status_string(status));
}

inline tsb_stream_t current_stream() {
  return reinterpret_cast<tsb_stream_t>(at::cuda::getCurrentCUDAStream().stream());
}

inline void check_index_dtype(const torch::Tensor &index, const char *name) {
  TORCH_CHECK(index.scalar_type() == at::ScalarType::Long, name, " must be an int64 tensor");
}

inline std::vector<int64_t> list2vec(const c10::List<int64_t> &list) {
  std::vector<int64_t> result;
  result.reserve(list.size());
  for (size_t i = 0; i < list.size(); i++) result.push_back(list[i]);
  return result;
}

// A [.., L] int64 tensor whose leading dims were expanded to `B` batches, reduced to what the
// kernels take: a dense base pointer plus the distance between consecutive batches (0 when every
// batch shares one row).  Keeps the backing tensor alive.
struct BatchedRows {
  torch::Tensor holder;
  int64_t batch_stride;
  const int64_t *ptr() const { return holder.data_ptr<int64_t>(); }
};

inline BatchedRows batched_rows(const torch::Tensor &t) {
  const int64_t last = t.dim() - 1;
  bool shared = true;
  for (int64_t i = 0; i < last; i++)
    if (t.size(i) != 1 && t.stride(i) != 0) shared = false;
  BatchedRows r;
  if (shared) {
    torch::Tensor row = t;
    for (int64_t i = 0; i < last; i++) row = row.select(0, 0);
    r.holder = row.contiguous();
    r.batch_stride = 0;
  } else {
    r.holder = t.contiguous();
    r.batch_stride = t.size(last);
  }
  return r;
}

// Every routine that touches tensor DATA is an operator of its own (torch_scatter::_*, CUDA kernels registered in the
// registry files, shape-only "fake" kernels registered from Python in pytorch_scatter_b200/_meta.py).  The drivers
// below look their operator up once and call it through the dispatcher, so the public operators - argument handling
// and autograd written against these drivers - run unchanged on real tensors, and on fake tensors when a tracing
// compiler propagates shapes through them (upstream registers no fake kernels: its operators break the graph).
template <typename Signature> inline c10::TypedOperatorHandle<Signature> internal_op(const char *name) {
  return c10::Dispatcher::singleton().findSchemaOrThrow(name, "").typed<Signature>();
}
inline torch::Tensor no_tensor(const torch::Tensor &like) { return torch::empty({0}, like.options()); }

// ---- forward/backward drivers shared by the registry files ------------------------------------
std::tuple<torch::Tensor, std::optional<torch::Tensor>>
segment_csr_fw(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out,
               const std::string &reduce);
torch::Tensor gather_csr_fw(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out,
                            bool divide_by_count, std::optional<int64_t> length);

std::tuple<torch::Tensor, std::optional<torch::Tensor>>
segment_coo_fw(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
               std::optional<int64_t> dim_size, const std::string &reduce);
torch::Tensor gather_coo_fw(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
                            std::optional<torch::Tensor> count);

// grad_in[.., arg, ..] = grad_out along `dim`, for every MIN/MAX backward.
torch::Tensor arg_backward(const torch::Tensor &grad_out, const torch::Tensor &arg_out,
                           std::vector<int64_t> src_shape, int64_t dim);

}  // namespace tsb_ops

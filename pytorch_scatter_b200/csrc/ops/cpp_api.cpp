// The C++ API declared in include/torchscatter/scatter.h: the fifteen free functions of the upstream
// project's <torchscatter/scatter.h> (csrc/scatter.h:13-80 there).  Each one looks up the operator of the same
// name in the `torch_scatter` namespace once and calls it through the dispatcher, so C++ callers get exactly
// what Python and TorchScript callers get (device guard, autograd, error wording).
#include <ATen/core/dispatch/Dispatcher.h>

#include "../../../include/torchscatter/scatter.h"
#include "../../../include/tsb200.h"

namespace {
using torch::Tensor;
using OptTensor = std::optional<Tensor>;
using OptInt = std::optional<int64_t>;
using Pair = std::tuple<Tensor, Tensor>;

template <typename Signature> c10::TypedOperatorHandle<Signature> op(const char *name) {
  return c10::Dispatcher::singleton().findSchemaOrThrow(name, "").typed<Signature>();
}
}  // namespace

namespace scatter {
int64_t cuda_version() noexcept { return tsb_cuda_version(); }
}  // namespace scatter

#define TSB_SCATTER_API(NAME, RET)                                                                            \
  RET NAME(Tensor src, Tensor index, int64_t dim, OptTensor optional_out, OptInt dim_size) {                  \
    static auto handle = op<RET(Tensor, Tensor, int64_t, OptTensor, OptInt)>("torch_scatter::" #NAME);        \
    return handle.call(std::move(src), std::move(index), dim, std::move(optional_out), dim_size);             \
  }
TSB_SCATTER_API(scatter_sum, Tensor)
TSB_SCATTER_API(scatter_mul, Tensor)
TSB_SCATTER_API(scatter_mean, Tensor)
TSB_SCATTER_API(scatter_min, Pair)
TSB_SCATTER_API(scatter_max, Pair)
#undef TSB_SCATTER_API

#define TSB_COO_API(NAME, RET)                                                                                \
  RET NAME(Tensor src, Tensor index, OptTensor optional_out, OptInt dim_size) {                               \
    static auto handle = op<RET(Tensor, Tensor, OptTensor, OptInt)>("torch_scatter::" #NAME);                 \
    return handle.call(std::move(src), std::move(index), std::move(optional_out), dim_size);                  \
  }
TSB_COO_API(segment_sum_coo, Tensor)
TSB_COO_API(segment_mean_coo, Tensor)
TSB_COO_API(segment_min_coo, Pair)
TSB_COO_API(segment_max_coo, Pair)
#undef TSB_COO_API

#define TSB_ROWS_API(NAME, RET)                                                                               \
  RET NAME(Tensor src, Tensor rows, OptTensor optional_out) {                                                 \
    static auto handle = op<RET(Tensor, Tensor, OptTensor)>("torch_scatter::" #NAME);                         \
    return handle.call(std::move(src), std::move(rows), std::move(optional_out));                             \
  }
TSB_ROWS_API(gather_coo, Tensor)
TSB_ROWS_API(segment_sum_csr, Tensor)
TSB_ROWS_API(segment_mean_csr, Tensor)
TSB_ROWS_API(segment_min_csr, Pair)
TSB_ROWS_API(segment_max_csr, Pair)
TSB_ROWS_API(gather_csr, Tensor)
#undef TSB_ROWS_API

// torch_scatter::segment_{sum,mean,min,max}_csr, torch_scatter::gather_csr and
// torch_scatter::cuda_version: schemas and autograd behaviour of the upstream registry
// (csrc/segment_csr.cpp:57-239, csrc/version.cpp:27-42) on top of the tsb200 C ABI.
#include "ops_common.h"

namespace tsb_ops {

namespace {
std::tuple<torch::Tensor, std::optional<torch::Tensor>>
segment_csr_impl(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out,
                 const std::string &reduce) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(indptr);
  if (optional_out.has_value()) TSB_CHECK_CUDA(optional_out.value());
  check_index_dtype(indptr, "indptr");
  c10::cuda::CUDAGuard guard(src.device());

  TSB_CHECK_INPUT(src.dim() >= indptr.dim());
  TSB_CHECK_INPUT(indptr.dim() >= 1);
  auto sizes = indptr.sizes().vec();
  for (int64_t i = 0; i < indptr.dim() - 1; i++) sizes[i] = src.size(i);
  indptr = indptr.expand(sizes);
  const int64_t dim = indptr.dim() - 1;

  src = src.contiguous();
  const int red = reduce_enum(reduce);
  TORCH_CHECK(red != TSB_MUL, "segment_csr does not support reduce='mul'");

  torch::Tensor out;
  bool copy_back = false;
  if (optional_out.has_value()) {
    copy_back = !optional_out.value().is_contiguous();
    out = optional_out.value().contiguous();
    TSB_CHECK_INPUT(out.dim() == src.dim());
    TSB_CHECK_INPUT(out.scalar_type() == src.scalar_type());
    for (int64_t i = 0; i < out.dim(); i++)
      if (i != dim) TSB_CHECK_INPUT(src.size(i) == out.size(i));
    TSB_CHECK_INPUT(src.numel() == 0 || out.size(dim) == indptr.size(dim) - 1);
  } else {
    sizes = src.sizes().vec();
    sizes[dim] = std::max<int64_t>(indptr.size(dim) - 1, 0);
    out = torch::empty(sizes, src.options());
  }

  std::optional<torch::Tensor> arg_out = std::nullopt;
  const bool minmax = red == TSB_MIN || red == TSB_MAX;
  if (src.numel() == 0) {
    if (minmax) arg_out = torch::full(out.sizes(), src.size(dim), indptr.options());
    if (!optional_out.has_value()) out.fill_(0);
    return std::make_tuple(out, arg_out);
  }
  if (minmax) arg_out = torch::empty(out.sizes(), indptr.options());

  const int64_t B = indptr.numel() / indptr.size(-1);
  const int64_t N = out.size(dim);
  const int64_t E = src.size(dim);
  const int64_t K = (B * N) > 0 ? out.numel() / (B * N) : 0;
  BatchedRows rows = batched_rows(indptr);
  const size_t ws_bytes = tsb_segment_csr_workspace_bytes(B, E, K, N, dtype_enum(src), red);
  auto workspace = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kUInt8));
  check_status(tsb_segment_csr(src.data_ptr(), rows.ptr(), out.data_ptr(),
                               minmax ? arg_out.value().data_ptr<int64_t>() : nullptr, B, E, K, N,
                               rows.batch_stride, dtype_enum(src), red, workspace.data_ptr(), ws_bytes,
                               current_stream()),
               "tsb_segment_csr");
  if (copy_back) {
    optional_out.value().copy_(out);
    out = optional_out.value();
  }
  return std::make_tuple(out, arg_out);
}

// `length`: the output's size along the gathered dimension when the caller knows it (no `out`, no host sync)
torch::Tensor gather_csr_impl(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out,
                              std::optional<int64_t> length, bool divide_by_count) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(indptr);
  if (optional_out.has_value()) TSB_CHECK_CUDA(optional_out.value());
  check_index_dtype(indptr, "indptr");
  c10::cuda::CUDAGuard guard(src.device());

  TSB_CHECK_INPUT(src.dim() >= indptr.dim());
  TSB_CHECK_INPUT(indptr.dim() >= 1);
  auto sizes = indptr.sizes().vec();
  for (int64_t i = 0; i < indptr.dim() - 1; i++) sizes[i] = src.size(i);
  indptr = indptr.expand(sizes);
  const int64_t dim = indptr.dim() - 1;
  TSB_CHECK_INPUT(src.size(dim) == 0 || src.size(dim) == indptr.size(dim) - 1);

  src = src.contiguous();

  torch::Tensor out;
  bool copy_back = false;
  if (optional_out.has_value()) {
    copy_back = !optional_out.value().is_contiguous();
    out = optional_out.value().contiguous();
    TSB_CHECK_INPUT(out.dim() == src.dim());
    TSB_CHECK_INPUT(out.scalar_type() == src.scalar_type());
    for (int64_t i = 0; i < out.dim(); i++)
      if (i != dim) TSB_CHECK_INPUT(src.size(i) == out.size(i));
  } else {
    auto out_sizes = src.sizes().vec();
    if (length.has_value())
      out_sizes[dim] = length.value();
    else if (src.numel() > 0)
      out_sizes[dim] = indptr.flatten()[-1].item<int64_t>();  // host sync, as upstream (segment_csr_cuda.cu:248)
    else
      out_sizes[dim] = 0;
    out = torch::empty(out_sizes, src.options());
  }

  if (src.numel() == 0) {
    if (!optional_out.has_value()) out.fill_(0);
    return out;
  }
  if (length.has_value() && !optional_out.has_value()) out.zero_();  // positions no row covers (a backward pass: no gradient)

  const int64_t B = indptr.numel() / indptr.size(-1);
  const int64_t N = src.size(dim);
  const int64_t E = out.size(dim);
  const int64_t K = src.numel() / (B * N);
  BatchedRows rows = batched_rows(indptr);
  check_status(tsb_gather_csr(src.data_ptr(), rows.ptr(), out.data_ptr(), B, E, K, N, rows.batch_stride,
                              dtype_enum(src), divide_by_count ? 1 : 0, current_stream()),
               "tsb_gather_csr");
  if (copy_back) {
    optional_out.value().copy_(out);
    out = optional_out.value();
  }
  return out;
}

torch::Tensor arg_backward_impl(torch::Tensor grad_out_, torch::Tensor arg_out, std::vector<int64_t> src_shape, int64_t dim) {
  c10::cuda::CUDAGuard guard(grad_out_.device());
  auto grad_out = grad_out_.contiguous();
  auto arg = arg_out.contiguous();
  auto grad_in = torch::empty(src_shape, grad_out.options());
  int64_t B = 1, K = 1;
  for (int64_t i = 0; i < dim; i++) B *= src_shape[i];
  for (size_t i = dim + 1; i < src_shape.size(); i++) K *= src_shape[i];
  const int64_t E = src_shape[dim];
  const int64_t N = grad_out.size(dim);
  check_status(tsb_arg_backward(grad_out.data_ptr(), arg.data_ptr<int64_t>(), grad_in.data_ptr(), B, E, K, N,
                                dtype_enum(grad_out), current_stream()),
               "tsb_arg_backward");
  return grad_in;
}

// dispatcher form: (out, arg_out or a placeholder)
std::tuple<torch::Tensor, torch::Tensor> segment_csr_op(torch::Tensor src, torch::Tensor indptr,
                                                        std::optional<torch::Tensor> optional_out, std::string reduce) {
  auto r = segment_csr_impl(src, indptr, optional_out, reduce);
  return std::make_tuple(std::get<0>(r), std::get<1>(r).has_value() ? std::get<1>(r).value() : no_tensor(indptr));
}
}  // namespace

std::tuple<torch::Tensor, std::optional<torch::Tensor>>
segment_csr_fw(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out,
               const std::string &reduce) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(indptr);
  static auto op = internal_op<std::tuple<torch::Tensor, torch::Tensor>(torch::Tensor, torch::Tensor, std::optional<torch::Tensor>,
                                                                        std::string)>("torch_scatter::_segment_csr_fw");
  auto r = op.call(src, indptr, optional_out, reduce);
  const bool minmax = reduce == "min" || reduce == "max";
  return std::make_tuple(std::get<0>(r), minmax ? std::optional<torch::Tensor>(std::get<1>(r)) : std::nullopt);
}

torch::Tensor gather_csr_fw(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out,
                            bool divide_by_count, std::optional<int64_t> length) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(indptr);
  static auto op = internal_op<torch::Tensor(torch::Tensor, torch::Tensor, std::optional<torch::Tensor>, std::optional<int64_t>,
                                             bool)>("torch_scatter::_gather_csr_fw");
  return op.call(src, indptr, optional_out, length, divide_by_count);
}

torch::Tensor arg_backward(const torch::Tensor &grad_out, const torch::Tensor &arg_out, std::vector<int64_t> src_shape,
                           int64_t dim) {
  static auto op = internal_op<torch::Tensor(torch::Tensor, torch::Tensor, std::vector<int64_t>, int64_t)>(
      "torch_scatter::_arg_backward");
  return op.call(grad_out, arg_out, src_shape, dim);
}

namespace {

using torch::autograd::AutogradContext;
using torch::autograd::Variable;
using torch::autograd::variable_list;

// SUM: backward is gather_csr of the incoming gradient (csrc/segment_csr.cpp:70-78).
// MEAN: the same with each row's gradient divided by the row length, fused (csrc/segment_csr.cpp:94-111).
template <bool MEAN> class SegmentSumMeanCSR : public torch::autograd::Function<SegmentSumMeanCSR<MEAN>> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable indptr,
                               std::optional<Variable> optional_out) {
    ctx->saved_data["src_shape"] = src.sizes();
    auto out = std::get<0>(segment_csr_fw(src, indptr, optional_out, MEAN ? "mean" : "sum"));
    ctx->save_for_backward({indptr});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto grad_out = grad_outs[0];
    auto indptr = ctx->get_saved_variables()[0];
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    // no `out`: an operator that writes into an argument is invisible to a tracing compiler
    auto grad_in = gather_csr_fw(grad_out, indptr, std::nullopt, MEAN, src_shape[indptr.dim() - 1]);
    return {grad_in, Variable(), Variable()};
  }
};

// MIN/MAX: the gradient goes to the arg position only (csrc/segment_csr.cpp:130-142,161-173).
template <bool MAX> class SegmentMinMaxCSR : public torch::autograd::Function<SegmentMinMaxCSR<MAX>> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable indptr,
                               std::optional<Variable> optional_out) {
    ctx->saved_data["src_shape"] = src.sizes();
    auto result = segment_csr_fw(src, indptr, optional_out, MAX ? "max" : "min");
    auto out = std::get<0>(result);
    auto arg_out = std::get<1>(result).value();
    ctx->saved_data["dim"] = (int64_t)(indptr.dim() - 1);
    ctx->save_for_backward({indptr, arg_out});
    ctx->mark_non_differentiable({arg_out});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out, arg_out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    auto grad_in = arg_backward(grad_outs[0], saved[1], src_shape, ctx->saved_data["dim"].toInt());
    return {grad_in, Variable(), Variable()};
  }
};

// gather_csr: backward is a segment sum of the gradient (csrc/segment_csr.cpp:189-198).
class GatherCSR : public torch::autograd::Function<GatherCSR> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable indptr,
                               std::optional<Variable> optional_out) {
    ctx->saved_data["src_shape"] = src.sizes();
    auto out = gather_csr_fw(src, indptr, optional_out, false, std::nullopt);
    ctx->save_for_backward({indptr});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto grad_out = grad_outs[0];
    auto indptr = ctx->get_saved_variables()[0];
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    const int64_t dim = indptr.dim() - 1;
    if (indptr.size(dim) - 1 == src_shape[dim])   // the usual case: no `out`, visible to a tracing compiler
      return {std::get<0>(segment_csr_fw(grad_out, indptr, std::nullopt, "sum")), Variable(), Variable()};
    auto grad_in = torch::empty(src_shape, grad_out.options());
    segment_csr_fw(grad_out, indptr, grad_in, "sum");
    return {grad_in, Variable(), Variable()};
  }
};

torch::Tensor segment_sum_csr(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out) {
  return SegmentSumMeanCSR<false>::apply(src, indptr, optional_out)[0];
}
torch::Tensor segment_mean_csr(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out) {
  return SegmentSumMeanCSR<true>::apply(src, indptr, optional_out)[0];
}
std::tuple<torch::Tensor, torch::Tensor> segment_min_csr(torch::Tensor src, torch::Tensor indptr,
                                                         std::optional<torch::Tensor> optional_out) {
  auto result = SegmentMinMaxCSR<false>::apply(src, indptr, optional_out);
  return std::make_tuple(result[0], result[1]);
}
std::tuple<torch::Tensor, torch::Tensor> segment_max_csr(torch::Tensor src, torch::Tensor indptr,
                                                         std::optional<torch::Tensor> optional_out) {
  auto result = SegmentMinMaxCSR<true>::apply(src, indptr, optional_out);
  return std::make_tuple(result[0], result[1]);
}
torch::Tensor gather_csr(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out) {
  return GatherCSR::apply(src, indptr, optional_out)[0];
}
int64_t cuda_version() { return tsb_cuda_version(); }

}  // namespace
}  // namespace tsb_ops

TORCH_LIBRARY_FRAGMENT(torch_scatter, m) {
  m.def("segment_sum_csr", &tsb_ops::segment_sum_csr);
  m.def("segment_mean_csr", &tsb_ops::segment_mean_csr);
  m.def("segment_min_csr", &tsb_ops::segment_min_csr);
  m.def("segment_max_csr", &tsb_ops::segment_max_csr);
  m.def("gather_csr", &tsb_ops::gather_csr);
  m.def("cuda_version", &tsb_ops::cuda_version);
  // the data-touching halves (see ops_common.h)
  m.def("_segment_csr_fw(Tensor src, Tensor indptr, Tensor? out, str reduce) -> (Tensor, Tensor)");
  m.def("_gather_csr_fw(Tensor src, Tensor indptr, Tensor? out, int? length, bool divide_by_count) -> Tensor");
  m.def("_arg_backward(Tensor grad_out, Tensor arg_out, int[] src_shape, int dim) -> Tensor");
}

TORCH_LIBRARY_IMPL(torch_scatter, CUDA, m) {
  m.impl("_segment_csr_fw", &tsb_ops::segment_csr_op);
  m.impl("_gather_csr_fw", &tsb_ops::gather_csr_impl);
  m.impl("_arg_backward", &tsb_ops::arg_backward_impl);
}

// torch_scatter::segment_{sum,mean,min,max}_coo and torch_scatter::gather_coo: schemas and
// autograd behaviour of the upstream registry (csrc/segment_coo.cpp:57-246) on top of the tsb200 C ABI.
#include "ops_common.h"

namespace tsb_ops {

namespace {
std::tuple<torch::Tensor, std::optional<torch::Tensor>>
segment_coo_impl(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
                 std::optional<int64_t> dim_size, const std::string &reduce) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  if (optional_out.has_value()) TSB_CHECK_CUDA(optional_out.value());
  check_index_dtype(index, "index");
  c10::cuda::CUDAGuard guard(src.device());

  TSB_CHECK_INPUT(src.dim() >= index.dim());
  TSB_CHECK_INPUT(index.dim() >= 1);
  auto sizes = index.sizes().vec();
  for (int64_t i = 0; i < index.dim(); i++) sizes[i] = src.size(i);
  index = index.expand(sizes);
  const int64_t dim = index.dim() - 1;

  src = src.contiguous();
  const int red = reduce_enum(reduce);
  TORCH_CHECK(red != TSB_MUL, "segment_coo does not support reduce='mul'");

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
    sizes = src.sizes().vec();
    if (dim_size.has_value())
      sizes[dim] = dim_size.value();
    else if (index.numel() == 0)
      sizes[dim] = 0;
    else {
      // host sync, as upstream (segment_coo_cuda.cu:186-190): the index is sorted, so its last
      // column holds the largest target of each batch
      auto tmp = index.select(dim, index.size(dim) - 1);
      tmp = tmp.numel() > 1 ? tmp.max() : tmp;
      sizes[dim] = 1 + tmp.item<int64_t>();
    }
    out = torch::empty(sizes, src.options());
  }

  const bool minmax = red == TSB_MIN || red == TSB_MAX;
  std::optional<torch::Tensor> arg_out = std::nullopt;
  auto count_sizes = index.sizes().vec();
  count_sizes[dim] = out.size(dim);

  if (src.numel() == 0) {
    if (minmax) arg_out = torch::full_like(out, src.size(dim), index.options());
    else if (red == TSB_MEAN) arg_out = torch::zeros(count_sizes, out.options());
    if (!optional_out.has_value()) out.fill_(0);
    return std::make_tuple(out, arg_out);
  }
  if (minmax) arg_out = torch::empty(out.sizes(), index.options());
  else if (red == TSB_MEAN) arg_out = torch::empty(count_sizes, out.options());

  const int64_t E = src.size(dim);
  const int64_t B = index.numel() / E;
  const int64_t K = src.numel() / index.numel();
  const int64_t N = out.size(dim);
  if (out.numel() > 0) {
    BatchedRows rows = batched_rows(index);
    const size_t ws_bytes = tsb_segment_coo_workspace_bytes(B, E, K, N, dtype_enum(src), red);
    auto workspace = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kUInt8));
    check_status(tsb_segment_coo(src.data_ptr(), rows.ptr(), out.data_ptr(),
                                 minmax ? arg_out.value().data_ptr<int64_t>() : nullptr,
                                 red == TSB_MEAN ? arg_out.value().data_ptr() : nullptr, B, E, K, N,
                                 rows.batch_stride, dtype_enum(src), red, optional_out.has_value() ? 1 : 0,
                                 workspace.data_ptr(), ws_bytes, current_stream()),
                 "tsb_segment_coo");
  }
  if (copy_back) {
    optional_out.value().copy_(out);
    out = optional_out.value();
  }
  return std::make_tuple(out, arg_out);
}

torch::Tensor gather_coo_impl(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
                              std::optional<torch::Tensor> count) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  if (optional_out.has_value()) TSB_CHECK_CUDA(optional_out.value());
  check_index_dtype(index, "index");
  c10::cuda::CUDAGuard guard(src.device());

  TSB_CHECK_INPUT(src.dim() >= index.dim());
  TSB_CHECK_INPUT(index.dim() >= 1);
  const int64_t dim = index.dim() - 1;
  {
    // leading dims of the index broadcast against src's, as upstream does (csrc/cuda/segment_coo_cuda.cu:337-340);
    // a stride-0 batch dim stays one shared row (batched_rows below)
    auto lead = index.sizes().vec();
    for (int64_t i = 0; i < dim; i++) {
      TSB_CHECK_INPUT(index.size(i) == src.size(i) || index.size(i) == 1);
      lead[i] = src.size(i);
    }
    index = index.expand(lead);
  }

  src = src.contiguous();

  torch::Tensor out;
  bool copy_back = false;
  if (optional_out.has_value()) {
    copy_back = !optional_out.value().is_contiguous();
    out = optional_out.value().contiguous();
    TSB_CHECK_INPUT(out.dim() == src.dim());
    TSB_CHECK_INPUT(out.scalar_type() == src.scalar_type());
    for (int64_t i = 0; i < src.dim(); i++)
      if (i != dim) TSB_CHECK_INPUT(src.size(i) == out.size(i));
    TSB_CHECK_INPUT(out.size(dim) == index.size(dim));
  } else {
    auto sizes = src.sizes().vec();
    sizes[dim] = index.size(dim);
    out = torch::empty(sizes, src.options());
  }

  if (src.numel() == 0) {
    if (!optional_out.has_value()) out.fill_(0);
    return out;
  }
  if (out.numel() == 0) return out;

  const int64_t E = index.size(dim);
  const int64_t B = index.numel() / E;
  const int64_t K = out.numel() / index.numel();
  const int64_t N = src.size(dim);
  BatchedRows rows = batched_rows(index);
  torch::Tensor count_c;
  if (count.has_value()) count_c = count.value().contiguous();
  check_status(tsb_gather_coo(src.data_ptr(), rows.ptr(), out.data_ptr(),
                              count.has_value() ? count_c.data_ptr() : nullptr, B, E, K, N, rows.batch_stride,
                              dtype_enum(src), current_stream()),
               "tsb_gather_coo");
  if (copy_back) {
    optional_out.value().copy_(out);
    out = optional_out.value();
  }
  return out;
}

// dispatcher form: (out, arg_out for MIN/MAX, count for MEAN, else a placeholder)
std::tuple<torch::Tensor, torch::Tensor> segment_coo_op(torch::Tensor src, torch::Tensor index,
                                                        std::optional<torch::Tensor> optional_out,
                                                        std::optional<int64_t> dim_size, std::string reduce) {
  auto r = segment_coo_impl(src, index, optional_out, dim_size, reduce);
  return std::make_tuple(std::get<0>(r), std::get<1>(r).has_value() ? std::get<1>(r).value() : no_tensor(index));
}
}  // namespace

std::tuple<torch::Tensor, std::optional<torch::Tensor>>
segment_coo_fw(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
               std::optional<int64_t> dim_size, const std::string &reduce) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  static auto op = internal_op<std::tuple<torch::Tensor, torch::Tensor>(torch::Tensor, torch::Tensor, std::optional<torch::Tensor>,
                                                                        std::optional<int64_t>, std::string)>(
      "torch_scatter::_segment_coo_fw");
  auto r = op.call(src, index, optional_out, dim_size, reduce);
  const bool extra = reduce == "min" || reduce == "max" || reduce == "mean";
  return std::make_tuple(std::get<0>(r), extra ? std::optional<torch::Tensor>(std::get<1>(r)) : std::nullopt);
}

torch::Tensor gather_coo_fw(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
                            std::optional<torch::Tensor> count) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  static auto op = internal_op<torch::Tensor(torch::Tensor, torch::Tensor, std::optional<torch::Tensor>,
                                             std::optional<torch::Tensor>)>("torch_scatter::_gather_coo_fw");
  return op.call(src, index, optional_out, count);
}

namespace {

using torch::autograd::AutogradContext;
using torch::autograd::Variable;
using torch::autograd::variable_list;

// backward of SUM is gather_coo (csrc/segment_coo.cpp:72-80)
class SegmentSumCOO : public torch::autograd::Function<SegmentSumCOO> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index,
                               std::optional<Variable> optional_out, std::optional<int64_t> dim_size) {
    ctx->saved_data["src_shape"] = src.sizes();
    auto out = std::get<0>(segment_coo_fw(src, index, optional_out, dim_size, "sum"));
    ctx->save_for_backward({index});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto grad_out = grad_outs[0];
    auto index = ctx->get_saved_variables()[0];
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    // no `out`: an operator that writes into an argument is invisible to a tracing compiler
    auto grad_in = gather_coo_fw(grad_out, index, std::nullopt, std::nullopt);
    return {grad_in, Variable(), Variable(), Variable()};
  }
};

// backward of MEAN is gather_coo divided by the gathered count, fused (csrc/segment_coo.cpp:99-112)
class SegmentMeanCOO : public torch::autograd::Function<SegmentMeanCOO> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index,
                               std::optional<Variable> optional_out, std::optional<int64_t> dim_size) {
    ctx->saved_data["src_shape"] = src.sizes();
    auto result = segment_coo_fw(src, index, optional_out, dim_size, "mean");
    auto out = std::get<0>(result);
    auto count = std::get<1>(result).value();
    ctx->save_for_backward({index, count});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto grad_out = grad_outs[0];
    auto saved = ctx->get_saved_variables();
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    auto grad_in = gather_coo_fw(grad_out, saved[0], std::nullopt, saved[1].to(grad_out.scalar_type()));
    return {grad_in, Variable(), Variable(), Variable()};
  }
};

template <bool MAX> class SegmentMinMaxCOO : public torch::autograd::Function<SegmentMinMaxCOO<MAX>> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index,
                               std::optional<Variable> optional_out, std::optional<int64_t> dim_size) {
    ctx->saved_data["src_shape"] = src.sizes();
    ctx->saved_data["dim"] = (int64_t)(index.dim() - 1);
    auto result = segment_coo_fw(src, index, optional_out, dim_size, MAX ? "max" : "min");
    auto out = std::get<0>(result);
    auto arg_out = std::get<1>(result).value();
    ctx->save_for_backward({index, arg_out});
    ctx->mark_non_differentiable({arg_out});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out, arg_out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    auto grad_in = arg_backward(grad_outs[0], saved[1], src_shape, ctx->saved_data["dim"].toInt());
    return {grad_in, Variable(), Variable(), Variable()};
  }
};

// backward of gather_coo is a segment sum into zeros (csrc/segment_coo.cpp:192-201)
class GatherCOO : public torch::autograd::Function<GatherCOO> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index,
                               std::optional<Variable> optional_out) {
    ctx->saved_data["src_shape"] = src.sizes();
    auto out = gather_coo_fw(src, index, optional_out, std::nullopt);
    ctx->save_for_backward({index});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto grad_out = grad_outs[0];
    auto index = ctx->get_saved_variables()[0];
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    auto grad_in = std::get<0>(segment_coo_fw(grad_out, index, std::nullopt, src_shape[index.dim() - 1], "sum"));
    return {grad_in, Variable(), Variable()};
  }
};

torch::Tensor segment_sum_coo(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
                              std::optional<int64_t> dim_size) {
  return SegmentSumCOO::apply(src, index, optional_out, dim_size)[0];
}
torch::Tensor segment_mean_coo(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out,
                               std::optional<int64_t> dim_size) {
  return SegmentMeanCOO::apply(src, index, optional_out, dim_size)[0];
}
std::tuple<torch::Tensor, torch::Tensor> segment_min_coo(torch::Tensor src, torch::Tensor index,
                                                         std::optional<torch::Tensor> optional_out,
                                                         std::optional<int64_t> dim_size) {
  auto result = SegmentMinMaxCOO<false>::apply(src, index, optional_out, dim_size);
  return std::make_tuple(result[0], result[1]);
}
std::tuple<torch::Tensor, torch::Tensor> segment_max_coo(torch::Tensor src, torch::Tensor index,
                                                         std::optional<torch::Tensor> optional_out,
                                                         std::optional<int64_t> dim_size) {
  auto result = SegmentMinMaxCOO<true>::apply(src, index, optional_out, dim_size);
  return std::make_tuple(result[0], result[1]);
}
torch::Tensor gather_coo(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out) {
  return GatherCOO::apply(src, index, optional_out)[0];
}

}  // namespace
}  // namespace tsb_ops

TORCH_LIBRARY_FRAGMENT(torch_scatter, m) {
  m.def("segment_sum_coo", &tsb_ops::segment_sum_coo);
  m.def("segment_mean_coo", &tsb_ops::segment_mean_coo);
  m.def("segment_min_coo", &tsb_ops::segment_min_coo);
  m.def("segment_max_coo", &tsb_ops::segment_max_coo);
  m.def("gather_coo", &tsb_ops::gather_coo);
  // the data-touching halves (see ops_common.h)
  m.def("_segment_coo_fw(Tensor src, Tensor index, Tensor? out, int? dim_size, str reduce) -> (Tensor, Tensor)");
  m.def("_gather_coo_fw(Tensor src, Tensor index, Tensor? out, Tensor? count) -> Tensor");
}

TORCH_LIBRARY_IMPL(torch_scatter, CUDA, m) {
  m.impl("_segment_coo_fw", &tsb_ops::segment_coo_op);
  m.impl("_gather_coo_fw", &tsb_ops::gather_coo_impl);
}

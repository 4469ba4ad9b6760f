// torch_scatter::scatter_{sum,mul,mean,min,max}: schemas and autograd behaviour of the upstream
// registry (csrc/scatter.cpp:54-277) on top of the tsb200 C ABI.  Unlike upstream, the Python
// scatter_sum / scatter_mean wrappers route here too instead of to ATen's scatter_add_.
#include "ops_common.h"

namespace tsb_ops {
namespace {

// index broadcast to src's shape (csrc/scatter.cpp:25-33)
torch::Tensor broadcast(torch::Tensor src, torch::Tensor other, int64_t dim) {
  if (src.dim() == 1)
    for (int64_t i = 0; i < dim; i++) src = src.unsqueeze(0);
  for (int64_t i = src.dim(); i < other.dim(); i++) src = src.unsqueeze(-1);
  src = src.expand(other.sizes().vec());
  return src;
}

// Stride of the dims [lo,hi) of `t` seen as one flattened dim, if such a single stride exists.
bool collapse_stride(const torch::Tensor &t, int64_t lo, int64_t hi, int64_t *stride) {
  int64_t s = 0;      // stride of the innermost non-trivial dim seen so far
  int64_t span = 1;   // number of elements that dim block covers
  bool any = false;
  for (int64_t i = hi - 1; i >= lo; i--) {
    if (t.size(i) == 1) continue;
    if (!any) {
      s = t.stride(i);
      span = t.size(i);
      any = true;
    } else {
      if (t.stride(i) != s * span) return false;
      span *= t.size(i);
    }
  }
  *stride = any ? s : 0;
  return true;
}

// The broadcast index as (tensor kept alive, strides over the flattened [B,E,K] view).
struct FlatIndex {
  torch::Tensor holder;
  int64_t sb, se, sk;
};

FlatIndex flatten_index(const torch::Tensor &index, int64_t dim) {
  FlatIndex f;
  f.holder = index;
  const int64_t nd = index.dim();
  if (collapse_stride(index, 0, dim, &f.sb) && collapse_stride(index, dim + 1, nd, &f.sk)) {
    f.se = index.size(dim) == 1 ? 0 : index.stride(dim);
    return f;
  }
  f.holder = index.contiguous();
  int64_t K = 1;
  for (int64_t i = dim + 1; i < nd; i++) K *= index.size(i);
  f.sk = K == 1 ? 0 : 1;
  f.se = K;
  f.sb = K * index.size(dim);
  return f;
}

struct ScatterResult {
  torch::Tensor out;
  std::optional<torch::Tensor> arg_out;
  std::optional<torch::Tensor> count;  // int32, MEAN only
};

// index must already be broadcast to src's shape.
ScatterResult scatter_impl(torch::Tensor src, torch::Tensor index, int64_t dim,
                           std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size,
                           const std::string &reduce) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  if (optional_out.has_value()) TSB_CHECK_CUDA(optional_out.value());
  check_index_dtype(index, "index");
  c10::cuda::CUDAGuard guard(src.device());

  TSB_CHECK_INPUT(src.dim() == index.dim());
  TSB_CHECK_INPUT(dim >= 0 && dim < src.dim());
  for (int64_t i = 0; i < index.dim(); i++) TSB_CHECK_INPUT(src.size(i) == index.size(i));

  src = src.contiguous();
  const int red = reduce_enum(reduce);

  ScatterResult r;
  bool copy_back = false;
  if (optional_out.has_value()) {
    copy_back = !optional_out.value().is_contiguous();
    r.out = optional_out.value().contiguous();
    TSB_CHECK_INPUT(r.out.dim() == src.dim());
    TSB_CHECK_INPUT(r.out.scalar_type() == src.scalar_type());
    for (int64_t i = 0; i < r.out.dim(); i++)
      if (i != dim) TSB_CHECK_INPUT(src.size(i) == r.out.size(i));
  } else {
    auto sizes = src.sizes().vec();
    if (dim_size.has_value())
      sizes[dim] = dim_size.value();
    else if (index.numel() == 0)
      sizes[dim] = 0;
    else
      sizes[dim] = 1 + index.max().item<int64_t>();  // host sync, as upstream (scatter_cuda.cu:87)
    r.out = torch::empty(sizes, src.options());
  }

  const bool minmax = red == TSB_MIN || red == TSB_MAX;
  int64_t B = 1;
  for (int64_t i = 0; i < dim; i++) B *= src.size(i);
  const int64_t E = src.size(dim);
  int64_t K = 1;
  for (int64_t i = dim + 1; i < src.dim(); i++) K *= src.size(i);
  const int64_t N = r.out.size(dim);

  if (src.numel() == 0) {
    if (minmax) r.arg_out = torch::full_like(r.out, src.size(dim), index.options());
    if (red == TSB_MEAN) r.count = torch::ones({1}, index.options().dtype(torch::kInt32));
    if (!optional_out.has_value()) r.out.fill_(0);
    return r;
  }

  FlatIndex fi = flatten_index(index, dim);
  if (minmax) r.arg_out = torch::empty(r.out.sizes(), index.options());
  if (red == TSB_MEAN) {
    // element counts over the dims the index really varies in (torch_scatter/scatter.py:52-61)
    r.count = torch::empty({fi.sb ? B : 1, N, fi.sk ? K : 1}, index.options().dtype(torch::kInt32));
  }
  if (r.out.numel() > 0) {
    const size_t ws_bytes = tsb_scatter_workspace_bytes(B, E, K, N, dtype_enum(src), red);
    auto workspace = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kUInt8));
    check_status(tsb_scatter(src.data_ptr(), fi.holder.data_ptr<int64_t>(), r.out.data_ptr(),
                             minmax ? r.arg_out.value().data_ptr<int64_t>() : nullptr,
                             red == TSB_MEAN ? r.count.value().data_ptr<int32_t>() : nullptr, B, E, K, N, fi.sb,
                             fi.se, fi.sk, dtype_enum(src), red, optional_out.has_value() ? 1 : 0,
                             workspace.data_ptr(), ws_bytes, current_stream()),
                 "tsb_scatter");
  }
  if (copy_back) {
    optional_out.value().copy_(r.out);
    r.out = optional_out.value();
  }
  return r;
}

// dispatcher form of the forward: (out, arg_out for MIN/MAX, int32 count for MEAN; placeholders otherwise)
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> scatter_op(torch::Tensor src, torch::Tensor index, int64_t dim,
                                                                   std::optional<torch::Tensor> optional_out,
                                                                   std::optional<int64_t> dim_size, std::string reduce) {
  auto r = scatter_impl(src, index, dim, optional_out, dim_size, reduce);
  return std::make_tuple(r.out, r.arg_out.has_value() ? r.arg_out.value() : no_tensor(index),
                         r.count.has_value() ? r.count.value() : no_tensor(index));
}

ScatterResult scatter_fw(torch::Tensor src, torch::Tensor index, int64_t dim, std::optional<torch::Tensor> optional_out,
                         std::optional<int64_t> dim_size, const std::string &reduce) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  static auto op = internal_op<std::tuple<torch::Tensor, torch::Tensor, torch::Tensor>(
      torch::Tensor, torch::Tensor, int64_t, std::optional<torch::Tensor>, std::optional<int64_t>, std::string)>(
      "torch_scatter::_scatter_fw");
  auto t = op.call(src, index, dim, optional_out, dim_size, reduce);
  ScatterResult r;
  r.out = std::get<0>(t);
  if (reduce == "min" || reduce == "max") r.arg_out = std::get<1>(t);
  if (reduce == "mean") r.count = std::get<2>(t);
  return r;
}

// grad_in[b,e,k] = grad_out[b, index(b,e,k), k] (/ count): the gather behind SUM / MEAN / MUL backward.
torch::Tensor scatter_bw_impl(torch::Tensor grad_out_, torch::Tensor index, int64_t dim, std::vector<int64_t> src_shape,
                              std::optional<torch::Tensor> count) {
  c10::cuda::CUDAGuard guard(grad_out_.device());
  auto grad_out = grad_out_.contiguous();
  auto grad_in = torch::empty(src_shape, grad_out.options());
  if (grad_in.numel() == 0) return grad_in;
  int64_t B = 1, K = 1;
  for (int64_t i = 0; i < dim; i++) B *= src_shape[i];
  for (size_t i = dim + 1; i < src_shape.size(); i++) K *= src_shape[i];
  const int64_t E = src_shape[dim];
  const int64_t N = grad_out.size(dim);
  FlatIndex fi = flatten_index(index, dim);
  check_status(tsb_scatter_backward(grad_out.data_ptr(), fi.holder.data_ptr<int64_t>(), grad_in.data_ptr(),
                                    count.has_value() ? count.value().data_ptr<int32_t>() : nullptr, B, E, K, N,
                                    fi.sb, fi.se, fi.sk, dtype_enum(grad_out), current_stream()),
               "tsb_scatter_backward");
  return grad_in;
}

torch::Tensor scatter_bw(const torch::Tensor &grad_out, const torch::Tensor &index, int64_t dim,
                         const std::vector<int64_t> &src_shape, std::optional<torch::Tensor> count) {
  static auto op = internal_op<torch::Tensor(torch::Tensor, torch::Tensor, int64_t, std::vector<int64_t>,
                                             std::optional<torch::Tensor>)>("torch_scatter::_scatter_bw");
  return op.call(grad_out, index, dim, src_shape, count);
}

using torch::autograd::AutogradContext;
using torch::autograd::Variable;
using torch::autograd::variable_list;

// SUM (csrc/scatter.cpp:54-81) and MEAN (csrc/scatter.cpp:115-161; the count and the divide are
// fused into the forward kernels, the gathered-count divide into the backward kernel).
template <bool MEAN> class ScatterSumMean : public torch::autograd::Function<ScatterSumMean<MEAN>> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim,
                               std::optional<Variable> optional_out, std::optional<int64_t> dim_size) {
    dim = dim < 0 ? src.dim() + dim : dim;
    ctx->saved_data["dim"] = dim;
    ctx->saved_data["src_shape"] = src.sizes();
    index = broadcast(index, src, dim);
    auto result = scatter_fw(src, index, dim, optional_out, dim_size, MEAN ? "mean" : "sum");
    if (MEAN) ctx->save_for_backward({index, result.count.value()});
    else ctx->save_for_backward({index});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {result.out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto dim = ctx->saved_data["dim"].toInt();
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    std::optional<torch::Tensor> count = std::nullopt;
    if (MEAN) count = saved[1];
    auto grad_in = scatter_bw(grad_outs[0], saved[0], dim, src_shape, count);
    return {grad_in, Variable(), Variable(), Variable(), Variable()};
  }
};

// MUL (csrc/scatter.cpp:83-113)
class ScatterMul : public torch::autograd::Function<ScatterMul> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim,
                               std::optional<Variable> optional_out, std::optional<int64_t> dim_size) {
    dim = dim < 0 ? src.dim() + dim : dim;
    ctx->saved_data["dim"] = dim;
    ctx->saved_data["src_shape"] = src.sizes();
    index = broadcast(index, src, dim);
    auto result = scatter_fw(src, index, dim, optional_out, dim_size, "mul");
    ctx->save_for_backward({src, index, result.out});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {result.out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto src = saved[0];
    auto index = saved[1];
    auto out = saved[2];
    auto dim = ctx->saved_data["dim"].toInt();
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    auto grad_in = scatter_bw(grad_outs[0] * out, index, dim, src_shape, std::nullopt).div_(src);
    grad_in.masked_fill_(grad_in.isnan(), 0);
    return {grad_in, Variable(), Variable(), Variable(), Variable()};
  }
};

// MIN / MAX (csrc/scatter.cpp:163-233)
template <bool MAX> class ScatterMinMax : public torch::autograd::Function<ScatterMinMax<MAX>> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim,
                               std::optional<Variable> optional_out, std::optional<int64_t> dim_size) {
    dim = dim < 0 ? src.dim() + dim : dim;
    ctx->saved_data["dim"] = dim;
    ctx->saved_data["src_shape"] = src.sizes();
    index = broadcast(index, src, dim);
    auto result = scatter_fw(src, index, dim, optional_out, dim_size, MAX ? "max" : "min");
    auto arg_out = result.arg_out.value();
    ctx->save_for_backward({index, arg_out});
    ctx->mark_non_differentiable({arg_out});
    if (optional_out.has_value()) ctx->mark_dirty({optional_out.value()});
    return {result.out, arg_out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto dim = ctx->saved_data["dim"].toInt();
    auto src_shape = list2vec(ctx->saved_data["src_shape"].toIntList());
    auto grad_in = arg_backward(grad_outs[0], saved[1], src_shape, dim);
    return {grad_in, Variable(), Variable(), Variable(), Variable()};
  }
};

// Read-back used by the composites: out[.., e, ..] = src[.., index[e], ..] along `dim` for an index in
// any order (the backward kernel of scatter sum used as a forward); its own backward is a scatter sum.
class GatherRows : public torch::autograd::Function<GatherRows> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim) {
    dim = dim < 0 ? src.dim() + dim : dim;
    TSB_CHECK_CUDA(src);
    TSB_CHECK_CUDA(index);
    check_index_dtype(index, "index");
    auto shape = src.sizes().vec();
    ctx->saved_data["dim"] = dim;
    ctx->saved_data["dim_size"] = shape[dim];
    shape[dim] = index.dim() == 1 ? index.size(0) : index.size(dim);
    auto like = torch::empty(shape, src.options().device(torch::kMeta));
    index = broadcast(index, like, dim);
    ctx->save_for_backward({index});
    return {scatter_bw(src, index, dim, shape, std::nullopt)};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto index = ctx->get_saved_variables()[0];
    auto dim = ctx->saved_data["dim"].toInt();
    auto result = scatter_fw(grad_outs[0], index, dim, std::nullopt, ctx->saved_data["dim_size"].toInt(), "sum");
    return {result.out, Variable(), Variable()};
  }
};

torch::Tensor gather_rows(torch::Tensor src, torch::Tensor index, int64_t dim) {
  return GatherRows::apply(src, index, dim)[0];
}

// Sharded building block: sums of this rank's edges (src [E, ...], 1-D index [E]) into the target rows
// [row_lo, row_hi) of `partial` [N, ...], which is held in accumulation precision (fp32 for 16-bit sources).
// Not differentiable; used by pytorch_scatter_b200.dist to overlap the collective with the next slice.
torch::Tensor scatter_sum_slice(torch::Tensor src, torch::Tensor index, torch::Tensor partial, int64_t row_lo,
                                int64_t row_hi) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(index);
  TSB_CHECK_CUDA(partial);
  check_index_dtype(index, "index");
  c10::cuda::CUDAGuard guard(src.device());
  TSB_CHECK_INPUT(index.dim() == 1 && src.dim() >= 1 && src.size(0) == index.size(0));
  TSB_CHECK_INPUT(partial.dim() == src.dim() && partial.is_contiguous());
  for (int64_t i = 1; i < src.dim(); i++) TSB_CHECK_INPUT(src.size(i) == partial.size(i));
  const bool k16 = src.scalar_type() == at::ScalarType::Half || src.scalar_type() == at::ScalarType::BFloat16;
  TORCH_CHECK(partial.scalar_type() == (k16 ? at::ScalarType::Float : src.scalar_type()),
              "partial must be float32 for 16-bit sources and of the source dtype otherwise");
  src = src.contiguous();
  index = index.contiguous();
  const int64_t E = src.size(0), N = partial.size(0);
  const int64_t K = E > 0 ? src.numel() / E : (N > 0 ? partial.numel() / N : 0);
  auto workspace = torch::empty({256}, src.options().dtype(torch::kUInt8));
  check_status(tsb_scatter_sum_slice(src.data_ptr(), index.data_ptr<int64_t>(), partial.data_ptr(), E, K, N,
                                     dtype_enum(src), row_lo, row_hi, workspace.data_ptr(), 256, current_stream()),
               "tsb_scatter_sum_slice");
  return partial;
}

// Sharded building blocks of the atomics-free path.  scatter_group: entry ids grouped by target row,
// (rowptr int64 [N+1], perm int32 [E]).  segment_sum_perm: sums src rows through that grouping into the rows
// [row_lo, row_hi) of `partial` [N, ...] (same dtype as src; 16-bit sources accumulate in fp32 registers and
// are rounded once).  Not differentiable.
std::tuple<torch::Tensor, torch::Tensor> scatter_group(torch::Tensor index, int64_t dim_size) {
  TSB_CHECK_CUDA(index);
  check_index_dtype(index, "index");
  TSB_CHECK_INPUT(index.dim() == 1 && dim_size >= 1);
  c10::cuda::CUDAGuard guard(index.device());
  index = index.contiguous();
  const int64_t E = index.numel();
  auto rowptr = torch::empty({dim_size + 1}, index.options());
  auto perm = torch::empty({E}, index.options().dtype(torch::kInt32));
  auto count = torch::empty({dim_size}, index.options().dtype(torch::kInt32));
  const size_t ws_bytes = tsb_scatter_group_workspace_bytes(E, dim_size);
  auto workspace = torch::empty({(int64_t)ws_bytes}, index.options().dtype(torch::kUInt8));
  check_status(tsb_scatter_group(index.data_ptr<int64_t>(), E, dim_size, rowptr.data_ptr<int64_t>(),
                                 perm.data_ptr<int32_t>(), count.data_ptr<int32_t>(), workspace.data_ptr(), ws_bytes,
                                 current_stream()),
               "tsb_scatter_group");
  return std::make_tuple(rowptr, perm);
}

torch::Tensor segment_sum_perm(torch::Tensor src, torch::Tensor rowptr, torch::Tensor perm, torch::Tensor partial,
                               int64_t row_lo, int64_t row_hi) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(rowptr);
  TSB_CHECK_CUDA(perm);
  TSB_CHECK_CUDA(partial);
  check_index_dtype(rowptr, "rowptr");
  TORCH_CHECK(perm.scalar_type() == at::ScalarType::Int, "perm must be int32");
  c10::cuda::CUDAGuard guard(src.device());
  TSB_CHECK_INPUT(rowptr.dim() == 1 && perm.dim() == 1 && src.dim() >= 1 && src.size(0) == perm.size(0));
  TSB_CHECK_INPUT(partial.dim() == src.dim() && partial.is_contiguous() && rowptr.is_contiguous() && perm.is_contiguous());
  TSB_CHECK_INPUT(partial.size(0) + 1 == rowptr.size(0) && partial.scalar_type() == src.scalar_type());
  for (int64_t i = 1; i < src.dim(); i++) TSB_CHECK_INPUT(src.size(i) == partial.size(i));
  src = src.contiguous();
  const int64_t E = src.size(0), N = partial.size(0);
  const int64_t K = E > 0 ? src.numel() / E : (N > 0 ? partial.numel() / N : 0);
  const size_t ws_bytes = tsb_segment_csr_perm_workspace_bytes(1, E, K, N, dtype_enum(src), TSB_SUM);
  auto workspace = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kUInt8));
  check_status(tsb_segment_csr_perm(src.data_ptr(), rowptr.data_ptr<int64_t>(), perm.data_ptr<int32_t>(),
                                    partial.data_ptr(), nullptr, 1, E, K, N, row_lo, row_hi, dtype_enum(src), TSB_SUM, 0,
                                    workspace.data_ptr(), ws_bytes, current_stream()),
               "tsb_segment_csr_perm");
  return partial;
}

// The same reduction with every finished row stored straight into its owner's staging buffer
// (owner_ptrs: device addresses of the `world` buffers [world, rows_per_owner, ...], peers included).
void segment_sum_perm_routed(torch::Tensor src, torch::Tensor rowptr, torch::Tensor perm, std::vector<int64_t> owner_ptrs,
                             int64_t rank, int64_t rows_per_owner, int64_t dim_size, bool wide_staging) {
  TSB_CHECK_CUDA(src);
  TSB_CHECK_CUDA(rowptr);
  TSB_CHECK_CUDA(perm);
  check_index_dtype(rowptr, "rowptr");
  TORCH_CHECK(perm.scalar_type() == at::ScalarType::Int, "perm must be int32");
  c10::cuda::CUDAGuard guard(src.device());
  TSB_CHECK_INPUT(rowptr.dim() == 1 && perm.dim() == 1 && src.dim() >= 1 && src.size(0) == perm.size(0));
  TSB_CHECK_INPUT(rowptr.is_contiguous() && perm.is_contiguous() && rowptr.size(0) == dim_size + 1);
  const int world = (int)owner_ptrs.size();
  TSB_CHECK_INPUT(world >= 1 && world <= 8 && rank >= 0 && rank < world && rows_per_owner * world >= dim_size);
  src = src.contiguous();
  const int64_t E = src.size(0);
  int64_t K = 1;
  for (int64_t i = 1; i < src.dim(); i++) K *= src.size(i);
  std::vector<void *> bases(world);
  for (int q = 0; q < world; ++q) bases[q] = reinterpret_cast<void *>(owner_ptrs[q]);
  const size_t ws_bytes = tsb_segment_csr_perm_workspace_bytes(1, E, K, dim_size, dtype_enum(src), TSB_SUM);
  auto workspace = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kUInt8));
  check_status(tsb_segment_csr_perm_routed(src.data_ptr(), rowptr.data_ptr<int64_t>(), perm.data_ptr<int32_t>(),
                                           bases.data(), world, (int)rank, rows_per_owner, wide_staging ? 1 : 0, E, K, dim_size, dtype_enum(src),
                                           TSB_SUM, workspace.data_ptr(), ws_bytes, current_stream()),
               "tsb_segment_csr_perm_routed");
}

// slabs [world, ...] -> their sum over dim 0 (the owner's last step of the routed scatter), in `dtype`; the slabs
// hold `dtype` or, for fp16 / bf16 results, fp32 partial sums
torch::Tensor sum_slabs(torch::Tensor slabs, at::ScalarType dtype) {
  TSB_CHECK_CUDA(slabs);
  TSB_CHECK_INPUT(slabs.dim() >= 1 && slabs.is_contiguous());
  const bool wide = slabs.scalar_type() != dtype;
  TSB_CHECK_INPUT(!wide || (slabs.scalar_type() == at::ScalarType::Float &&
                            (dtype == at::ScalarType::Half || dtype == at::ScalarType::BFloat16)));
  c10::cuda::CUDAGuard guard(slabs.device());
  auto out = torch::empty(slabs.sizes().slice(1), slabs.options().dtype(dtype));
  check_status(tsb_sum_slabs(slabs.data_ptr(), out.data_ptr(), (int)slabs.size(0), out.numel(), dtype_enum(out),
                             wide ? 1 : 0, current_stream()),
               "tsb_sum_slabs");
  return out;
}

torch::Tensor scatter_sum(torch::Tensor src, torch::Tensor index, int64_t dim,
                          std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size) {
  return ScatterSumMean<false>::apply(src, index, dim, optional_out, dim_size)[0];
}
torch::Tensor scatter_mul(torch::Tensor src, torch::Tensor index, int64_t dim,
                          std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size) {
  return ScatterMul::apply(src, index, dim, optional_out, dim_size)[0];
}
torch::Tensor scatter_mean(torch::Tensor src, torch::Tensor index, int64_t dim,
                           std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size) {
  return ScatterSumMean<true>::apply(src, index, dim, optional_out, dim_size)[0];
}
std::tuple<torch::Tensor, torch::Tensor> scatter_min(torch::Tensor src, torch::Tensor index, int64_t dim,
                                                     std::optional<torch::Tensor> optional_out,
                                                     std::optional<int64_t> dim_size) {
  auto result = ScatterMinMax<false>::apply(src, index, dim, optional_out, dim_size);
  return std::make_tuple(result[0], result[1]);
}
std::tuple<torch::Tensor, torch::Tensor> scatter_max(torch::Tensor src, torch::Tensor index, int64_t dim,
                                                     std::optional<torch::Tensor> optional_out,
                                                     std::optional<int64_t> dim_size) {
  auto result = ScatterMinMax<true>::apply(src, index, dim, optional_out, dim_size);
  return std::make_tuple(result[0], result[1]);
}

}  // namespace
}  // namespace tsb_ops

TORCH_LIBRARY_FRAGMENT(torch_scatter, m) {
  m.def("scatter_sum", &tsb_ops::scatter_sum);
  m.def("scatter_mul", &tsb_ops::scatter_mul);
  m.def("scatter_mean", &tsb_ops::scatter_mean);
  m.def("scatter_min", &tsb_ops::scatter_min);
  m.def("scatter_max", &tsb_ops::scatter_max);
  // not part of upstream's operator set: the index read-back its composites do with Tensor.gather
  m.def("gather_rows", &tsb_ops::gather_rows);
  // the data-touching halves (see ops_common.h)
  m.def("_scatter_fw(Tensor src, Tensor index, int dim, Tensor? out, int? dim_size, str reduce) -> (Tensor, Tensor, Tensor)");
  m.def("_scatter_bw(Tensor grad_out, Tensor index, int dim, int[] src_shape, Tensor? count) -> Tensor");
  m.def("scatter_sum_slice", &tsb_ops::scatter_sum_slice);
  m.def("scatter_group", &tsb_ops::scatter_group);
  m.def("segment_sum_perm", &tsb_ops::segment_sum_perm);
  m.def("segment_sum_perm_routed", &tsb_ops::segment_sum_perm_routed);
  m.def("sum_slabs", &tsb_ops::sum_slabs);
}

TORCH_LIBRARY_IMPL(torch_scatter, CUDA, m) {
  m.impl("_scatter_fw", &tsb_ops::scatter_op);
  m.impl("_scatter_bw", &tsb_ops::scatter_bw_impl);
}

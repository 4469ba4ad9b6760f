// Fused forms of upstream's softmax composites (torch_scatter/composite/softmax.py:9-51,
// logsumexp.py:8-56) for an index that is 1-D and ascending: one online log-sum-exp reduction per group
// (TSB_LSE through the row-pointer reduction) and one gather pass with the exp / subtract fused in - two
// passes over the source where the composed form makes six.  Not part of upstream's operator set; the
// Python composites call these when `index_is_sorted` says the index qualifies, and compose the general
// operators otherwise.
#include "ops_common.h"

namespace tsb_ops {
namespace {

using torch::autograd::AutogradContext;
using torch::autograd::Variable;
using torch::autograd::variable_list;

// 1-D index -> a view with `dim` leading singleton dims expanded to src's leading sizes ([.., E])
torch::Tensor index_view(const torch::Tensor &index, const torch::Tensor &like, int64_t dim) {
  std::vector<int64_t> shape(dim + 1, 1), full(dim + 1);
  shape[dim] = index.size(0);
  for (int64_t i = 0; i < dim; i++) full[i] = like.size(i);
  full[dim] = index.size(0);
  return index.view(shape).expand(full);
}

struct Flat { int64_t B, E, K; };
Flat flat_dims(const torch::Tensor &x, int64_t dim) {
  Flat f{1, x.size(dim), 1};
  for (int64_t i = 0; i < dim; i++) f.B *= x.size(i);
  for (int64_t i = dim + 1; i < x.dim(); i++) f.K *= x.size(i);
  return f;
}

// fp32 table [.., N, ..] of log-sum-exp per group along dim (-inf for groups nobody names)
torch::Tensor segment_lse_impl(torch::Tensor src_, torch::Tensor index, int64_t dim, int64_t N) {
  c10::cuda::CUDAGuard guard(src_.device());
  auto src = src_.contiguous();
  auto sizes = src.sizes().vec();
  sizes[dim] = N;
  auto table = torch::empty(sizes, src.options().dtype(torch::kFloat32));
  if (table.numel() == 0) return table;
  if (src.numel() == 0) return table.fill_(-std::numeric_limits<float>::infinity());
  const Flat f = flat_dims(src, dim);
  auto idx = index.contiguous();
  const size_t ws_bytes = tsb_segment_coo_workspace_bytes(f.B, f.E, f.K, N, dtype_enum(src), TSB_LSE);
  auto workspace = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kUInt8));
  check_status(tsb_segment_coo(src.data_ptr(), idx.data_ptr<int64_t>(), table.data_ptr(), nullptr, nullptr, f.B, f.E, f.K,
                               N, 0, dtype_enum(src), TSB_LSE, 0, workspace.data_ptr(), ws_bytes, current_stream()),
               "tsb_segment_coo");
  return table;
}

// out = op(x, table[.., index, ..]) [* scale[.., index, ..]] along dim, tables fp32;
// op 1: exp(x - row), 2: x - row, 3: (x - row)^2
torch::Tensor gather_apply_impl(torch::Tensor x_, torch::Tensor table_, torch::Tensor index, int64_t dim, int64_t op,
                                std::optional<torch::Tensor> scale_) {
  c10::cuda::CUDAGuard guard(x_.device());
  auto x = x_.contiguous();
  auto table = table_.contiguous();
  torch::Tensor scale;
  if (scale_.has_value()) scale = scale_.value().contiguous();
  auto out = torch::empty_like(x);
  if (x.numel() == 0) return out;
  const Flat f = flat_dims(x, dim);
  auto idx = index.contiguous();
  check_status(tsb_gather_coo_apply2(x.data_ptr(), table.data_ptr<float>(), scale.defined() ? scale.data_ptr<float>() : nullptr,
                                     idx.data_ptr<int64_t>(), out.data_ptr(), f.B, f.E, f.K, table.size(dim), 0,
                                     dtype_enum(x), (int)op, current_stream()),
               "tsb_gather_coo_apply2");
  return out;
}

// the two data-touching routines above as operators (see ops_common.h)
torch::Tensor segment_lse(const torch::Tensor &src, const torch::Tensor &index, int64_t dim, int64_t N) {
  static auto op = internal_op<torch::Tensor(torch::Tensor, torch::Tensor, int64_t, int64_t)>("torch_scatter::_segment_lse");
  return op.call(src, index, dim, N);
}
torch::Tensor gather_apply(const torch::Tensor &x, const torch::Tensor &table, const torch::Tensor &index, int64_t dim,
                           int64_t op_code, const std::optional<torch::Tensor> &scale = std::nullopt) {
  static auto op = internal_op<torch::Tensor(torch::Tensor, torch::Tensor, torch::Tensor, int64_t, int64_t,
                                             std::optional<torch::Tensor>)>("torch_scatter::_gather_apply");
  return op.call(x, table, index, dim, op_code, scale);
}

bool index_is_sorted(torch::Tensor index) {
  TSB_CHECK_CUDA(index);
  check_index_dtype(index, "index");
  TSB_CHECK_INPUT(index.dim() == 1);
  c10::cuda::CUDAGuard guard(index.device());
  auto idx = index.contiguous();
  auto flag = torch::empty({1}, index.options().dtype(torch::kInt32));
  check_status(tsb_index_unsorted(idx.data_ptr<int64_t>(), idx.numel(), flag.data_ptr<int32_t>(), current_stream()),
               "tsb_index_unsorted");
  return flag.item<int32_t>() == 0;  // one host sync, like upstream's dim_size inference
}

// The kernels take the entry count from src and read that many index entries: a shorter index (say, the wrong
// `dim`) would be read out of bounds, a longer one would silently drop entries.  Upstream raises in its
// broadcast/expand for the same mistake (torch_scatter/utils.py:4-13).
int64_t checked_dim(const torch::Tensor &src, const torch::Tensor &index, int64_t dim) {
  dim = dim < 0 ? src.dim() + dim : dim;
  TSB_CHECK_INPUT(dim >= 0 && dim < src.dim());
  TSB_CHECK_INPUT(index.dim() == 1 && index.size(0) == src.size(dim));
  return dim;
}

int64_t groups_of(const torch::Tensor &index, std::optional<int64_t> dim_size) {
  if (dim_size.has_value()) return dim_size.value();
  return index.numel() == 0 ? 0 : index[-1].item<int64_t>() + 1;  // ascending: the last entry is the largest
}

// y = softmax / log_softmax per group.  backward: softmax gx = y * (g - sum_group(g * y));
// log_softmax gx = g - exp(y) * sum_group(g).
class SoftmaxSorted : public torch::autograd::Function<SoftmaxSorted> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim,
                               std::optional<int64_t> dim_size, bool log) {
    dim = checked_dim(src, index, dim);
    const int64_t N = groups_of(index, dim_size);
    auto lse = segment_lse(src, index, dim, N);
    auto out = gather_apply(src, lse, index, dim, log ? 2 : 1);
    ctx->saved_data["dim"] = dim;
    ctx->saved_data["N"] = N;
    ctx->saved_data["log"] = log;
    ctx->save_for_backward({index, out});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto index = saved[0], y = saved[1];
    const int64_t dim = ctx->saved_data["dim"].toInt(), N = ctx->saved_data["N"].toInt();
    const bool log = ctx->saved_data["log"].toBool();
    auto g = grad_outs[0].contiguous();
    auto iv = index_view(index, g, dim);
    torch::Tensor grad_in;
    if (log) {
      auto total = std::get<0>(segment_coo_fw(g, iv, std::nullopt, N, "sum"));
      grad_in = g - y.exp() * gather_coo_fw(total, iv, std::nullopt, std::nullopt);
    } else {
      auto gy = g * y;
      auto total = std::get<0>(segment_coo_fw(gy, iv, std::nullopt, N, "sum"));
      grad_in = gy - y * gather_coo_fw(total, iv, std::nullopt, std::nullopt);
    }
    return {grad_in, Variable(), Variable(), Variable(), Variable()};
  }
};

// lse per group, 0 for groups nobody names (upstream: nan_to_num_(neginf=0), logsumexp.py:52).
// backward: gx = g[group] * exp(x - lse[group]).
class LogSumExpSorted : public torch::autograd::Function<LogSumExpSorted> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim,
                               std::optional<int64_t> dim_size) {
    dim = checked_dim(src, index, dim);
    const int64_t N = groups_of(index, dim_size);
    auto lse = segment_lse(src, index, dim, N);
    ctx->saved_data["dim"] = dim;
    ctx->save_for_backward({src, index, lse});
    return {lse.nan_to_num(/*nan=*/std::nullopt, /*posinf=*/std::nullopt, /*neginf=*/0.0).to(src.scalar_type())};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto src = saved[0], index = saved[1], lse = saved[2];
    const int64_t dim = ctx->saved_data["dim"].toInt();
    auto iv = index_view(index, src, dim);
    auto weights = gather_apply(src, lse, index, dim, 1);  // softmax weights
    auto grad_in = weights * gather_coo_fw(grad_outs[0].contiguous(), iv, std::nullopt, std::nullopt);
    return {grad_in, Variable(), Variable(), Variable()};
  }
};

// Grouped standard deviation of fp32 data over an ascending 1-D index in three passes (upstream composes seven,
// torch_scatter/composite/std.py:8-39): group means (and counts), the squared deviations through the gather with
// (x - mean)^2 fused in, their group sums.  out = sqrt(S / (c + 1e-6)) with c = max(count - 1, 1) when unbiased.
// backward: gx = g[group] * (x - mean[group]) / ((c + 1e-6) * out)[group]  (the mean's own derivative sums to zero).
class StdSorted : public torch::autograd::Function<StdSorted> {
public:
  static variable_list forward(AutogradContext *ctx, Variable src, Variable index, int64_t dim,
                               std::optional<int64_t> dim_size, bool unbiased) {
    dim = checked_dim(src, index, dim);
    const int64_t N = groups_of(index, dim_size);
    auto iv = index_view(index, src, dim);
    auto mean_count = segment_coo_fw(src, iv, std::nullopt, N, "mean");
    auto mean = std::get<0>(mean_count);
    auto count = std::get<1>(mean_count).value();  // clamped to >= 1, shaped like the index view with N along dim
    auto squares = gather_apply(src, mean, index, dim, 3);
    auto total = std::get<0>(segment_coo_fw(squares, iv, std::nullopt, N, "sum"));
    while (count.dim() < total.dim()) count = count.unsqueeze(-1);
    if (unbiased) count = count.sub(1).clamp_min(1);
    auto denom = count + 1e-6;
    auto out = total.div(denom).sqrt();
    ctx->saved_data["dim"] = dim;
    ctx->save_for_backward({src, index, mean, denom, out});
    return {out};
  }
  static variable_list backward(AutogradContext *ctx, variable_list grad_outs) {
    auto saved = ctx->get_saved_variables();
    auto src = saved[0], index = saved[1], mean = saved[2], denom = saved[3], out = saved[4];
    const int64_t dim = ctx->saved_data["dim"].toInt();
    auto scale = grad_outs[0].div(denom * out).expand_as(out).contiguous();
    auto grad_in = gather_apply(src, mean, index, dim, 2, scale);
    return {grad_in, Variable(), Variable(), Variable(), Variable()};
  }
};

torch::Tensor std_sorted(torch::Tensor src, torch::Tensor index, int64_t dim, std::optional<int64_t> dim_size, bool unbiased) {
  return StdSorted::apply(src, index, dim, dim_size, unbiased)[0];
}

torch::Tensor softmax_sorted(torch::Tensor src, torch::Tensor index, int64_t dim, std::optional<int64_t> dim_size,
                             bool log) {
  return SoftmaxSorted::apply(src, index, dim, dim_size, log)[0];
}
torch::Tensor logsumexp_sorted(torch::Tensor src, torch::Tensor index, int64_t dim, std::optional<int64_t> dim_size) {
  return LogSumExpSorted::apply(src, index, dim, dim_size)[0];
}

}  // namespace
}  // namespace tsb_ops

TORCH_LIBRARY_FRAGMENT(torch_scatter, m) {
  m.def("index_is_sorted(Tensor index) -> bool");   // reads the data: a CUDA kernel of its own, with a fake twin
  m.def("softmax_sorted", &tsb_ops::softmax_sorted);
  m.def("logsumexp_sorted", &tsb_ops::logsumexp_sorted);
  m.def("std_sorted", &tsb_ops::std_sorted);
  m.def("_segment_lse(Tensor src, Tensor index, int dim, int groups) -> Tensor");
  m.def("_gather_apply(Tensor x, Tensor table, Tensor index, int dim, int op, Tensor? scale) -> Tensor");
}

TORCH_LIBRARY_IMPL(torch_scatter, CUDA, m) {
  m.impl("index_is_sorted", &tsb_ops::index_is_sorted);
  m.impl("_segment_lse", &tsb_ops::segment_lse_impl);
  m.impl("_gather_apply", &tsb_ops::gather_apply_impl);
}

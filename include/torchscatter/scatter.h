/*
 * C++ API of the B200 (sm_100a) build of the torch_scatter operator set.
 *
 * The same fifteen free functions, with the same signatures, that the upstream project installs in
 * <torchscatter/scatter.h> (csrc/scatter.h:13-80 there), so that C++ and TorchScript deployments written
 * against it link against this build unchanged:
 *
 *     find_package(TorchScatter REQUIRED)
 *     target_link_libraries(app TorchScatter::TorchScatter)
 *
 * Every function forwards to the operator of the same name registered in the `torch_scatter` namespace
 * (autograd included); tensors must live on a CUDA device, there is no CPU path.  Loading the library also
 * registers the operators for TorchScript modules that call torch.ops.torch_scatter.*.
 */
#pragma once

#include <torch/torch.h>

#include <cstdint>
#include <optional>
#include <tuple>

#if defined(_WIN32)
#error "this build targets Linux + sm_100a only"
#endif
#define TORCHSCATTER_API __attribute__((visibility("default")))

namespace scatter {
/* CUDA toolkit version the kernels were compiled with (e.g. 12090), as upstream's scatter::cuda_version(). */
TORCHSCATTER_API int64_t cuda_version() noexcept;
}  // namespace scatter

/* scatter: out[.., index[..], ..] (+)= src along `dim`; optional_out is accumulated into when given. */
TORCHSCATTER_API torch::Tensor scatter_sum(torch::Tensor src, torch::Tensor index, int64_t dim,
                                           std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size);
TORCHSCATTER_API torch::Tensor scatter_mul(torch::Tensor src, torch::Tensor index, int64_t dim,
                                           std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size);
TORCHSCATTER_API torch::Tensor scatter_mean(torch::Tensor src, torch::Tensor index, int64_t dim,
                                            std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size);
/* (values, arg indices); arg == src.size(dim) where no element won */
TORCHSCATTER_API std::tuple<torch::Tensor, torch::Tensor> scatter_min(torch::Tensor src, torch::Tensor index, int64_t dim,
                                                                      std::optional<torch::Tensor> optional_out,
                                                                      std::optional<int64_t> dim_size);
TORCHSCATTER_API std::tuple<torch::Tensor, torch::Tensor> scatter_max(torch::Tensor src, torch::Tensor index, int64_t dim,
                                                                      std::optional<torch::Tensor> optional_out,
                                                                      std::optional<int64_t> dim_size);

/* segment_coo: the same reductions keyed by a SORTED index along its last dimension. */
TORCHSCATTER_API torch::Tensor segment_sum_coo(torch::Tensor src, torch::Tensor index,
                                               std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size);
TORCHSCATTER_API torch::Tensor segment_mean_coo(torch::Tensor src, torch::Tensor index,
                                                std::optional<torch::Tensor> optional_out, std::optional<int64_t> dim_size);
TORCHSCATTER_API std::tuple<torch::Tensor, torch::Tensor> segment_min_coo(torch::Tensor src, torch::Tensor index,
                                                                          std::optional<torch::Tensor> optional_out,
                                                                          std::optional<int64_t> dim_size);
TORCHSCATTER_API std::tuple<torch::Tensor, torch::Tensor> segment_max_coo(torch::Tensor src, torch::Tensor index,
                                                                          std::optional<torch::Tensor> optional_out,
                                                                          std::optional<int64_t> dim_size);
TORCHSCATTER_API torch::Tensor gather_coo(torch::Tensor src, torch::Tensor index, std::optional<torch::Tensor> optional_out);

/* segment_csr: the same reductions over the row ranges of a row-pointer tensor. */
TORCHSCATTER_API torch::Tensor segment_sum_csr(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out);
TORCHSCATTER_API torch::Tensor segment_mean_csr(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out);
TORCHSCATTER_API std::tuple<torch::Tensor, torch::Tensor> segment_min_csr(torch::Tensor src, torch::Tensor indptr,
                                                                          std::optional<torch::Tensor> optional_out);
TORCHSCATTER_API std::tuple<torch::Tensor, torch::Tensor> segment_max_csr(torch::Tensor src, torch::Tensor indptr,
                                                                          std::optional<torch::Tensor> optional_out);
TORCHSCATTER_API torch::Tensor gather_csr(torch::Tensor src, torch::Tensor indptr, std::optional<torch::Tensor> optional_out);

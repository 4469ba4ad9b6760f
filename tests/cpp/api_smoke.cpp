// Links against the C++ API (include/torchscatter/scatter.h) the way a deployment would and runs one operator of
// every family on cuda:0, checking the known answers of upstream's README example and segment tests.
#include <torchscatter/scatter.h>

#include <cstdio>

static int fail(const char *what) {
  std::printf("FAIL %s\n", what);
  return 1;
}

int main() {
  if (!torch::cuda::is_available()) return fail("no CUDA device");
  if (scatter::cuda_version() < 12000) return fail("cuda_version");
  auto dev = torch::Device(torch::kCUDA, 0);
  auto f32 = torch::TensorOptions().dtype(torch::kFloat32).device(dev);
  auto i64 = torch::TensorOptions().dtype(torch::kInt64).device(dev);
  // upstream's README example: scatter_max over dim -1
  auto src = torch::tensor({2.f, 0.f, 1.f, 4.f, 3.f, 0.f, 2.f, 1.f, 3.f, 4.f}, f32).view({2, 5});
  auto index = torch::tensor({4, 5, 4, 2, 3, 0, 0, 2, 2, 1}, i64).view({2, 5});
  auto [out, argmax] = scatter_max(src, index, -1, std::nullopt, std::nullopt);
  auto want = torch::tensor({0.f, 0.f, 4.f, 3.f, 2.f, 0.f, 2.f, 4.f, 3.f, 0.f, 0.f, 0.f}, f32).view({2, 6});
  auto want_arg = torch::tensor({5, 5, 3, 4, 0, 1, 1, 4, 3, 5, 5, 5}, i64).view({2, 6});
  if (!torch::equal(out, want) || !torch::equal(argmax, want_arg)) return fail("scatter_max");
  // segment_csr / segment_coo / gathers on one small row structure, with autograd through the C++ API
  auto x = torch::arange(12, f32).view({6, 2}).requires_grad_(true);
  auto indptr = torch::tensor({0, 2, 5, 5, 6}, i64);
  auto idx = torch::tensor({0, 0, 1, 1, 1, 3}, i64);
  auto sums = segment_sum_csr(x, indptr, std::nullopt);
  auto want_sums = torch::tensor({2.f, 4.f, 18.f, 21.f, 0.f, 0.f, 10.f, 11.f}, f32).view({4, 2});
  if (!torch::equal(sums, want_sums)) return fail("segment_sum_csr");
  if (!torch::equal(segment_sum_coo(x, idx, std::nullopt, 4), want_sums)) return fail("segment_sum_coo");
  auto mean = segment_mean_csr(x, indptr, std::nullopt);
  mean.sum().backward();
  auto want_grad = torch::tensor({.5f, .5f, .5f, .5f, 1.f / 3, 1.f / 3, 1.f / 3, 1.f / 3, 1.f / 3, 1.f / 3, 1.f, 1.f}, f32).view({6, 2});
  if (!torch::allclose(x.grad(), want_grad)) return fail("segment_mean_csr backward");
  auto table = torch::arange(8, f32).view({4, 2});
  if (!torch::equal(gather_csr(table, indptr, std::nullopt), gather_coo(table, idx, std::nullopt))) return fail("gather");
  if (!torch::equal(scatter_sum(x.detach(), idx, 0, std::nullopt, 4), want_sums)) return fail("scatter_sum");
  std::printf("cpp api ok\n");
  return 0;
}

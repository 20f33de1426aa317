// Host-only check of the registry / run layer: argument errors come back with the reference's codes before any
// CUDA call, find_best falls back from the activation-specific key to the act = None entry, and an empty registry
// yields -100; the convolution's operator API rejects bad tensors with the reference's Status values.  Prints "ok" or the first failing line; exit code 0 / 1.
#include <cstdio>

#include "ge2_conv2d_api.hpp"
#include "ge2_dispatch.hpp"

using namespace ai;
namespace shim = ai::cuda::shim;

#define CHECK(cond) do { if (!(cond)) { std::printf("FAILED line %d: %s\n", __LINE__, #cond); return 1; } } while (0)

int main() {
  float dummy = 0.f;
  Tensor A = shim::make_tensor2d(&dummy, 4, 8), B = shim::make_tensor2d(&dummy, 8, 3), Y = shim::make_tensor2d(&dummy, 4, 3);
  GemmAttrs at{};
  CHECK(ops::gemm_run(A, B, nullptr, Y, at, nullptr) == -100);          // nothing registered yet
  register_b200_gemm_kernels();
  register_b200_gemm_kernels();                                          // idempotent
  Tensor none;                                                           // null data
  CHECK(ops::gemm_run(none, B, nullptr, Y, at, nullptr) == -1);
  at.trans_b = true;
  CHECK(ops::gemm_run(A, B, nullptr, Y, at, nullptr) == -11);
  at.trans_b = false;
  Tensor Bh = B; Bh.desc.dtype = shim::DType::BF16;
  CHECK(ops::gemm_run(A, Bh, nullptr, Y, at, nullptr) == -2);
  Tensor Ac = A; Ac.device = shim::Device::CPU;
  CHECK(ops::gemm_run(Ac, B, nullptr, Y, at, nullptr) == -4);
  Tensor B2 = shim::make_tensor2d(&dummy, 9, 3);
  CHECK(ops::gemm_run(A, B2, nullptr, Y, at, nullptr) == -6);
  Tensor Y2 = shim::make_tensor2d(&dummy, 4, 5);
  CHECK(ops::gemm_run(A, B, nullptr, Y2, at, nullptr) == -7);
  Tensor bias2d = shim::make_tensor2d(&dummy, 1, 3);
  CHECK(ops::gemm_run(A, B, &bias2d, Y, at, nullptr) == -9);
  Tensor bias; bias.data = &dummy; bias.desc.shape = {7}; bias.desc.stride = {1};
  CHECK(ops::gemm_run(A, B, &bias, Y, at, nullptr) == -10);
  at.save_z = true;
  CHECK(ops::gemm_run_ex(A, B, nullptr, Y, at, nullptr, nullptr) == -13);
  at.save_z = false;
  // fallback: a GELU query finds the act = None entry
  at.act = shim::ActKind::GELU;
  OpQuery q{OpKind::GEMM, A, B, nullptr, Y, at};
  CHECK(OpRegistry::inst().find_best(q) == ge2b::gemm_forward_kernel_fn());
  BwdOpQuery bq{OpKind::GEMM_BWD, A, B, nullptr, Y, Y, at};
  CHECK(BwdOpRegistry::inst().find_best(bq) == ge2b::gemm_backward_kernel_fn());
  // the operator API's own validation order (no CUDA call is reached)
  at.act = shim::ActKind::None;
  CHECK(shim::GemmCudaLaunch(A, B2, nullptr, Y, at, nullptr) == shim::Status::ShapeMismatch);
  Tensor Ys = Y; Ys.desc.stride = {2, 1};
  CHECK(shim::GemmCudaLaunch(A, B, nullptr, Ys, at, nullptr) == shim::Status::StrideMismatch);
  at.save_z = true;
  CHECK(shim::GemmCudaLaunch(A, B, nullptr, Y, at, nullptr, nullptr) == shim::Status::MissingOutput);
  at.save_z = false;
  shim::GemmWorkspace ws; ws.lt_workspace = reinterpret_cast<void*>(0x1004);
  CHECK(shim::GemmCudaLaunch(A, B, nullptr, Y, at, nullptr, nullptr, &ws) == shim::Status::Invalid);
  Tensor gC = Y;
  CHECK(shim::GemmCudaBackward(A, B, nullptr, Y, Y, nullptr, nullptr, &gC, nullptr, at, nullptr) == shim::Status::MissingInput);
  // the convolution's operator API: validation order of conv2d/launcher.cu (no CUDA call is reached)
  {
    auto t4 = [&](std::int64_t a, std::int64_t b, std::int64_t c, std::int64_t d) {
      Tensor t; t.data = &dummy; t.desc.shape = {a, b, c, d}; t.desc.stride = {b * c * d, c * d, d, 1}; return t;
    };
    Tensor X = t4(2, 3, 8, 8), W = t4(4, 3, 3, 3), Yc = t4(2, 4, 6, 6);
    Conv2DAttrs ca{};
    Tensor Xi = X; Xi.desc.dtype = shim::DType::I32;
    CHECK(Conv2DCudaLaunch(Xi, W, nullptr, Yc, ca, nullptr) == shim::Status::Invalid);
    Tensor X3 = X; X3.desc.shape = {2, 3, 64};
    CHECK(Conv2DCudaLaunch(X3, W, nullptr, Yc, ca, nullptr) == shim::Status::Invalid);
    ca.groups = 2;
    CHECK(Conv2DCudaLaunch(X, W, nullptr, Yc, ca, nullptr) == shim::Status::Unimplemented);
    ca.groups = 1;
    Tensor W2 = t4(4, 5, 3, 3);
    CHECK(Conv2DCudaLaunch(X, W2, nullptr, Yc, ca, nullptr) == shim::Status::ShapeMismatch);
    Tensor Ybad = t4(2, 4, 8, 8);                       // no padding: the output is 6 x 6
    CHECK(Conv2DCudaLaunch(X, W, nullptr, Ybad, ca, nullptr) == shim::Status::ShapeMismatch);
    Tensor Wbig = t4(4, 3, 9, 9), Y1 = t4(2, 4, 1, 1);   // kernel larger than the image: computed size 0 x 0
    CHECK(Conv2DCudaLaunch(X, Wbig, nullptr, Y1, ca, nullptr) == shim::Status::ShapeMismatch);
    Tensor Y0 = t4(2, 4, 0, 0);
    CHECK(Conv2DCudaLaunch(X, Wbig, nullptr, Y0, ca, nullptr) == shim::Status::Invalid);
    Tensor dWbad = t4(4, 3, 5, 5);
    CHECK(Conv2DCudaBackwardLaunch(X, W, Yc, Yc, &dWbad, nullptr, nullptr, ca, nullptr) == shim::Status::ShapeMismatch);
    Tensor dXbad = t4(2, 3, 8, 9);
    CHECK(Conv2DCudaBackwardLaunch(X, W, Yc, Yc, nullptr, nullptr, &dXbad, ca, nullptr) == shim::Status::ShapeMismatch);
  }
  std::printf("ok\n");
  return 0;
}

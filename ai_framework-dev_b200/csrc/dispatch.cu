// Registry and run functions declared in include/ge2_dispatch.hpp.
#include "../../include/ge2_dispatch.hpp"

namespace ai {

OpRegistry& OpRegistry::inst() { static OpRegistry r; return r; }
void OpRegistry::reg(const OpKey& key, KernelFn fn) { std::lock_guard<std::mutex> g(mu_); table_[key] = fn; }

KernelFn OpRegistry::find_best(const OpQuery& q) const {
  OpKey k{};
  k.kind = q.kind;
  k.dev = q.A.device;
  k.dtype = q.A.desc.dtype;
  k.layout = q.Y.desc.layout;
  k.act = q.attrs.act;
  k.with_bias = q.Bias && q.Bias->data;
  std::lock_guard<std::mutex> g(mu_);
  if (auto it = table_.find(k); it != table_.end()) return it->second;
  k.act = ActKind::None;
  if (auto it = table_.find(k); it != table_.end()) return it->second;
  k.layout = Layout::RowMajor;
  if (auto it = table_.find(k); it != table_.end()) return it->second;
  return nullptr;
}

BwdOpRegistry& BwdOpRegistry::inst() { static BwdOpRegistry r; return r; }
void BwdOpRegistry::reg(const BwdOpKey& key, GemmBwdFn fn) { std::lock_guard<std::mutex> g(mu_); table_[key] = fn; }

GemmBwdFn BwdOpRegistry::find_best(const BwdOpQuery& q) const {
  BwdOpKey k{};
  k.kind = q.kind;
  k.dev = q.A.device;
  k.dtype = q.A.desc.dtype;
  k.layout = q.Z.desc.layout;
  k.act = q.attrs.act;
  k.with_bias = q.attrs.with_bias;
  std::lock_guard<std::mutex> g(mu_);
  if (auto it = table_.find(k); it != table_.end()) return it->second;
  k.act = ActKind::None;
  if (auto it = table_.find(k); it != table_.end()) return it->second;
  k.layout = Layout::RowMajor;
  if (auto it = table_.find(k); it != table_.end()) return it->second;
  return nullptr;
}

void register_b200_gemm_kernels() {
  static std::once_flag once;
  std::call_once(once, [] {
    for (DType dt : {DType::F32, DType::F16, DType::BF16})
      for (bool bias : {false, true}) {
        OpKey k{};
        k.kind = OpKind::GEMM; k.dtype = dt; k.with_bias = bias;
        OpRegistry::inst().reg(k, ge2b::gemm_forward_kernel_fn());
        BwdOpKey b{};
        b.kind = OpKind::GEMM_BWD; b.dtype = dt; b.with_bias = bias;
        BwdOpRegistry::inst().reg(b, ge2b::gemm_backward_kernel_fn());
      }
  });
}

namespace ops {
namespace {
int status_to_code(Status st) {
  switch (st) {
    case Status::Ok:                    return 0;
    case Status::DeviceMismatch:        return -2;
    case Status::ShapeMismatch:         return -5;
    case Status::StrideMismatch:        return -7;
    case Status::TransposeNotSupported: return -11;
    case Status::MissingInput:          return -12;
    case Status::MissingOutput:         return -13;
    default:                            return -7;
  }
}
bool float_dtype(DType d) { return d == DType::F32 || d == DType::F16 || d == DType::BF16; }
}  // namespace

int gemm_run_ex(const Tensor& A, const Tensor& B, const Tensor* Bias, Tensor& Y, const GemmAttrs& attrs,
                StreamHandle stream, Tensor* Z_saved) {
  if (!A.data || !B.data || !Y.data) return -1;
  if (attrs.trans_a || attrs.trans_b) return -11;
  if (!float_dtype(A.desc.dtype) || B.desc.dtype != A.desc.dtype || Y.desc.dtype != A.desc.dtype) return -2;
  if (A.desc.layout != Layout::RowMajor || B.desc.layout != Layout::RowMajor || Y.desc.layout != Layout::RowMajor) return -3;
  if (A.device != Device::CUDA || B.device != Device::CUDA || Y.device != Device::CUDA) return -4;
  if (A.desc.shape.size() != 2 || B.desc.shape.size() != 2 || Y.desc.shape.size() != 2) return -5;
  const std::int64_t M = A.desc.shape[0], K = A.desc.shape[1], Kb = B.desc.shape[0], N = B.desc.shape[1];
  if (K != Kb) return -6;
  if (Y.desc.shape[0] != M || Y.desc.shape[1] != N) return -7;
  const Tensor* bias = nullptr;
  if (Bias && Bias->data) {
    if (Bias->desc.dtype != DType::F32) return -8;
    if (Bias->desc.shape.size() != 1) return -9;
    const auto bl = Bias->desc.shape[0];
    if (!(bl == 1 || bl == M || bl == N)) return -10;
    bias = Bias;
  }
  if (attrs.save_z) {
    if (!Z_saved || !Z_saved->data) return -13;
    if (!(Z_saved->desc.dtype == A.desc.dtype || Z_saved->desc.dtype == DType::F32)) return -2;
    if (Z_saved->desc.layout != Layout::RowMajor) return -3;
    if (Z_saved->device != Device::CUDA) return -4;
    if (Z_saved->desc.shape.size() != 2 || Z_saved->desc.shape[0] != M || Z_saved->desc.shape[1] != N) return -5;
  }
  OpQuery q{OpKind::GEMM, A, B, bias, Y, attrs};
  KernelFn fn = OpRegistry::inst().find_best(q);
  if (!fn) return -100;
  return status_to_code(fn(A, B, bias, Y, attrs, stream, attrs.save_z ? Z_saved : nullptr));
}

int gemm_run(const Tensor& A, const Tensor& B, const Tensor* Bias, Tensor& Y, const GemmAttrs& attrs,
             StreamHandle stream) {
  return gemm_run_ex(A, B, Bias, Y, attrs, stream, nullptr);
}

int gemm_bwd_run(const Tensor& A, const Tensor& B, const Tensor* C, const Tensor& gY, const Tensor& Z, Tensor* gA,
                 Tensor* gB, Tensor* gC, Tensor* gBias, const GemmAttrs& attrs, StreamHandle stream) {
  BwdOpQuery q{OpKind::GEMM_BWD, A, B, C, gY, Z, attrs};
  GemmBwdFn fn = BwdOpRegistry::inst().find_best(q);
  if (!fn) return -100;
  return fn(A, B, C, gY, Z, gA, gB, gC, gBias, attrs, stream) == Status::Ok ? 0 : -7;
}

}  // namespace ops
}  // namespace ai

// C entry used by tests and by hosts that cannot call C++ directly.
extern "C" void ge2b_register_gemm_kernels(void) { ai::register_b200_gemm_kernels(); }

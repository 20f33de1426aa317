// Kernel registry and int-returning run functions of the reference's dispatch layer, over this library's kernels.
//
// Same names and call shapes as graph_executor_v2/include/ai/dispatch.hpp:9-125, src/dispatch/registry.cpp:10-93 and
// src/ops/gemm.cpp:9-82 (which the reference itself does not compile): OpKey / BwdOpKey, OpRegistry / BwdOpRegistry
// with reg() and find_best() (exact key, then the key with act = None, then that key with row-major layout), and
// ai::ops::gemm_run, gemm_run_ex, gemm_bwd_run returning 0 or the reference's negative codes
// (-1 null data, -2 dtype, -3 layout, -4 device, -5..-7 shapes, -8..-10 bias, -11 transpose, -13 missing Z,
// -100 no kernel registered).  ai::register_b200_gemm_kernels() fills both registries with this library's entries
// for F32, F16 and BF16 row-major tensors; it replaces the reference's never-defined ai_backend_cuda_register_all.
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <tuple>

#include "ge2_op_api.hpp"

namespace ai {

using cuda::shim::ActKind;
using cuda::shim::Device;
using cuda::shim::DType;
using cuda::shim::GemmAttrs;
using cuda::shim::Layout;
using cuda::shim::Status;
using cuda::shim::StreamHandle;
using cuda::shim::Tensor;

enum class OpKind : std::uint8_t { GEMM = 0, GEMM_BWD = 1 };

using KernelFn = ge2b::KernelFn;
using GemmBwdFn = ge2b::GemmBwdFn;

struct OpKey {
  OpKind kind{OpKind::GEMM};
  Device dev{Device::CUDA};
  DType dtype{DType::F32};
  Layout layout{Layout::RowMajor};
  bool trans_a{false}, trans_b{false};
  ActKind act{ActKind::None};
  bool with_bias{false};
  bool save_z{false};
  bool operator<(const OpKey& o) const {
    return std::tie(kind, dev, dtype, layout, trans_a, trans_b, act, with_bias, save_z) <
           std::tie(o.kind, o.dev, o.dtype, o.layout, o.trans_a, o.trans_b, o.act, o.with_bias, o.save_z);
  }
};

struct OpQuery {
  OpKind kind;
  const Tensor& A;
  const Tensor& B;
  const Tensor* Bias;
  Tensor& Y;
  GemmAttrs attrs;
};

class OpRegistry {
 public:
  static OpRegistry& inst();
  void reg(const OpKey& key, KernelFn fn);
  KernelFn find_best(const OpQuery& q) const;
 private:
  mutable std::mutex mu_;
  std::map<OpKey, KernelFn> table_;
};

struct BwdOpKey {
  OpKind kind{OpKind::GEMM_BWD};
  Device dev{Device::CUDA};
  DType dtype{DType::F32};
  Layout layout{Layout::RowMajor};
  bool trans_a{false}, trans_b{false};
  ActKind act{ActKind::None};
  bool with_bias{false};
  bool operator<(const BwdOpKey& o) const {
    return std::tie(kind, dev, dtype, layout, trans_a, trans_b, act, with_bias) <
           std::tie(o.kind, o.dev, o.dtype, o.layout, o.trans_a, o.trans_b, o.act, o.with_bias);
  }
};

struct BwdOpQuery {
  OpKind kind;
  const Tensor& A;
  const Tensor& B;
  const Tensor* C;
  const Tensor& gY;
  const Tensor& Z;
  GemmAttrs attrs;
};

class BwdOpRegistry {
 public:
  static BwdOpRegistry& inst();
  void reg(const BwdOpKey& key, GemmBwdFn fn);
  GemmBwdFn find_best(const BwdOpQuery& q) const;
 private:
  mutable std::mutex mu_;
  std::map<BwdOpKey, GemmBwdFn> table_;
};

// Registers this library's forward and backward entries (act = None keys, which find_best falls back to for every
// activation; with and without bias; F32 / F16 / BF16).  Idempotent.
void register_b200_gemm_kernels();

namespace ops {
int gemm_run_ex(const Tensor& A, const Tensor& B, const Tensor* Bias, Tensor& Y, const GemmAttrs& attrs,
                StreamHandle stream, Tensor* Z_saved);
int gemm_run(const Tensor& A, const Tensor& B, const Tensor* Bias, Tensor& Y, const GemmAttrs& attrs,
             StreamHandle stream);
int gemm_bwd_run(const Tensor& A, const Tensor& B, const Tensor* C, const Tensor& gY, const Tensor& Z, Tensor* gA,
                 Tensor* gB, Tensor* gC, Tensor* gBias, const GemmAttrs& attrs, StreamHandle stream);
}  // namespace ops

}  // namespace ai

// Instantiates the tensor-core GEMM for 16-bit (bf16 / f16) operands, A stored with its reduction index contiguous and
// B stored with its reduction index contiguous.
#include "gemm_tc_kernel.cuh"

namespace ge2b {
namespace tc {
template cudaError_t launch_bn<2, false, false>(const GemmProblem&, TcParams&, TileChoice, cudaStream_t);
// the dense layer's backward pair: dX = gZ.W^T (both operands reduction-contiguous) and dW = X^T.gZ (both M/N-contiguous)
template cudaError_t launch_dual_cfg<2, false, false, true, true>(const GemmProblem&, TcParams&, const GemmProblem&, TcParams&,
                                                                   cudaStream_t);
}  // namespace tc
}  // namespace ge2b

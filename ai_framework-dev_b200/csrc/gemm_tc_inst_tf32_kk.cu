// Instantiates the tensor-core GEMM for 32-bit (TF32) operands, A stored with its reduction index contiguous and
// B stored with its reduction index contiguous.
#include "gemm_tc_kernel.cuh"

namespace ge2b {
namespace tc {
template cudaError_t prepare_bn<4, false, false>(const GemmProblem&, TcParams&, TileChoice, cudaStream_t, PreparedLaunch&);
// the dense layer's backward pair: dX = gZ.W^T (both operands reduction-contiguous) and dW = X^T.gZ (both M/N-contiguous)
template cudaError_t prepare_dual_cfg<4, false, false, true, true>(const GemmProblem&, TcParams&, const GemmProblem&, TcParams&,
                                                                    PreparedLaunch&);
}  // namespace tc
}  // namespace ge2b

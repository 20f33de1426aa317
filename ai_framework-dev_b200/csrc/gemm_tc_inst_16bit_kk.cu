// Instantiates the tensor-core GEMM for 16-bit (bf16 / f16) operands, A stored with its reduction index contiguous and
// B stored with its reduction index contiguous.
#include "gemm_tc_kernel.cuh"

namespace ge2b {
namespace tc {
template cudaError_t prepare_bn<2, false, false>(const GemmProblem&, TcParams&, TileChoice, cudaStream_t, PreparedLaunch&);
// the dense layer's backward pair: dX = gZ.W^T (both operands reduction-contiguous) and dW = X^T.gZ (both M/N-contiguous)
template cudaError_t prepare_dual_cfg<2, false, false, true, true>(const GemmProblem&, TcParams&, const GemmProblem&, TcParams&,
                                                                    PreparedLaunch&);
}  // namespace tc
}  // namespace ge2b

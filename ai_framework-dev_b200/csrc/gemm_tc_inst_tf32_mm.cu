// Instantiates the tensor-core GEMM for 32-bit (TF32) operands, A stored with its M index contiguous and
// B stored with its N index contiguous.
#include "gemm_tc_kernel.cuh"

namespace ge2b {
namespace tc {
template cudaError_t prepare_bn<4, true, true>(const GemmProblem&, TcParams&, TileChoice, cudaStream_t, PreparedLaunch&);
}  // namespace tc
}  // namespace ge2b

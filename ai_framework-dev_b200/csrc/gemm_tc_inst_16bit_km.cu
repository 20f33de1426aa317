// Instantiates the tensor-core GEMM for 16-bit (bf16 / f16) operands, A stored with its reduction index contiguous and
// B stored with its N index contiguous.
#include "gemm_tc_kernel.cuh"

namespace ge2b {
namespace tc {
template cudaError_t prepare_bn<2, false, true>(const GemmProblem&, TcParams&, TileChoice, cudaStream_t, PreparedLaunch&);
}  // namespace tc
}  // namespace ge2b

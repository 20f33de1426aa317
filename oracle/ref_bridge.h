// Force-included (after ref_prefix.h) when compiling reference ops that are still written against the old flat
// `ai::` namespace (conv2d): brings the shim types into it, as the reference's own build would have to.
#include "backends/cuda/ops/_common/shim/ai_shim.hpp"
namespace ai { using namespace ::ai::cuda::shim; }

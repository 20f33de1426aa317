// Force-included when compiling reference sources on Linux: makes std::expf visible
// (the reference was developed against a toolchain whose <cmath> declares it).
#include <cmath>
#include <math.h>
namespace std { using ::expf; }

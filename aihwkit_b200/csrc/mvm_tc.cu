// Tensor-core (tcgen05 / TMEM / TMA) IO-managed MVM. Placeholder selection logic until the
// kernel lands: every problem goes to the CUDA-core path.
#include "tile.h"

namespace ab200 {
bool tcMvmSupported(const MvmProblem &) { return false; }
void launchMvmTc(const MvmProblem &, cudaStream_t) { AB200_FATAL("tensor-core MVM not built"); }
} // namespace ab200

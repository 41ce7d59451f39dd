// step_kernel<1, false, slim>: one coordinate per lane, without free rigid bodies, held to 128 registers.
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepNarrowSlim, 1, false, true, false)
}  // namespace nkb

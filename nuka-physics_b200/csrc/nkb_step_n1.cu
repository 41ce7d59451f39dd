// step_kernel<1, false>: one coordinate per lane, without free rigid bodies.
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepNarrow, 1, false, false, false)
}  // namespace nkb

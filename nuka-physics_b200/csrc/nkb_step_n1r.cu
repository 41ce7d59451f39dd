// step_kernel<1, true>: one coordinate per lane, with free rigid bodies.
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepNarrowRigid, 1, true, false, false)
}  // namespace nkb

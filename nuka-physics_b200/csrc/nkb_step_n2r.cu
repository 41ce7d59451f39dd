// step_kernel<2, true>: two coordinates per lane, with free rigid bodies.
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepWideRigid, 2, true, false, false)
}  // namespace nkb

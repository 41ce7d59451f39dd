// step_kernel<1, true, false, control>: one coordinate per lane, with free rigid bodies, with the computed-torque and
// operational-space controllers between two dynamics passes (control modes 3 and 4).
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepNarrowRigidControl, 1, true, false, true)
}  // namespace nkb

// step_kernel<2, true, false, control>: two coordinates per lane, with free rigid bodies, with the computed-torque and
// operational-space controllers between two dynamics passes (control modes 3 and 4).
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepWideRigidControl, 2, true, false, true)
}  // namespace nkb

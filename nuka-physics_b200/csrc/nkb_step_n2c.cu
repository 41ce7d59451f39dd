// step_kernel<2, false, false, control>: two coordinates per lane, without free rigid bodies, with the computed-torque and
// operational-space controllers between two dynamics passes (control modes 3 and 4).
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepWideControl, 2, false, false, true)
}  // namespace nkb

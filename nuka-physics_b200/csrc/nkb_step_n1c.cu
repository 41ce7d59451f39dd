// step_kernel<1, false, false, control>: one coordinate per lane, without free rigid bodies, with the computed-torque and
// operational-space controllers between two dynamics passes (control modes 3 and 4).
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepNarrowControl, 1, false, false, true)
}  // namespace nkb

// step_kernel<2, false>: two coordinates per lane, without free rigid bodies.
#include "nkb_step.cuh"

namespace nkb {
NKB_STEP_VARIANT(kStepWide, 2, false, false, false)
}  // namespace nkb

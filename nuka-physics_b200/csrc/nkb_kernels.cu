// Host side of the kernels: picks the step-kernel variant of a world, and the small reset / observation kernels.
#include <cuda_runtime.h>
#include <algorithm>
#include <cstdio>
#include "nkb_launch.h"

namespace nkb {

// Per-env reset from the creation snapshot (reference ops/readout.cu:771-776 RestoreState semantics).
__global__ void reset_kernel(ResetParams r) {
    const uint32_t slot = blockIdx.x;
    const uint32_t env = r.env_ids != nullptr ? r.env_ids[slot] : slot;
    if (env >= r.env_count) return;
    if (r.env_ids == nullptr && r.env_mask != nullptr && r.env_mask[env] == 0u) return;
    for (uint32_t f = 0u; f < r.field_count; ++f) {
        const ResetField fd = r.fields[f];
        uint32_t* dst = reinterpret_cast<uint32_t*>(fd.dst) + (size_t)env * fd.words;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(fd.src);
        for (uint32_t k = threadIdx.x; k < fd.words; k += blockDim.x) dst[k] = fd.per_env_src ? src[(size_t)env * fd.words + k] : (fd.src != nullptr ? src[k] : fd.fill);
    }
}

extern const StepVariant kStepNarrow, kStepNarrowSlim, kStepNarrowRigid, kStepWide, kStepWideRigid;
extern const StepVariant kStepNarrowControl, kStepNarrowRigidControl, kStepWideControl, kStepWideRigidControl;

bool step_kernel_has_slim(uint32_t ndof, uint32_t n_free, bool control) { return ndof <= 32u && n_free == 0u && !control; }

// up to 32 or up to 64 coordinates per articulation; with or without free rigid bodies; the slim (128-register) build
// exists for the first kind only
static const StepVariant& step_variant(uint32_t ndof, uint32_t n_free, bool slim, bool control) {
    // control modes 3 and 4 run the builds that hold the controllers
    if (control) return ndof > 32u ? (n_free != 0u ? kStepWideRigidControl : kStepWideControl) : (n_free != 0u ? kStepNarrowRigidControl : kStepNarrowControl);
    if (ndof > 32u) return n_free != 0u ? kStepWideRigid : kStepWide;
    if (n_free != 0u) return kStepNarrowRigid;
    return slim ? kStepNarrowSlim : kStepNarrow;
}

int step_kernel_registers(uint32_t ndof, uint32_t n_free, bool slim, bool control) { return step_variant(ndof, n_free, slim, control).registers(); }

int step_kernel_resident_blocks(uint32_t ndof, uint32_t n_free, bool slim, bool control, uint32_t warps_per_block, size_t shared_bytes) {
    return step_variant(ndof, n_free, slim, control).resident_blocks(warps_per_block, shared_bytes);
}

cudaError_t launch_step(const StepParams& p, uint32_t warps_per_block, bool slim, cudaStream_t stream) {
    const bool control = p.t.cfg.control_mode == 3u || p.t.cfg.control_mode == 4u;
    return step_variant(p.t.ndof, p.t.n_free, slim && !control, control).launch(p, warps_per_block, stream);
}

// One observation record per env, composed from the state arrays in one pass (the reference's gym layer builds the same
// record with a chain of torch ops on the field views, python/nuka/tasks/go2_obs.py:282-305).  One thread per output
// value; the record is short, so consecutive threads write consecutive floats.
__global__ void pack_observations_kernel(const StateView s, uint32_t L, const ObservationParams o, float* out) {
    const uint32_t nj = L - 1u, width = 12u + 3u * nj + (o.reward != nullptr ? 1u : 0u);
    const size_t total = (size_t)s.env_count * width;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (size_t)gridDim.x * blockDim.x) {
        const uint32_t env = (uint32_t)(at / width), k = (uint32_t)(at % width);
        const float* twist = s.link_vel + (size_t)env * L * 6u;          // root link: angular (3) then linear (3), base frame
        float v;
        if (k < 3u) v = twist[3u + k] * o.lin_vel_scale;
        else if (k < 6u) v = twist[k - 3u] * o.ang_vel_scale;
        else if (k < 9u) {
            // world (0, 0, -1) in the base frame: R(q)^T g = (w^2 - |u|^2) g - 2 w (u x g) + 2 u (u . g), python/nuka/tasks/go2_obs.py:96-112
            const float* pose = s.link_pose + (size_t)env * L * 7u;
            const float w = pose[3], x = pose[4], y = pose[5], z = pose[6];
            const float a = w * w - (x * x + y * y + z * z);
            const float cross[3] = {-y, x, 0.f};                         // u x g with g = (0, 0, -1)
            const float u[3] = {x, y, z};
            const float g[3] = {0.f, 0.f, -1.f};
            const uint32_t c = k - 6u;
            v = a * g[c] - 2.0f * w * cross[c] + 2.0f * u[c] * (-z);
        } else if (k < 12u) {
            const uint32_t c = k - 9u;
            v = o.command[(size_t)env * o.command_stride + c] * o.command_scale[c];
        } else if (k < 12u + 2u * nj) {
            const bool vel = k >= 12u + nj;
            const uint32_t i = k - 12u - (vel ? nj : 0u);
            const uint32_t slot = o.joint_order != nullptr ? o.joint_order[i] : i;
            const size_t src = (size_t)env * L + 1u + slot;
            v = vel ? s.qdot[src] * o.dof_vel_scale
                    : (s.q[src] - (o.default_position != nullptr ? o.default_position[i] : 0.f)) * o.dof_pos_scale;
        } else if (k < 12u + 3u * nj) {
            v = o.last_action != nullptr ? o.last_action[(size_t)env * nj + (k - 12u - 2u * nj)] : 0.f;
        } else {
            out[(size_t)env * o.row_stride + k] = o.reward[env];          // the reward rides along unclipped
            continue;
        }
        out[(size_t)env * o.row_stride + k] = fminf(fmaxf(v, -o.clip), o.clip);
    }
}

cudaError_t launch_pack_observations(const StateView& s, uint32_t L, const ObservationParams& o, float* out, cudaStream_t stream) {
    if (s.env_count == 0u || L < 2u) return cudaSuccess;
    const size_t total = (size_t)s.env_count * (12u + 3u * (L - 1u) + (o.reward != nullptr ? 1u : 0u));
    const uint32_t blocks = (uint32_t)std::min<size_t>((total + 255u) / 256u, 148u * 8u);
    pack_observations_kernel<<<blocks, 256, 0, stream>>>(s, L, o, out);
    return cudaGetLastError();
}

cudaError_t launch_reset(const ResetParams& r, uint32_t count, cudaStream_t stream) {
    if (count == 0u) return cudaSuccess;
    reset_kernel<<<count, 128, 0, stream>>>(r);
    return cudaGetLastError();
}

}  // namespace nkb

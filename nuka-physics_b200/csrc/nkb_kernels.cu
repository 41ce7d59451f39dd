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
    for (uint32_t f = 0u; f < r.field_count; ++f) {
        const ResetField fd = r.fields[f];
        uint32_t* dst = reinterpret_cast<uint32_t*>(fd.dst) + (size_t)env * fd.words;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(fd.src);
        for (uint32_t k = threadIdx.x; k < fd.words; k += blockDim.x) dst[k] = fd.per_env_src ? src[(size_t)env * fd.words + k] : (fd.src != nullptr ? src[k] : fd.fill);
    }
}

extern const StepVariant kStepNarrow, kStepNarrowRigid, kStepWide, kStepWideRigid;

// up to 32 or up to 64 coordinates per articulation; with or without free rigid bodies
static const StepVariant& step_variant(uint32_t ndof, uint32_t n_free) {
    if (ndof > 32u) return n_free != 0u ? kStepWideRigid : kStepWide;
    return n_free != 0u ? kStepNarrowRigid : kStepNarrow;
}

int step_kernel_registers(uint32_t ndof, uint32_t n_free) { return step_variant(ndof, n_free).registers(); }

int step_kernel_resident_blocks(uint32_t ndof, uint32_t n_free, uint32_t warps_per_block, size_t shared_bytes) {
    return step_variant(ndof, n_free).resident_blocks(warps_per_block, shared_bytes);
}

cudaError_t launch_step(const StepParams& p, uint32_t warps_per_block, cudaStream_t stream) {
    return step_variant(p.t.ndof, p.t.n_free).launch(p, warps_per_block, stream);
}

// One record per env for the RL caller (python/nuka/tasks/go2_obs.py:47-48 composes the same quantities):
// joint positions and velocities (L - 1 each), base pose (7), root twist (6), drive targets of all joints but the
// last (L - 2), and the base height as reward: 3 (L - 1) + 13 floats.
__global__ void pack_observations_kernel(const StateView s, uint32_t L, float* out) {
    const uint32_t width = 3u * (L - 1u) + 13u, nq = L - 1u;
    const size_t total = (size_t)s.env_count * width;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (size_t)gridDim.x * blockDim.x) {
        const uint32_t env = (uint32_t)(at / width), k = (uint32_t)(at % width);
        float v;
        if (k < nq) v = s.q[(size_t)env * L + 1u + k];
        else if (k < 2u * nq) v = s.qdot[(size_t)env * L + 1u + (k - nq)];
        else if (k < 2u * nq + 7u) v = s.base_pose[(size_t)env * 7u + (k - 2u * nq)];
        else if (k < 2u * nq + 13u) v = s.link_vel[(size_t)env * L * 6u + (k - 2u * nq - 7u)];
        else if (k < width - 1u) v = s.drive_target[(size_t)env * L + 1u + (k - 2u * nq - 13u)];
        else v = s.base_pose[(size_t)env * 7u + 2u];
        out[at] = v;
    }
}

cudaError_t launch_pack_observations(const StateView& s, uint32_t L, float* out, cudaStream_t stream) {
    if (s.env_count == 0u || L < 2u) return cudaSuccess;
    const size_t total = (size_t)s.env_count * (3u * (L - 1u) + 13u);
    const uint32_t blocks = (uint32_t)std::min<size_t>((total + 255u) / 256u, 148u * 8u);
    pack_observations_kernel<<<blocks, 256, 0, stream>>>(s, L, out);
    return cudaGetLastError();
}

cudaError_t launch_reset(const ResetParams& r, uint32_t count, cudaStream_t stream) {
    if (count == 0u) return cudaSuccess;
    reset_kernel<<<count, 128, 0, stream>>>(r);
    return cudaGetLastError();
}

}  // namespace nkb

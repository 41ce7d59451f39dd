// Launch entry points of the CUDA side, callable from plain C++ translation units.
#pragma once
#include <cuda_runtime.h>
#include "nkb_types.h"

namespace nkb {

constexpr uint32_t kWarpsPerBlockMax = 8u;

struct ResetField {
    void* dst;            // E x words
    const void* src;      // template words, per-env snapshot, or null for a constant fill
    uint32_t words;
    uint32_t per_env_src; // 1: src is E x words
    uint32_t fill;
};
constexpr uint32_t kMaxResetFields = 36u;
struct ResetParams {
    uint32_t env_count;
    const uint32_t* env_ids;   // device list of envs to reset, or null for all
    const uint32_t* env_mask;  // device array of env_count words; with env_ids null, only envs with a non-zero word reset
    uint32_t field_count;
    ResetField fields[kMaxResetFields];
};

// Blocks of `warps_per_block` warps with `shared_bytes` of dynamic shared memory that one SM keeps resident (registers,
// shared memory and block slots considered); 0 when the shape cannot launch.  The device must be current.
// The step kernel has one variant per (coordinates per lane, free rigid bodies present) pair, chosen from `ndof`
// (up to 32 / up to 64 coordinates) and `n_free` (free dynamic bodies per env).
int step_kernel_resident_blocks(uint32_t ndof, uint32_t n_free, bool slim, bool control, uint32_t warps_per_block, size_t shared_bytes);
// Whether a slim (128-register) build of the world's kernel variant exists.
bool step_kernel_has_slim(uint32_t ndof, uint32_t n_free, bool control);
// Registers per thread of the step kernel variant that serves the world.
int step_kernel_registers(uint32_t ndof, uint32_t n_free, bool slim, bool control);
// Host-side handle of one compiled step-kernel variant.
struct StepParams;
struct StepVariant {
    int (*resident_blocks)(uint32_t warps_per_block, size_t shared_bytes);
    int (*registers)();
    cudaError_t (*launch)(const StepParams& p, uint32_t warps_per_block, cudaStream_t stream);
};
// Enqueues `p.steps` fused steps (or one parity-tap stage, see StepMode) for every env.
cudaError_t launch_step(const StepParams& p, uint32_t warps_per_block, bool slim, cudaStream_t stream);
// Restores `count` envs (all when r.env_ids is null) from their snapshots.
cudaError_t launch_reset(const ResetParams& r, uint32_t count, cudaStream_t stream);
// Observation record of the reference's gym layer (python/nuka/tasks/go2_obs.py:11-20) for a floating-base robot with
// nj = L - 1 actuated joints: base linear velocity x lin_scale (3), base angular velocity x ang_scale (3), gravity
// direction in the base frame (3), command x command_scale (3), (q - default) x pos_scale in caller joint order (nj),
// qdot x vel_scale in caller joint order (nj), last action (nj); every value clipped to [-clip, clip].  An optional
// reward column follows.  All pointers are device memory.
struct ObservationParams {
    const float* command;           // E x 3, or 3 floats shared by every env when command_stride == 0
    uint32_t command_stride;        // floats between the commands of consecutive envs (0 or >= 3)
    const float* last_action;       // E x nj, or null for zeros
    const float* default_position;  // nj, caller joint order; null for zeros
    const uint32_t* joint_order;    // nj: library joint slot (0-based, slot j is link j + 1) read for caller joint i; null = identity
    const float* reward;            // E, copied into column 9 + 3 + 3 nj when non-null
    float lin_vel_scale, ang_vel_scale, dof_pos_scale, dof_vel_scale;
    float command_scale[3];
    float clip;
    uint32_t row_stride;            // floats between consecutive records in the output (>= the record width)
};
cudaError_t launch_pack_observations(const StateView& s, uint32_t L, const ObservationParams& o, float* out, cudaStream_t stream);
// Partial reset without a device allocation: the ids travel through a fixed device array of kStaticResetMaxIds words
// that every world on `device` shares.  `device` must be current; r.env_ids is ignored.
constexpr uint32_t kStaticResetMaxIds = 4096u;
// On success *device_ids is the array's address on `device` (the ids stay there until the next call).
cudaError_t launch_reset_static_ids(const ResetParams& r, const uint32_t* host_ids, uint32_t count, int device, cudaStream_t stream,
                                    const uint32_t** device_ids);

}  // namespace nkb

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
constexpr uint32_t kMaxResetFields = 24u;
struct ResetParams {
    uint32_t env_count;
    const uint32_t* env_ids;   // device list of envs to reset, or null for all
    uint32_t field_count;
    ResetField fields[kMaxResetFields];
};

// Blocks of `warps_per_block` warps with `shared_bytes` of dynamic shared memory that one SM keeps resident (registers,
// shared memory and block slots considered); 0 when the shape cannot launch.  The device must be current.
// The step kernel has one variant per (coordinates per lane, free rigid bodies present) pair, chosen from `ndof`
// (up to 32 / up to 64 coordinates) and `n_free` (free dynamic bodies per env).
int step_kernel_resident_blocks(uint32_t ndof, uint32_t n_free, uint32_t warps_per_block, size_t shared_bytes);
// Registers per thread of the step kernel variant that serves the world.
int step_kernel_registers(uint32_t ndof, uint32_t n_free);
// Host-side handle of one compiled step-kernel variant.
struct StepParams;
struct StepVariant {
    int (*resident_blocks)(uint32_t warps_per_block, size_t shared_bytes);
    int (*registers)();
    cudaError_t (*launch)(const StepParams& p, uint32_t warps_per_block, cudaStream_t stream);
};
// Enqueues `p.steps` fused steps (or one parity-tap stage, see StepMode) for every env.
cudaError_t launch_step(const StepParams& p, uint32_t warps_per_block, cudaStream_t stream);
// Restores `count` envs (all when r.env_ids is null) from their snapshots.
cudaError_t launch_reset(const ResetParams& r, uint32_t count, cudaStream_t stream);
// Packs the per-env observation record (3 (L - 1) + 13 floats) of every env into `out` (device memory).
cudaError_t launch_pack_observations(const StateView& s, uint32_t L, float* out, cudaStream_t stream);
// Partial reset without a device allocation: the ids travel through a fixed device array of kStaticResetMaxIds words
// that every world on `device` shares.  `device` must be current; r.env_ids is ignored.
constexpr uint32_t kStaticResetMaxIds = 4096u;
cudaError_t launch_reset_static_ids(const ResetParams& r, const uint32_t* host_ids, uint32_t count, int device, cudaStream_t stream);

}  // namespace nkb

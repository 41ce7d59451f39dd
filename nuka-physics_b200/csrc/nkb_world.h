// Host runtime of the batched articulated step: cooked-template parsing, device storage, the field table,
// step/reset/refresh launches.  Mirrors the role of the reference's nk::World (src/nk/pipeline/world.cpp)
// for this path; there is no op list to dispatch because the step is one fused kernel.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>
#include "nkb_launch.h"
#include "nkb_types.h"

namespace nkb {

struct Error : std::runtime_error {
    int code;   // nuka_result_t value
    Error(int c, const std::string& what) : std::runtime_error(what), code(c) {}
};

// One env's cooked template on the host.
struct HostTemplate {
    uint32_t L = 0, B = 0, ndof = 0, max_depth = 0, floating_root = 0;
    Config cfg{};
    std::vector<uint32_t> parent, jtype, depth, child_begin, children, link_dof, link_body, geom_kind, limit_flags, dof_link, anc_mask;
    std::vector<float> axis, offset, local_quat, inertia10, damping, armature, frictionloss, stiffness, spring_ref;
    std::vector<float> limit_lower, limit_upper, geom_pos, geom_quat, q0, base_pose0, kp0, kd0, force_limit0;
    std::vector<uint32_t> shape_kind, contype, conaffinity, group, body_to_link;
    std::vector<int32_t> body_id;
    std::vector<float> shape_params, mu, inv_mass, inv_inertia, inertial_pos, inertial_quat, body_pose0;
    std::vector<unsigned long long> excluded;
    std::vector<uint32_t> adm_pairs;
    std::vector<uint32_t> adm_mask;      // B x ceil(B / 32) words, bit b of row a for admissible a < b
    uint32_t max_points = 0;            // template's contact-point capacity, 0 = default
    std::vector<std::string> link_names;   // optional: one name per link (the joint whose child the link is, else the body's)
    std::vector<uint32_t> body_geom_kind;          // per collidable row (several rows may mirror one link)
    std::vector<float> body_geom_pos, body_geom_quat;
    std::vector<uint32_t> free_slot;
    uint32_t n_free = 0;
    uint32_t joint_rows = 0;     // limit + friction + drive rows one env can emit
    static HostTemplate Parse(const void* blob, size_t bytes);
};

struct FieldInfo {
    void* ptr = nullptr;
    size_t per_env = 0;          // elements per env
    uint32_t dtype = 0;          // 0 f32, 1 u32
    bool writable = false;
};

class World {
public:
    World(int device, cudaStream_t stream, const HostTemplate& tpl, uint32_t env_count);
    ~World();
    World(const World&) = delete;
    World& operator=(const World&) = delete;

    void Step(uint32_t n);
    void RunStage(uint32_t mode);
    void Refresh(const uint32_t* ids = nullptr, uint32_t count = 0u, const uint32_t* mask = nullptr);
    void Reset(const uint32_t* env_ids, uint32_t count);   // null ids: all envs
    void ResetStaticIds(const uint32_t* env_ids, uint32_t count);   // partial reset that allocates nothing
    void ResetMasked(const uint32_t* device_mask);                  // partial reset chosen on the device, no host sync
    void SetContactReadout(bool on);
    void SetBroadphase(uint32_t mode);                              // 0: by table size, 1: admissible-pair table, 2: per-env tree
    void Synchronize();
    uint32_t ObservationWidth() const { return tpl_.L >= 2u ? 3u * (tpl_.L - 1u) + 12u : 0u; }      // without the reward column
    void PackObservations(const ObservationParams& o, float* device_out);
    bool Field(uint32_t id, FieldInfo* out);
    void SetVelocityIterations(uint32_t n) { params_.t.cfg.vel_iters = n; graph_valid_ = false; }
    uint32_t VelocityIterations() const { return params_.t.cfg.vel_iters; }
    void SetGravityZ(float g) { params_.t.cfg.gravity[2] = g; graph_valid_ = false; }
    void SetGraphMode(bool on);
    // Persistent state: every per-env array a step carries over (coordinates, velocities, poses, carried constraint
    // velocities, the contact cache, status words, drive inputs), in a fixed order.  A checkpoint is these bytes
    // plus the host settings below (reference src/c_abi/checkpoint.cpp:442-520 captures the same split).
    size_t PersistentBytes() const;
    uint64_t PersistentLayoutHash() const;
    void DownloadPersistent(uint8_t* out);          // synchronises the stream
    void UploadPersistent(const uint8_t* in);       // then refreshes the derived poses
    uint64_t step_count() const { return step_count_; }
    void set_step_count(uint64_t n) { step_count_ = n; }
    const float* gravity() const { return params_.t.cfg.gravity; }
    void SetGravity(const float g[3]) { for (int k = 0; k < 3; ++k) params_.t.cfg.gravity[k] = g[k]; graph_valid_ = false; }
    cudaStream_t stream() const { return stream_; }
    int device() const { return device_; }
    uint32_t env_count() const { return env_count_; }
    const HostTemplate& tpl() const { return tpl_; }
    uint32_t shared_bytes_per_env() const { return params_.sm.words * 4u; }
    uint32_t warps_per_block() const { return warps_per_block_; }
    uint64_t launches() const { return launches_; }

private:
    template <typename T> T* Alloc(size_t count, bool zero = true);
    template <typename T> const T* Upload(const std::vector<T>& v);
    void Check(cudaError_t err, const char* what);
    void BuildLayout();
    void Seed();

    int device_;
    cudaStream_t stream_;
    HostTemplate tpl_;
    uint32_t env_count_;
    StepParams params_{};
    StateView readout_{};               // contact read-out pointers while the read-out is switched off
    uint32_t warps_per_block_ = 1;
    bool slim_ = false;        // the world runs the 128-register build of its kernel variant
    std::vector<void*> allocations_;
    ResetParams reset_{};
    uint32_t* reset_ids_ = nullptr;
    uint32_t reset_ids_cap_ = 0;
    uint32_t static_ids_host_[kStaticResetMaxIds];      // sorted, de-duplicated ids of the partial reset being issued
    CacheEntry* cache_empty_ = nullptr;
    bool graph_mode_ = false, graph_valid_ = false;
    cudaGraph_t graph_ = nullptr;
    cudaGraphExec_t graph_exec_ = nullptr;
    uint64_t launches_ = 0;
    uint64_t step_count_ = 0;
    struct PersistentField { void* ptr; uint32_t words; };
    std::vector<PersistentField> persistent_;
};

}  // namespace nkb

// extern "C" boundary: handle tables, result codes, thread-local error text.  No exception crosses it
// (reference src/c_abi/error.cpp:12-60, src/c_abi/handle_table.hpp:13-60, src/c_abi/world.cpp:493-731,
// src/c_abi/buffer.cpp:31-205).
#include <atomic>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <mutex>
#include <sstream>
#include <unordered_map>

#include "../../include/nuka_b200.h"
#include "nkb_scene.h"
#include "nkb_world.h"

namespace {

thread_local std::string g_last_error;
thread_local std::string g_last_error_out;

void SetError(const std::string& text) { g_last_error = text; }

struct DeviceRecord {
    int gpu = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    uint32_t worlds = 0;
};

// Handles are ids that count up and are never handed out twice: a handle kept after its object was destroyed stays
// unknown for good, whatever is created later (reference src/c_abi/handle_table.hpp:18-26).
template <typename T>
class HandleTable {
public:
    uintptr_t Insert(std::unique_ptr<T> value) {
        std::lock_guard<std::mutex> lock(mutex_);
        const uintptr_t id = next_id_++;
        values_.emplace(id, std::move(value));
        return id;
    }
    T* Get(uintptr_t handle) {
        std::lock_guard<std::mutex> lock(mutex_);
        const auto it = values_.find(handle);
        return it == values_.end() ? nullptr : it->second.get();
    }
    std::unique_ptr<T> Remove(uintptr_t handle) {
        std::lock_guard<std::mutex> lock(mutex_);
        const auto it = values_.find(handle);
        if (it == values_.end()) return nullptr;
        std::unique_ptr<T> value = std::move(it->second);
        values_.erase(it);
        return value;
    }
private:
    std::mutex mutex_;
    uintptr_t next_id_ = 1;
    std::unordered_map<uintptr_t, std::unique_ptr<T>> values_;
};

struct WorldRecord {
    std::unique_ptr<nkb::World> world;
    uintptr_t device = 0;
    uint64_t serial = 0;        // creation order; a checkpoint remembers its owner's
};

// Host copy of a world's persistent state and settings (reference src/c_abi/checkpoint.cpp:442-520).
struct CheckpointRecord {
    uintptr_t owner = 0;
    uint64_t owner_serial = 0;
    uint64_t layout_hash = 0;
    uint64_t step_count = 0;
    uint32_t velocity_iterations = 0;
    float gravity[3] = {0.f, 0.f, 0.f};
    std::vector<uint8_t> persistent;
};

constexpr uint64_t kCheckpointMagic = 0x3143424b554eull;      // "NUKBC1"

uint64_t Fnv1a(uint64_t h, const void* data, size_t bytes) {
    const uint8_t* p = static_cast<const uint8_t*>(data);
    for (size_t k = 0; k < bytes; ++k) { h ^= p[k]; h *= 1099511628211ull; }
    return h;
}

// The tables live until the process ends and are never destroyed: an object a caller left alive must not run its
// destructor (CUDA calls) during static destruction, when the CUDA runtime may already be gone.
HandleTable<DeviceRecord>& Devices() { static auto* t = new HandleTable<DeviceRecord>; return *t; }
HandleTable<WorldRecord>& Worlds() { static auto* t = new HandleTable<WorldRecord>; return *t; }
HandleTable<CheckpointRecord>& Checkpoints() { static auto* t = new HandleTable<CheckpointRecord>; return *t; }
std::atomic<uint64_t> g_world_serial{0};

template <typename Fn>
nuka_result_t Guard(Fn&& fn) {
    try {
        return fn();
    } catch (const nkb::Error& e) {
        SetError(e.what());
        return static_cast<nuka_result_t>(e.code);
    } catch (const std::bad_alloc&) {
        SetError("host allocation failed");
        return NUKA_RESULT_OUT_OF_MEMORY;
    } catch (const std::exception& e) {
        SetError(e.what());
        return NUKA_RESULT_INTERNAL;
    } catch (...) {
        SetError("unknown failure");
        return NUKA_RESULT_INTERNAL;
    }
}

nkb::World* WorldOf(nuka_world_handle h) {
    WorldRecord* r = Worlds().Get(reinterpret_cast<uintptr_t>(h));
    return r ? r->world.get() : nullptr;
}

nuka_result_t ValidateDesc(const nuka_world_desc_t* d) {
    // reference src/c_abi/world.cpp:493-528
    if (d == nullptr) { SetError("world desc is null"); return NUKA_RESULT_INVALID_ARG; }
    if (d->env_count == 0u) { SetError("env_count must be positive"); return NUKA_RESULT_INVALID_ARG; }
    if (d->determinism > 1u) { SetError("determinism must be 0 or 1"); return NUKA_RESULT_INVALID_ARG; }
    if (d->fixed_dt < 0.f || d->fixed_dt != d->fixed_dt) { SetError("fixed_dt must be positive"); return NUKA_RESULT_INVALID_ARG; }
    if (d->control_mode > 5u) { SetError("control_mode must be 0..5"); return NUKA_RESULT_INVALID_ARG; }
    if (d->control_mode != 4u && d->osc_task_link != 0u) { SetError("osc_task_link is read in control mode 4 only"); return NUKA_RESULT_NOT_SUPPORTED; }
    const bool unsupported = d->terrain_step_height != 0.f || d->terrain_step_width != 0.f || d->terrain_platform_width != 0.f ||
        d->terrain_grid_width != 0.f || d->terrain_grid_height_max != 0.f || d->instance_count > 1u || d->contact_family != 0u ||
        d->heightfield_terrain_type != 0u || (d->heightfield_image_path != nullptr && d->heightfield_image_path[0] != '\0') ||
        d->curric_levels != 0u || d->curric_types != 0u || d->cloth_integrator != 0u || d->ogc_contact_capacity != 0u ||
        d->solver_substeps > 1u || d->contact_detection_substeps > 1u;
    if (unsupported) { SetError("the world desc selects a feature outside the articulated step path"); return NUKA_RESULT_NOT_SUPPORTED; }
    if (d->solver_vel_iters > 65535u) { SetError("solver_vel_iters exceeds 65535"); return NUKA_RESULT_INVALID_ARG; }
    if (d->solver_pos_iters > 65535u) { SetError("solver_pos_iters exceeds 65535"); return NUKA_RESULT_INVALID_ARG; }
    return NUKA_RESULT_OK;
}

nuka_result_t CreateWorld(nuka_device_handle device, const nuka_world_desc_t* desc, const void* blob, size_t bytes, nuka_world_handle* out) {
    if (out == nullptr) { SetError("out handle is null"); return NUKA_RESULT_INVALID_ARG; }
    *out = nullptr;
    DeviceRecord* dev = Devices().Get(reinterpret_cast<uintptr_t>(device));
    if (dev == nullptr) { SetError("device handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    const nuka_result_t valid = ValidateDesc(desc);
    if (valid != NUKA_RESULT_OK) return valid;
    return Guard([&]() {
        nkb::HostTemplate tpl = nkb::HostTemplate::Parse(blob, bytes);
        if (desc->fixed_dt > 0.f) tpl.cfg.dt = desc->fixed_dt;
        tpl.cfg.control_mode = desc->control_mode;
        tpl.cfg.task_link = desc->osc_task_link;
        if (desc->gravity_x != 0.f || desc->gravity_y != 0.f || desc->gravity_z != 0.f) {
            tpl.cfg.gravity[0] = desc->gravity_x; tpl.cfg.gravity[1] = desc->gravity_y; tpl.cfg.gravity[2] = desc->gravity_z;
        }
        if (desc->solver_vel_iters != 0u) tpl.cfg.vel_iters = desc->solver_vel_iters;
        if (desc->solver_pos_iters != 0u) tpl.cfg.pos_iters = desc->solver_pos_iters;
        if (desc->solver_contact_margin > 0.f) tpl.cfg.contact_margin = desc->solver_contact_margin;
        if (desc->solver_max_pairs != 0u) tpl.cfg.max_pairs = desc->solver_max_pairs;
        if (desc->solver_baumgarte_max_velocity > 0.f) tpl.cfg.baumgarte_max_velocity = desc->solver_baumgarte_max_velocity;
        if (desc->solver_overlap_recovery_velocity > 0.f) tpl.cfg.overlap_recovery_velocity = desc->solver_overlap_recovery_velocity;
        auto record = std::make_unique<WorldRecord>();
        record->world = std::make_unique<nkb::World>(dev->gpu, dev->stream, tpl, desc->env_count);
        record->device = reinterpret_cast<uintptr_t>(device);
        record->serial = ++g_world_serial;
        ++dev->worlds;
        *out = reinterpret_cast<nuka_world_handle>(Worlds().Insert(std::move(record)));
        return NUKA_RESULT_OK;
    });
}

}  // namespace

extern "C" {

nuka_version_t nuka_get_version(void) { return {0, 1, 0}; }

const char* nuka_result_message(nuka_result_t result) {
    switch (result) {
        case NUKA_RESULT_OK: return "ok";
        case NUKA_RESULT_INVALID_ARG: return "invalid argument";
        case NUKA_RESULT_NULL_HANDLE: return "null or stale handle";
        case NUKA_RESULT_CUDA_ERROR: return "CUDA error";
        case NUKA_RESULT_FILE_NOT_FOUND: return "file not found";
        case NUKA_RESULT_PARSE_ERROR: return "parse error";
        case NUKA_RESULT_OUT_OF_MEMORY: return "out of memory";
        case NUKA_RESULT_NOT_SUPPORTED: return "not supported";
        case NUKA_RESULT_INTERNAL: return "internal error";
    }
    return "unknown result";
}

const char* nuka_last_error_message(void) {
    g_last_error_out = g_last_error;
    g_last_error.clear();
    return g_last_error_out.c_str();
}

nuka_result_t nuka_device_create(const nuka_device_desc_t* desc, nuka_device_handle* out) {
    if (out == nullptr || desc == nullptr) { SetError("device desc or out handle is null"); return NUKA_RESULT_INVALID_ARG; }
    *out = nullptr;
    return Guard([&]() {
        int count = 0;
        const cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess || count == 0) {
            // no CPU fallback: without a CUDA device there is nothing to run on
            SetError(std::string("no CUDA device: ") + cudaGetErrorString(err));
            return NUKA_RESULT_CUDA_ERROR;
        }
        if (desc->gpu_index >= static_cast<uint32_t>(count)) { SetError("gpu_index out of range"); return NUKA_RESULT_INVALID_ARG; }
        auto rec = std::make_unique<DeviceRecord>();
        rec->gpu = static_cast<int>(desc->gpu_index);
        if (cudaSetDevice(rec->gpu) != cudaSuccess) { SetError("cudaSetDevice failed"); return NUKA_RESULT_CUDA_ERROR; }
        if (desc->cuda_stream != nullptr) rec->stream = static_cast<cudaStream_t>(desc->cuda_stream);
        else {
            if (cudaStreamCreateWithFlags(&rec->stream, cudaStreamNonBlocking) != cudaSuccess) { SetError("stream creation failed"); return NUKA_RESULT_CUDA_ERROR; }
            rec->owns_stream = true;
        }
        *out = reinterpret_cast<nuka_device_handle>(Devices().Insert(std::move(rec)));
        return NUKA_RESULT_OK;
    });
}

void nuka_device_destroy(nuka_device_handle device) {
    auto rec = Devices().Remove(reinterpret_cast<uintptr_t>(device));
    if (!rec) return;
    if (rec->owns_stream) { cudaSetDevice(rec->gpu); cudaStreamDestroy(rec->stream); }
}

nuka_result_t nuka_world_create_from_template(nuka_device_handle device, const nuka_world_desc_t* desc,
                                              const void* template_bytes, size_t template_size, nuka_world_handle* out) {
    if (template_bytes == nullptr || template_size == 0) { SetError("template bytes are null"); return NUKA_RESULT_INVALID_ARG; }
    return CreateWorld(device, desc, template_bytes, template_size, out);
}

nuka_result_t nuka_b200_template_check(const void* template_bytes, size_t template_size) {
    if (template_bytes == nullptr || template_size == 0) { SetError("template bytes are null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() { (void)nkb::HostTemplate::Parse(template_bytes, template_size); return NUKA_RESULT_OK; });
}

void nuka_b200_cook_options_defaults(nuka_b200_cook_options_t* options) {
    if (options == nullptr) return;
    const nkb::CookOptions d;
    options->dt = d.dt; options->velocity_iterations = d.vel_iters; options->position_iterations = d.pos_iters;
    options->default_kp = d.kp; options->default_kd = d.kd;
    options->add_default_ground = d.default_ground ? 1u : 0u; options->ground_height = d.ground_height; options->ground_mu = d.ground_mu;
    options->self_collision = d.self_collision ? 1u : 0u; options->scene_filters = d.scene_filters ? 1u : 0u;
    options->max_contacts = d.max_contacts; options->max_points = d.max_points;
}

nuka_result_t nuka_b200_scene_cook(const char* scene_json, size_t scene_size, const nuka_b200_cook_options_t* options, void* out,
                                   size_t capacity, size_t* out_size) {
    if (scene_json == nullptr || out_size == nullptr) { SetError("scene text or out_size is null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() {
        nkb::CookOptions o;
        if (options != nullptr) {
            o.dt = options->dt; o.vel_iters = options->velocity_iterations; o.pos_iters = options->position_iterations;
            o.kp = options->default_kp; o.kd = options->default_kd;
            o.default_ground = options->add_default_ground != 0u; o.ground_height = options->ground_height; o.ground_mu = options->ground_mu;
            o.self_collision = options->self_collision != 0u; o.scene_filters = options->scene_filters != 0u;
            o.max_contacts = options->max_contacts; o.max_points = options->max_points;
        }
        const std::vector<uint8_t> blob = nkb::CookSceneForWorld(std::string(scene_json, scene_size), o);
        *out_size = blob.size();
        if (out == nullptr) return NUKA_RESULT_OK;                       // size query
        if (capacity < blob.size()) { SetError("output buffer is smaller than the cooked template"); return NUKA_RESULT_INVALID_ARG; }
        std::memcpy(out, blob.data(), blob.size());
        return NUKA_RESULT_OK;
    });
}

nuka_result_t nuka_world_create_from_scene(nuka_device_handle device, const nuka_world_desc_t* desc, nuka_world_handle* out) {
    if (desc == nullptr || desc->scene_path == nullptr) { SetError("scene_path is null"); if (out) *out = nullptr; return NUKA_RESULT_INVALID_ARG; }
    const std::string path = desc->scene_path;
    const auto ends_with = [&](const char* suffix) { const size_t n = std::strlen(suffix); return path.size() > n && path.compare(path.size() - n, n, suffix) == 0; };
    if (!ends_with(".nks") && !ends_with(".nkt")) {
        SetError("scene files (.nks) and cooked templates (.nkt) are loadable; the USD / URDF / MJCF importers are outside this path");
        if (out) *out = nullptr;
        return NUKA_RESULT_NOT_SUPPORTED;
    }
    std::ifstream in(path, std::ios::binary);
    if (!in) { SetError("cannot open " + path); if (out) *out = nullptr; return NUKA_RESULT_FILE_NOT_FOUND; }
    std::stringstream ss;
    ss << in.rdbuf();
    std::string bytes = ss.str();
    // a scene document (.nks, JSON) is cooked here with the reference cooker's rules: drives from the scene's actuators,
    // the scene's own ground and filter bits, one candidate slot per admissible pair; a cooked template (.nkt) loads as is
    if (nkb::LooksLikeScene(bytes)) {
        std::vector<uint8_t> cooked;
        const nuka_result_t r = Guard([&]() {
            nkb::CookOptions options;
            if (desc->fixed_dt > 0.f) options.dt = desc->fixed_dt;
            if (desc->solver_vel_iters != 0u) options.vel_iters = desc->solver_vel_iters;
            if (desc->solver_pos_iters != 0u) options.pos_iters = desc->solver_pos_iters;
            cooked = nkb::CookSceneForWorld(bytes, options);
            return NUKA_RESULT_OK;
        });
        if (r != NUKA_RESULT_OK) { if (out) *out = nullptr; return r; }
        return CreateWorld(device, desc, cooked.data(), cooked.size(), out);
    }
    return CreateWorld(device, desc, bytes.data(), bytes.size(), out);
}

void nuka_world_destroy(nuka_world_handle world) {
    auto rec = Worlds().Remove(reinterpret_cast<uintptr_t>(world));
    if (!rec) return;
    if (DeviceRecord* dev = Devices().Get(rec->device)) { if (dev->worlds) --dev->worlds; }
    rec->world.reset();
}

#define NKB_WORLD(w)                                                          \
    nkb::World* w = WorldOf(world);                                           \
    if (w == nullptr) { SetError("world handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }

nuka_result_t nuka_world_step(nuka_world_handle world) { return nuka_world_step_n(world, 1u); }

nuka_result_t nuka_world_step_n(nuka_world_handle world, uint32_t step_count) {
    NKB_WORLD(w)
    return Guard([&]() { w->Step(step_count); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_world_set_execution_mode(nuka_world_handle world, nuka_execution_mode_t mode) {
    NKB_WORLD(w)
    if (mode != NUKA_EXECUTION_EAGER && mode != NUKA_EXECUTION_GRAPH) { SetError("unknown execution mode"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() { w->SetGraphMode(mode == NUKA_EXECUTION_GRAPH); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_world_set_gravity_z(nuka_world_handle world, float gravity_z) {
    NKB_WORLD(w)
    if (gravity_z != gravity_z) { SetError("gravity_z is NaN"); return NUKA_RESULT_INVALID_ARG; }
    w->SetGravityZ(gravity_z);
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_world_set_velocity_iterations(nuka_world_handle world, uint32_t iterations) {
    NKB_WORLD(w)
    if (iterations == 0u || iterations > 65535u) { SetError("velocity iterations must be in 1..65535"); return NUKA_RESULT_INVALID_ARG; }
    w->SetVelocityIterations(iterations);
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_world_get_velocity_iterations(nuka_world_handle world, uint32_t* out_iterations) {
    NKB_WORLD(w)
    if (out_iterations == nullptr) { SetError("out pointer is null"); return NUKA_RESULT_INVALID_ARG; }
    *out_iterations = w->VelocityIterations();
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_world_synchronize(nuka_world_handle world) {
    NKB_WORLD(w)
    return Guard([&]() { w->Synchronize(); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_world_reset(nuka_world_handle world) {
    NKB_WORLD(w)
    return Guard([&]() { w->Reset(nullptr, 0u); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_world_reset_envs(nuka_world_handle world, const uint32_t* env_ids, uint32_t count) {
    NKB_WORLD(w)
    if (count == 0u) return NUKA_RESULT_OK;
    if (env_ids == nullptr) { SetError("env_ids is null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() { w->Reset(env_ids, count); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_b200_world_reset_envs_static(nuka_world_handle world, const uint32_t* env_ids, uint32_t count) {
    NKB_WORLD(w)
    if (count == 0u) return NUKA_RESULT_OK;
    if (env_ids == nullptr) { SetError("env_ids is null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() { w->ResetStaticIds(env_ids, count); return NUKA_RESULT_OK; });
}

// ---- checkpoints (reference nuka.h:387-404, src/c_abi/checkpoint.cpp:442-635) ----

namespace {
void CaptureInto(nkb::World* w, CheckpointRecord* c) {
    c->layout_hash = w->PersistentLayoutHash();
    c->step_count = w->step_count();
    c->velocity_iterations = w->VelocityIterations();
    for (int k = 0; k < 3; ++k) c->gravity[k] = w->gravity()[k];
    c->persistent.resize(w->PersistentBytes());
    w->DownloadPersistent(c->persistent.data());
}
}  // namespace

nuka_result_t nuka_world_checkpoint_capture(nuka_world_handle world, nuka_checkpoint_handle* out) {
    if (out == nullptr) { SetError("out handle is null"); return NUKA_RESULT_INVALID_ARG; }
    *out = nullptr;
    WorldRecord* rec = Worlds().Get(reinterpret_cast<uintptr_t>(world));
    if (rec == nullptr || !rec->world) { SetError("world handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    return Guard([&]() {
        auto c = std::make_unique<CheckpointRecord>();
        c->owner = reinterpret_cast<uintptr_t>(world);
        c->owner_serial = rec->serial;
        CaptureInto(rec->world.get(), c.get());
        *out = reinterpret_cast<nuka_checkpoint_handle>(Checkpoints().Insert(std::move(c)));
        return NUKA_RESULT_OK;
    });
}

nuka_result_t nuka_world_checkpoint_restore(nuka_world_handle world, nuka_checkpoint_handle checkpoint) {
    WorldRecord* rec = Worlds().Get(reinterpret_cast<uintptr_t>(world));
    CheckpointRecord* c = Checkpoints().Get(reinterpret_cast<uintptr_t>(checkpoint));
    if (rec == nullptr || !rec->world || c == nullptr) { SetError("world or checkpoint handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    if (c->owner != reinterpret_cast<uintptr_t>(world) || c->owner_serial != rec->serial) {
        SetError("checkpoint belongs to another world");
        return NUKA_RESULT_INVALID_ARG;
    }
    nkb::World* w = rec->world.get();
    if (c->layout_hash != w->PersistentLayoutHash() || c->persistent.size() != w->PersistentBytes()) {
        SetError("checkpoint layout does not match the world");
        return NUKA_RESULT_INVALID_ARG;
    }
    return Guard([&]() {
        w->SetGravity(c->gravity);
        w->SetVelocityIterations(c->velocity_iterations);
        w->UploadPersistent(c->persistent.data());
        w->set_step_count(c->step_count);
        return NUKA_RESULT_OK;
    });
}

void nuka_checkpoint_destroy(nuka_checkpoint_handle checkpoint) {
    Checkpoints().Remove(reinterpret_cast<uintptr_t>(checkpoint));
}

nuka_result_t nuka_checkpoint_write(nuka_checkpoint_handle checkpoint, const char* path) {
    CheckpointRecord* c = Checkpoints().Get(reinterpret_cast<uintptr_t>(checkpoint));
    if (c == nullptr) { SetError("checkpoint handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    if (path == nullptr) { SetError("path is null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() {
        std::ofstream file(path, std::ios::binary | std::ios::trunc);
        const uint64_t header[4] = {kCheckpointMagic, c->layout_hash, c->step_count, c->persistent.size()};
        file.write(reinterpret_cast<const char*>(header), sizeof(header));
        file.write(reinterpret_cast<const char*>(c->persistent.data()), static_cast<std::streamsize>(c->persistent.size()));
        file.write(reinterpret_cast<const char*>(&c->velocity_iterations), sizeof(uint32_t));
        file.write(reinterpret_cast<const char*>(c->gravity), sizeof(c->gravity));
        file.flush();
        if (!file.good()) { SetError(std::string("cannot write ") + path); return NUKA_RESULT_INTERNAL; }
        return NUKA_RESULT_OK;
    });
}

nuka_result_t nuka_world_checkpoint_read(nuka_world_handle world, const char* path, nuka_checkpoint_handle* out) {
    if (out == nullptr || path == nullptr) { SetError("out handle or path is null"); return NUKA_RESULT_INVALID_ARG; }
    *out = nullptr;
    WorldRecord* rec = Worlds().Get(reinterpret_cast<uintptr_t>(world));
    if (rec == nullptr || !rec->world) { SetError("world handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    return Guard([&]() {
        nkb::World* w = rec->world.get();
        std::ifstream file(path, std::ios::binary);
        uint64_t header[4] = {};
        file.read(reinterpret_cast<char*>(header), sizeof(header));
        if (!file.good() || header[0] != kCheckpointMagic || header[1] != w->PersistentLayoutHash() || header[3] != w->PersistentBytes()) {
            SetError(std::string("not a checkpoint of this world's layout: ") + path);
            return NUKA_RESULT_INVALID_ARG;
        }
        auto c = std::make_unique<CheckpointRecord>();
        c->owner = reinterpret_cast<uintptr_t>(world);
        c->owner_serial = rec->serial;
        c->layout_hash = header[1];
        c->step_count = header[2];
        c->persistent.resize(header[3]);
        file.read(reinterpret_cast<char*>(c->persistent.data()), static_cast<std::streamsize>(header[3]));
        file.read(reinterpret_cast<char*>(&c->velocity_iterations), sizeof(uint32_t));
        file.read(reinterpret_cast<char*>(c->gravity), sizeof(c->gravity));
        if (!file.good()) { SetError(std::string("checkpoint file is short: ") + path); return NUKA_RESULT_INVALID_ARG; }
        *out = reinterpret_cast<nuka_checkpoint_handle>(Checkpoints().Insert(std::move(c)));
        return NUKA_RESULT_OK;
    });
}

nuka_result_t nuka_checkpoint_byte_size(nuka_checkpoint_handle checkpoint, uint64_t* out_bytes) {
    CheckpointRecord* c = Checkpoints().Get(reinterpret_cast<uintptr_t>(checkpoint));
    if (c == nullptr) { SetError("checkpoint handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    if (out_bytes == nullptr) { SetError("out_bytes is null"); return NUKA_RESULT_INVALID_ARG; }
    *out_bytes = c->persistent.size();
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_checkpoint_equal(nuka_checkpoint_handle a, nuka_checkpoint_handle b, uint32_t* out_equal) {
    CheckpointRecord* x = Checkpoints().Get(reinterpret_cast<uintptr_t>(a));
    CheckpointRecord* y = Checkpoints().Get(reinterpret_cast<uintptr_t>(b));
    if (x == nullptr || y == nullptr) { SetError("checkpoint handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    if (out_equal == nullptr) { SetError("out_equal is null"); return NUKA_RESULT_INVALID_ARG; }
    *out_equal = (x->layout_hash == y->layout_hash && x->step_count == y->step_count && x->persistent == y->persistent) ? 1u : 0u;
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_world_state_hash(nuka_world_handle world, uint64_t* out_hash) {
    if (out_hash == nullptr) { SetError("out_hash is null"); return NUKA_RESULT_INVALID_ARG; }
    WorldRecord* rec = Worlds().Get(reinterpret_cast<uintptr_t>(world));
    if (rec == nullptr || !rec->world) { SetError("world handle is null or stale"); return NUKA_RESULT_NULL_HANDLE; }
    return Guard([&]() {
        CheckpointRecord c;
        CaptureInto(rec->world.get(), &c);
        uint64_t h = 1469598103934665603ull;
        h = Fnv1a(h, c.persistent.data(), c.persistent.size());
        h = Fnv1a(h, &c.step_count, sizeof(c.step_count));
        h = Fnv1a(h, &c.velocity_iterations, sizeof(c.velocity_iterations));
        h = Fnv1a(h, c.gravity, sizeof(c.gravity));
        *out_hash = h;
        return NUKA_RESULT_OK;
    });
}

nuka_result_t nuka_world_forward_kinematics(nuka_world_handle world) {
    NKB_WORLD(w)
    return Guard([&]() { w->Refresh(); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_world_get_stream(nuka_world_handle world, void** out_stream) {
    NKB_WORLD(w)
    if (out_stream == nullptr) { SetError("out pointer is null"); return NUKA_RESULT_INVALID_ARG; }
    *out_stream = static_cast<void*>(w->stream());
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_world_record_event(nuka_world_handle world, void* cuda_event) {
    NKB_WORLD(w)
    if (cuda_event == nullptr) { SetError("event is null"); return NUKA_RESULT_INVALID_ARG; }
    if (cudaSetDevice(w->device()) != cudaSuccess || cudaEventRecord(static_cast<cudaEvent_t>(cuda_event), w->stream()) != cudaSuccess) {
        SetError("cudaEventRecord failed");
        return NUKA_RESULT_CUDA_ERROR;
    }
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_world_get_buffer_view(nuka_world_handle world, nuka_state_field_t field, nuka_buffer_view_t* out) {
    NKB_WORLD(w)
    if (out == nullptr) { SetError("out view is null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() {
        nkb::FieldInfo info;
        if (!w->Field(static_cast<uint32_t>(field), &info)) { SetError("field is not served by this path"); return NUKA_RESULT_NOT_SUPPORTED; }
        out->device_ptr = info.ptr;
        out->element_count = info.per_env * w->env_count();
        out->element_stride_bytes = 4u;
        out->dtype = static_cast<uint8_t>(info.dtype);
        return NUKA_RESULT_OK;
    });
}

// Argument checks in the reference's order (src/c_abi/buffer.cpp:98-110): a null buffer with a size first, then the
// handle, then the empty transfer.
static nuka_result_t Transfer(nuka_world_handle world, nuka_state_field_t field, void* bytes, size_t nbytes, size_t offset, bool upload) {
    if (bytes == nullptr && nbytes > 0u) { SetError("bytes is null"); return NUKA_RESULT_INVALID_ARG; }
    NKB_WORLD(w)
    if (nbytes == 0u) return NUKA_RESULT_OK;
    return Guard([&]() {
        nkb::FieldInfo info;
        if (!w->Field(static_cast<uint32_t>(field), &info)) { SetError("field is not served by this path"); return NUKA_RESULT_NOT_SUPPORTED; }
        if (upload && !info.writable) { SetError("field is an output of the step and cannot be uploaded"); return NUKA_RESULT_NOT_SUPPORTED; }
        const size_t total = info.per_env * w->env_count() * 4u;
        if (offset > total || nbytes > total - offset) { SetError("transfer exceeds the field"); return NUKA_RESULT_INVALID_ARG; }
        if (cudaSetDevice(w->device()) != cudaSuccess) { SetError("cudaSetDevice failed"); return NUKA_RESULT_CUDA_ERROR; }
        auto* dev = static_cast<uint8_t*>(info.ptr) + offset;
        const cudaError_t err = upload ? cudaMemcpyAsync(dev, bytes, nbytes, cudaMemcpyHostToDevice, w->stream())
                                       : cudaMemcpyAsync(bytes, dev, nbytes, cudaMemcpyDeviceToHost, w->stream());
        // pageable host memory makes the copy synchronous with respect to the host buffer; pinned buffers stay
        // asynchronous on upload, downloads always complete before returning
        if (err != cudaSuccess) { SetError(std::string("field copy: ") + cudaGetErrorString(err)); return NUKA_RESULT_CUDA_ERROR; }
        if (!upload && cudaStreamSynchronize(w->stream()) != cudaSuccess) { SetError("field download sync failed"); return NUKA_RESULT_CUDA_ERROR; }
        return NUKA_RESULT_OK;
    });
}

nuka_result_t nuka_world_upload_field(nuka_world_handle world, nuka_state_field_t field, const void* bytes, size_t nbytes, size_t byte_offset) {
    return Transfer(world, field, const_cast<void*>(bytes), nbytes, byte_offset, true);
}

nuka_result_t nuka_world_download_field(nuka_world_handle world, nuka_state_field_t field, void* bytes, size_t nbytes, size_t byte_offset) {
    return Transfer(world, field, bytes, nbytes, byte_offset, false);
}

nuka_result_t nuka_b200_world_info(nuka_world_handle world, nuka_b200_world_info_t* out) {
    NKB_WORLD(w)
    if (out == nullptr) { SetError("out pointer is null"); return NUKA_RESULT_INVALID_ARG; }
    out->env_count = w->env_count();
    out->links_per_env = w->tpl().L; out->bodies_per_env = w->tpl().B; out->dofs_per_env = w->tpl().ndof;
    out->contact_slots_per_env = w->tpl().cfg.max_contacts;
    out->shared_bytes_per_env = w->shared_bytes_per_env(); out->warps_per_block = w->warps_per_block();
    out->fixed_dt = w->tpl().cfg.dt;
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_b200_world_run_stage(nuka_world_handle world, uint32_t stage) {
    NKB_WORLD(w)
    if (stage != 1u && stage != 2u) { SetError("stage must be 1 (dynamics) or 2 (collision)"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() { w->RunStage(stage); return NUKA_RESULT_OK; });
}

void nuka_b200_observation_desc_defaults(nuka_b200_observation_desc_t* d) {
    if (d == nullptr) return;
    // python/nuka/tasks/go2_obs.py:56-66
    d->lin_vel_scale = 2.0f; d->ang_vel_scale = 0.25f; d->dof_pos_scale = 1.0f; d->dof_vel_scale = 0.05f;
    d->command_scale[0] = 2.0f; d->command_scale[1] = 2.0f; d->command_scale[2] = 0.25f;
    d->clip = 100.0f;
}

nuka_result_t nuka_b200_world_pack_observations(nuka_world_handle world, const nuka_b200_observation_desc_t* desc,
                                                float* device_out, size_t capacity_floats, uint32_t* out_width) {
    NKB_WORLD(w)
    const uint32_t width = w->ObservationWidth();
    if (out_width != nullptr) *out_width = width;
    if (device_out == nullptr) return NUKA_RESULT_OK;          // width query only
    if (width == 0u) { SetError("the world has no actuated joints to observe"); return NUKA_RESULT_NOT_SUPPORTED; }
    if (desc == nullptr || desc->command == nullptr) { SetError("observation desc or its command pointer is null"); return NUKA_RESULT_INVALID_ARG; }
    if (desc->command_stride != 0u && desc->command_stride < 3u) { SetError("command_stride must be 0 or at least 3"); return NUKA_RESULT_INVALID_ARG; }
    const uint32_t record = width + (desc->reward != nullptr ? 1u : 0u);
    const uint32_t stride = desc->row_stride != 0u ? desc->row_stride : record;
    if (stride < record) { SetError("row_stride is below the record width"); return NUKA_RESULT_INVALID_ARG; }
    const size_t need = static_cast<size_t>(stride) * (w->env_count() - 1u) + record;
    if (capacity_floats < need) { SetError("observation buffer is too small"); return NUKA_RESULT_INVALID_ARG; }
    if (!(desc->clip >= 0.f)) { SetError("clip must not be negative"); return NUKA_RESULT_INVALID_ARG; }
    nkb::ObservationParams o{};
    o.command = desc->command; o.command_stride = desc->command_stride; o.last_action = desc->last_action;
    o.default_position = desc->default_position; o.joint_order = desc->joint_order; o.reward = desc->reward;
    o.lin_vel_scale = desc->lin_vel_scale; o.ang_vel_scale = desc->ang_vel_scale; o.dof_pos_scale = desc->dof_pos_scale;
    o.dof_vel_scale = desc->dof_vel_scale;
    for (int k = 0; k < 3; ++k) o.command_scale[k] = desc->command_scale[k];
    o.clip = desc->clip; o.row_stride = stride;
    return Guard([&]() { w->PackObservations(o, device_out); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_b200_world_reset_envs_masked(nuka_world_handle world, const uint32_t* device_mask) {
    NKB_WORLD(w)
    if (device_mask == nullptr) { SetError("device_mask is null"); return NUKA_RESULT_INVALID_ARG; }
    return Guard([&]() { w->ResetMasked(device_mask); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_b200_world_set_broadphase(nuka_world_handle world, uint32_t mode) {
    NKB_WORLD(w)
    return Guard([&]() { w->SetBroadphase(mode); return NUKA_RESULT_OK; });
}

nuka_result_t nuka_b200_world_set_contact_readout(nuka_world_handle world, uint32_t enabled) {
    NKB_WORLD(w)
    return Guard([&]() { w->SetContactReadout(enabled != 0u); return NUKA_RESULT_OK; });
}

// src/c_abi/world.cpp:1170-1215: link_index runs over every env's links; a null `out` is a size query
nuka_result_t nuka_world_get_dof_name(nuka_world_handle world, uint32_t link_index, char* out, size_t cap, size_t* out_len) {
    if (out_len != nullptr) *out_len = 0u;
    NKB_WORLD(w)
    const std::vector<std::string>& names = w->tpl().link_names;
    if (names.empty()) { SetError("the world's template carries no link names"); return NUKA_RESULT_NOT_SUPPORTED; }
    const uint64_t total = static_cast<uint64_t>(names.size()) * w->env_count();
    if (link_index >= total) { SetError("link_index is out of range"); return NUKA_RESULT_INVALID_ARG; }
    const std::string& name = names[link_index % names.size()];
    if (out_len != nullptr) *out_len = name.size();
    if (out == nullptr) return NUKA_RESULT_OK;
    if (name.size() + 1u > cap) { SetError("the buffer cannot hold the name and its terminator"); return NUKA_RESULT_INVALID_ARG; }
    std::memcpy(out, name.c_str(), name.size() + 1u);
    return NUKA_RESULT_OK;
}

nuka_result_t nuka_b200_world_launch_count(nuka_world_handle world, uint64_t* out) {
    NKB_WORLD(w)
    if (out == nullptr) { SetError("out pointer is null"); return NUKA_RESULT_INVALID_ARG; }
    *out = w->launches();
    return NUKA_RESULT_OK;
}

}  // extern "C"

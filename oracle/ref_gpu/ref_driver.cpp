// Test infrastructure: drives the UNMODIFIED reference (kry4r/Nuka-Physics) through its own scene loader, cooker and
// nk::World on the GPU, and writes what it computes into a named-array container (the "NKT1" layout that
// nuka/nkt.py reads).  Built by oracle/ref_gpu/Makefile from the reference checkout where it lies; nothing of the
// reference is copied into this repository.  The product never links or runs this program: tests compare against the
// files it wrote (tests/golden/ref_*.nkt) and bench reports quote the timings it printed.
//
//   ref_driver --scene robot.nks --envs E --dt 0.005 --vel-iters 4 [--pos-iters k] [--no-contacts] [--control-mode m]
//              [--state state.nkt]            per-env q, qdot, base_pose, link_velocity, drive_target, kp, kd, force_limit (any subset)
//              [--cook-only]                  stop after cooking (runs without a GPU) and dump the cooked model tables
//              [--dump out.nkt]               model tables + single-op dynamics + trajectory samples
//              [--steps N --every k]          trajectory length and sampling stride
//              [--time warm,timed,repeats]    wall-clock timing of StepConfigured in eager and graph mode, JSON on stdout
//              [--active sigma]               with --time: every timed step first uploads fresh drive targets (cooked targets +
//                                             N(0, sigma) rad, a pool of 16 sets), the regime of an RL caller; eager mode only
//
// Reference entry points used (paths in the reference): scene::nks::Load (src/scene/format/nks.hpp),
// scene::cook::CookToModel (src/scene/cook/cook_to_model.hpp), nk::World (src/nk/pipeline/world.hpp),
// World::DispatchOp with ArticulationDynamicsParams{integrate_velocity = 0} as tests/oracle/
// featherstone_oracle_harness.cpp:160-190 does, nk::Data::Upload/DownloadField (src/nk/data/data.hpp).
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <string>
#include <vector>

#include "nk/model/generated/field_ids.hpp"
#include "nk/model/model.hpp"
#include "nk/pipeline/world.hpp"
#include "phi/backend.hpp"
#include "phi/op_schema.hpp"
#include "scene/cook/cook_to_model.hpp"
#include "scene/format/nks.hpp"

namespace nk = nuka::nk;
namespace nphi = nuka::phi;

namespace {

struct Container {      // name -> (dtype, raw bytes); dtype 0 f32, 1 u32, 2 i32, 3 u64
    std::vector<std::string> order;
    std::map<std::string, std::pair<uint32_t, std::vector<uint8_t>>> items;
    void Put(const std::string& name, uint32_t dtype, const void* data, size_t bytes) {
        if (!items.count(name)) order.push_back(name);
        auto& slot = items[name];
        slot.first = dtype;
        slot.second.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + bytes);
    }
    void F32(const std::string& n, const std::vector<float>& v) { Put(n, 0, v.data(), v.size() * 4); }
    void U32(const std::string& n, const std::vector<uint32_t>& v) { Put(n, 1, v.data(), v.size() * 4); }
    void I32(const std::string& n, const std::vector<int32_t>& v) { Put(n, 2, v.data(), v.size() * 4); }
    void U64(const std::string& n, const std::vector<uint64_t>& v) { Put(n, 3, v.data(), v.size() * 8); }
    bool Write(const std::string& path) const {
        std::ofstream f(path, std::ios::binary | std::ios::trunc);
        f.write("NKT1", 4);
        const uint32_t count = static_cast<uint32_t>(order.size());
        f.write(reinterpret_cast<const char*>(&count), 4);
        for (const auto& name : order) {
            const auto& it = items.at(name);
            char nm[32] = {0};
            std::strncpy(nm, name.c_str(), 31);
            const uint32_t pad = 0;
            const uint64_t n = it.second.size() / (it.first == 3 ? 8 : 4);
            f.write(nm, 32); f.write(reinterpret_cast<const char*>(&it.first), 4); f.write(reinterpret_cast<const char*>(&pad), 4);
            f.write(reinterpret_cast<const char*>(&n), 8);
            f.write(reinterpret_cast<const char*>(it.second.data()), static_cast<std::streamsize>(it.second.size()));
            const char zeros[8] = {0};
            f.write(zeros, static_cast<std::streamsize>((8 - it.second.size() % 8) % 8));
        }
        return f.good();
    }
    static bool Read(const std::string& path, std::map<std::string, std::vector<float>>* floats) {
        std::ifstream f(path, std::ios::binary);
        std::vector<char> raw((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        if (raw.size() < 8 || std::memcmp(raw.data(), "NKT1", 4) != 0) return false;
        uint32_t count; std::memcpy(&count, raw.data() + 4, 4);
        size_t at = 8;
        for (uint32_t i = 0; i < count; ++i) {
            if (at + 48 > raw.size()) return false;
            uint32_t dtype; uint64_t n;
            std::memcpy(&dtype, raw.data() + at + 32, 4); std::memcpy(&n, raw.data() + at + 40, 8);
            const size_t bytes = n * (dtype == 3 ? 8 : 4);
            if (at + 48 + bytes > raw.size()) return false;
            if (dtype == 0) {
                std::vector<float> v(n);
                std::memcpy(v.data(), raw.data() + at + 48, bytes);
                (*floats)[std::string(raw.data() + at)] = std::move(v);
            }
            at += 48 + ((bytes + 7) & ~size_t{7});
        }
        return true;
    }
};

void PutVec3(std::vector<float>& out, const nuka::math::Vec3& v) { out.push_back(v.x); out.push_back(v.y); out.push_back(v.z); }
void PutPose(std::vector<float>& out, const nuka::math::Transform& t) {
    PutVec3(out, t.position);
    out.push_back(t.rotation.w); out.push_back(t.rotation.x); out.push_back(t.rotation.y); out.push_back(t.rotation.z);
}

// The cooked model's tables, for comparing another cooker's output with the reference's cook of the same scene.
void DumpModel(const nk::Model& m, Container* c) {
    const auto& cap = m.capacities;
    c->U32("cap", {cap.env_count, cap.articulations_per_env, cap.dofs_per_env, cap.links_per_env, cap.bodies_per_env, cap.max_contacts_per_env,
                   cap.max_rows_per_env, cap.max_bodies_total, cap.max_excluded_pairs, cap.joint_limit_rows_per_env, cap.joint_friction_rows_per_env,
                   cap.joint_drive_rows_per_env, cap.rigid_contact_rows_per_env});
    const auto& a = m.articulation;
    c->U32("parent_link", a.parent_link);
    c->U32("joint_type", std::vector<uint32_t>(a.joint_type.begin(), a.joint_type.end()));
    std::vector<float> axis, offset, local, inertial, init_pose, geom_local;
    for (const auto& v : a.joint_axis) PutVec3(axis, v);
    for (const auto& v : a.parent_offset) PutVec3(offset, v);
    for (const auto& t : a.link_local_pose) PutPose(local, t);
    for (const auto& t : a.link_inertial_frame) PutPose(inertial, t);
    for (const auto& t : a.initial_link_pose) PutPose(init_pose, t);
    for (const auto& t : a.link_geom_local) PutPose(geom_local, t);
    c->F32("joint_axis", axis); c->F32("parent_offset", offset); c->F32("link_local_pose", local); c->F32("link_inertial_frame", inertial);
    c->F32("initial_link_pose", init_pose); c->F32("link_geom_local", geom_local);
    c->U32("link_body", a.link_body);
    c->F32("link_inertia_spatial", a.link_inertia_spatial);
    c->F32("joint_damping", a.joint_damping); c->F32("joint_armature", a.joint_armature); c->F32("joint_frictionloss", a.joint_frictionloss);
    c->F32("joint_stiffness", a.joint_stiffness); c->F32("joint_spring_reference", a.joint_spring_reference);
    c->F32("joint_limit_lower", a.joint_limit_lower); c->F32("joint_limit_upper", a.joint_limit_upper);
    c->U32("joint_limit_flags", std::vector<uint32_t>(a.joint_limit_flags.begin(), a.joint_limit_flags.end()));
    c->F32("initial_q", a.initial_q);
    std::vector<float> base; PutPose(base, a.base_pose); c->F32("base_pose", base);
    c->U32("artic", {a.dof_count, a.link_count, a.root_link, a.articulation_count});
    c->U32("link_geom_kind", a.link_geom_kind); c->F32("link_geom_params", a.link_geom_params);
    c->F32("hold_targets", m.hold_drives.targets); c->F32("hold_stiffness", m.hold_drives.stiffness); c->F32("hold_damping", m.hold_drives.damping);
    c->F32("hold_force_limits", m.hold_drives.force_limits); c->F32("hold_joint_force_limits", m.hold_drives.joint_force_limits);
    std::vector<uint32_t> kind, contype, conaff, group;
    std::vector<int32_t> body_id;
    std::vector<float> params;
    for (const auto& s : m.shape_table_rows) {
        kind.push_back(s.kind); contype.push_back(s.contype); conaff.push_back(s.conaffinity); group.push_back(s.group); body_id.push_back(s.body_id);
        for (float p : s.params) params.push_back(p);
    }
    c->U32("shape_kind", kind); c->U32("shape_contype", contype); c->U32("shape_conaffinity", conaff); c->U32("shape_group", group);
    c->I32("shape_body_id", body_id); c->F32("shape_params", params);
    std::vector<float> bpose, binv, binertial;
    for (const auto& b : m.body_init) { PutPose(bpose, b.pose); binv.push_back(b.inv_mass); PutVec3(binv, b.inv_inertia); PutPose(binertial, b.inertial_frame); }
    c->F32("body_pose", bpose); c->F32("body_inv_mass_inertia", binv); c->F32("body_inertial_frame", binertial);
    c->U64("excluded_pairs", m.excluded_pairs);
    c->U32("body_to_link", m.body_to_link); c->U32("body_collidable_link", m.body_collidable_link);
    std::vector<float> coll_local;
    for (const auto& t : m.body_collidable_local) PutPose(coll_local, t);
    c->F32("body_collidable_local", coll_local);
    c->U32("dof_to_link", m.dof_to_link); c->U32("dof_to_component", m.dof_to_component);
    c->F32("model_scalars", {m.ground_height, m.friction_coefficient, m.baumgarte_max_velocity, m.overlap_recovery_velocity,
                             m.contact_solref[0], m.contact_solref[1]});
    std::vector<float> buckets;
    for (const auto& b : m.material_buckets) for (float v : b.values) buckets.push_back(v);
    c->F32("material_buckets", buckets);
    c->U32("body_material_bucket", m.body_material_bucket);
}

struct Args {
    std::string scene, state, dump;
    uint32_t envs = 1, vel_iters = 0, pos_iters = 0xffffffffu, steps = 0, every = 1, control_mode = 0, task_link = 0;
    float dt = 1.0f / 200.0f;
    bool contacts = true, cook_only = false, taps = false;
    int warm = 0, timed = 0, repeats = 1;
    float active_sigma = 0.0f;
};

template <typename T>
std::vector<T> Download(nk::World& w, nk::FieldId id, size_t count) {
    std::vector<T> out(count);
    if (count != 0 && !w.GetData().DownloadField(id, out.data(), count * sizeof(T))) out.clear();
    return out;
}

}  // namespace

int main(int argc, char** argv) {
    Args a;
    for (int i = 1; i < argc; ++i) {
        const std::string k = argv[i];
        auto next = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
        if (k == "--scene") a.scene = next();
        else if (k == "--envs") a.envs = static_cast<uint32_t>(std::atoi(next()));
        else if (k == "--dt") a.dt = static_cast<float>(std::atof(next()));
        else if (k == "--vel-iters") a.vel_iters = static_cast<uint32_t>(std::atoi(next()));
        else if (k == "--pos-iters") a.pos_iters = static_cast<uint32_t>(std::atoi(next()));
        else if (k == "--control-mode") a.control_mode = static_cast<uint32_t>(std::atoi(next()));
        else if (k == "--task-link") a.task_link = static_cast<uint32_t>(std::atoi(next()));
        else if (k == "--steps") a.steps = static_cast<uint32_t>(std::atoi(next()));
        else if (k == "--every") a.every = std::max(1, std::atoi(next()));
        else if (k == "--state") a.state = next();
        else if (k == "--dump") a.dump = next();
        else if (k == "--no-contacts") a.contacts = false;
        else if (k == "--cook-only") a.cook_only = true;
        else if (k == "--taps") a.taps = true;
        else if (k == "--time") { std::sscanf(next(), "%d,%d,%d", &a.warm, &a.timed, &a.repeats); }
        else if (k == "--active") a.active_sigma = static_cast<float>(std::atof(next()));
        else { std::fprintf(stderr, "unknown argument %s\n", k.c_str()); return 2; }
    }
    if (a.scene.empty()) { std::fprintf(stderr, "--scene is required\n"); return 2; }
    try {
        nuka::scene::SceneIR scene = nuka::scene::nks::Load(a.scene);
        nuka::scene::cook::CookToModelOptions options;
        options.enable_contacts = a.contacts;
        auto cooked = nuka::scene::cook::CookToModel(scene, static_cast<int>(a.envs), options);
        Container out;
        cooked.model.drive_mode = a.control_mode;          // as src/c_abi/world.cpp:160-166 routes the descriptor's control mode
        cooked.model.osc_task_link = a.task_link;          // src/c_abi/world.cpp:167
        DumpModel(cooked.model, &out);
        if (a.cook_only) {
            if (!a.dump.empty() && !out.Write(a.dump)) { std::fprintf(stderr, "cannot write %s\n", a.dump.c_str()); return 1; }
            std::printf("{\"cooked\": true, \"links\": %u, \"dofs\": %u, \"bodies\": %u, \"contact_slots\": %u}\n", cooked.model.capacities.links_per_env,
                        cooked.model.capacities.dofs_per_env, cooked.model.capacities.bodies_per_env, cooked.model.capacities.max_contacts_per_env);
            return 0;
        }
        nphi::Device* dev = nphi::InitBestDevice();
        nphi::Backend* backend = dev ? nphi::DeviceInitBackend(dev, nullptr) : nullptr;
        if (backend == nullptr) { std::fprintf(stderr, "no CUDA backend\n"); return 3; }
        nk::Pipeline::SolverConfig cfg;
        cfg.dt = a.dt;
        if (a.vel_iters != 0u) { cfg.vel_iters = static_cast<uint16_t>(a.vel_iters); cfg.velocity_iterations_override = true; }
        if (a.pos_iters != 0xffffffffu) cfg.pos_iters = static_cast<uint16_t>(a.pos_iters);
        const uint32_t L = cooked.model.capacities.links_per_env, n = cooked.model.capacities.dofs_per_env;
        const uint32_t B = cooked.model.capacities.bodies_per_env, S = cooked.model.capacities.max_contacts_per_env;
        const uint32_t E = a.envs;
        nk::World world(std::move(cooked.model), E, dev, backend, cfg);
        if (!world.Ready()) { std::fprintf(stderr, "world creation failed: %s\n", world.CreationError().c_str()); return 4; }
        // per-env state: the reference seeds every env from the template; callers randomise through field uploads
        if (!a.state.empty()) {
            std::map<std::string, std::vector<float>> st;
            if (!Container::Read(a.state, &st)) { std::fprintf(stderr, "cannot read %s\n", a.state.c_str()); return 2; }
            const std::pair<const char*, nk::FieldId> fields[] = {
                {"q", nk::FieldId::Q}, {"qdot", nk::FieldId::Qdot}, {"base_pose", nk::FieldId::BasePose}, {"link_velocity", nk::FieldId::LinkVelocity},
                {"drive_target", nk::FieldId::DriveTarget}, {"vel_target", nk::FieldId::VelocityTarget}, {"acc_target", nk::FieldId::AccelerationTarget},
                {"kp", nk::FieldId::DriveStiffness}, {"kd", nk::FieldId::DriveDamping}, {"force_limit", nk::FieldId::DriveForceLimit},
                {"noload_speed", nk::FieldId::ActuatorNoloadSpeed}, {"feedforward", nk::FieldId::JointF},
                {"task_target", nk::FieldId::TaskTarget}, {"task_rotation", nk::FieldId::TaskRotationTarget}, {"task_frame", nk::FieldId::TaskLocalPose},
                {"null_kp", nk::FieldId::TaskNullspaceStiffness}, {"null_kd", nk::FieldId::TaskNullspaceDamping},
                {"body_pose", nk::FieldId::BodyPose}};
            for (const auto& f : fields) {
                const auto it = st.find(f.first);
                if (it == st.end()) continue;
                if (!world.GetData().UploadField(f.second, it->second.data(), it->second.size() * 4)) {
                    std::fprintf(stderr, "upload of %s (%zu floats) was rejected\n", f.first, it->second.size());
                    return 2;
                }
            }
            if (world.ForwardKinematics() != nphi::Status::Ok) { std::fprintf(stderr, "forward kinematics failed\n"); return 4; }
            if (const auto it = st.find("link_velocity"); it != st.end())      // the refresh above may rewrite link velocities
                world.GetData().UploadField(nk::FieldId::LinkVelocity, it->second.data(), it->second.size() * 4);
        }
        world.Synchronize();
        out.U32("run", {E, L, n, B, S, a.vel_iters, a.steps, a.every});
        out.F32("run_dt", {a.dt});
        if (!a.dump.empty()) {
            // single-op dynamics without the velocity update: joint accelerations and the mass matrix of the start state
            if (L != 0u) {
                nphi::ArticulationDynamicsParams dyn{};
                dyn.dt = a.dt; dyn.max_dof = n; dyn.integrate_velocity = 0u; dyn.fold_drive_damping = 0u; dyn.reuse_mass = 0u;
                dyn.gravity[0] = cfg.gravity[0]; dyn.gravity[1] = cfg.gravity[1]; dyn.gravity[2] = cfg.gravity[2];
                dyn.articulation_count = E; dyn.total_link_count = E * L; dyn.apply_link_wrench = 0u; dyn.max_links = L; dyn.links_per_env = L;
                dyn.bodies_per_env = B;
                if (world.DispatchOp(nphi::NkOp::ArticulationDynamics, &dyn) != nphi::Status::Ok) { std::fprintf(stderr, "dynamics dispatch failed\n"); return 4; }
                world.Synchronize();
                out.F32("dyn_qddot", Download<float>(world, nk::FieldId::Qddot, size_t{E} * L));
                out.F32("dyn_mass", Download<float>(world, nk::FieldId::M, size_t{E} * n * n));
                out.F32("dyn_bias", Download<float>(world, nk::FieldId::ArticulationBias, size_t{E} * n));
                out.F32("dyn_link_acceleration", Download<float>(world, nk::FieldId::LinkAcceleration, size_t{E} * L * 6));
            }
            out.F32("start_q", Download<float>(world, nk::FieldId::Q, size_t{E} * L));
            out.F32("start_link_pose", Download<float>(world, nk::FieldId::LinkPose, size_t{E} * L * 7));
            out.F32("start_body_pose", Download<float>(world, nk::FieldId::BodyPose, size_t{E} * B * 7));
            out.F32("start_kp", Download<float>(world, nk::FieldId::DriveStiffness, size_t{E} * L));
            out.F32("start_kd", Download<float>(world, nk::FieldId::DriveDamping, size_t{E} * L));
            out.F32("start_force_limit", Download<float>(world, nk::FieldId::DriveForceLimit, size_t{E} * L));
            out.F32("start_drive_target", Download<float>(world, nk::FieldId::DriveTarget, size_t{E} * L));
            std::vector<float> tq, tqd, tbase, ttwist, tbody, tresidual, tpseudo, tlinkpseudo, tbodypl, tbodypa, tlimit, tdepth;
            std::vector<uint32_t> tstatus, tpairs, tpaircount, tcount, tsweeps, status_any, tstatusany;
            for (uint32_t s = 1; s <= a.steps; ++s) {
                const nk::StepResult r = world.Step();
                if (!r.AllOk()) { std::fprintf(stderr, "step %u failed\n", s); return 5; }
                {   // the gyro bit describes one step only: keep every bit any step so far has raised
                    const auto now = Download<uint32_t>(world, nk::FieldId::EnvStatus, E);
                    if (status_any.size() != now.size()) status_any.assign(now.size(), 0u);
                    for (size_t i = 0; i < now.size(); ++i) status_any[i] |= now[i];
                }
                if (s % a.every != 0u && s != 1u && s != a.steps) continue;
                world.Synchronize();
                auto append = [](auto& dst, const auto& src) { dst.insert(dst.end(), src.begin(), src.end()); };
                append(tq, Download<float>(world, nk::FieldId::Q, size_t{E} * L));
                append(tqd, Download<float>(world, nk::FieldId::Qdot, size_t{E} * L));
                append(tbase, Download<float>(world, nk::FieldId::BasePose, size_t{E} * (L ? 7 : 0)));
                append(ttwist, Download<float>(world, nk::FieldId::LinkVelocity, size_t{E} * L * 6));
                append(tbody, Download<float>(world, nk::FieldId::BodyPose, size_t{E} * B * 7));
                append(tstatus, Download<uint32_t>(world, nk::FieldId::EnvStatus, E));
                append(tstatusany, status_any);
                append(tresidual, Download<float>(world, nk::FieldId::SolverResidual, size_t{E} * 4));
                append(tsweeps, Download<uint32_t>(world, nk::FieldId::VbdVelocitySweepCount, E));
                if (a.taps) {
                    append(tpseudo, Download<float>(world, nk::FieldId::QdotPseudo, size_t{E} * L));
                    append(tlinkpseudo, Download<float>(world, nk::FieldId::LinkVelocityPseudo, size_t{E} * L * 6));
                    append(tbodypl, Download<float>(world, nk::FieldId::BodyPseudoLinearVelocity, size_t{E} * B * 3));
                    append(tbodypa, Download<float>(world, nk::FieldId::BodyPseudoAngularVelocity, size_t{E} * B * 3));
                    append(tlimit, Download<float>(world, nk::FieldId::JointLimitImpulse, size_t{E} * L * 2));
                    if (S != 0u) append(tdepth, Download<float>(world, nk::FieldId::UcontactDepth, size_t{E} * S * 4));
                }
                if (S != 0u) {
                    append(tpaircount, Download<uint32_t>(world, nk::FieldId::PairCount, E));
                    append(tpairs, Download<uint32_t>(world, nk::FieldId::CandidatePairs, size_t{E} * S * 2));
                    append(tcount, Download<uint32_t>(world, nk::FieldId::UcontactCount, size_t{E} * S));
                }
                std::vector<uint32_t> mark = {s};
                auto it = out.items.find("traj_steps");
                std::vector<uint32_t> marks;
                if (it != out.items.end()) { marks.resize(it->second.second.size() / 4); std::memcpy(marks.data(), it->second.second.data(), it->second.second.size()); }
                marks.push_back(s);
                out.U32("traj_steps", marks);
            }
            out.F32("traj_q", tq); out.F32("traj_qdot", tqd); out.F32("traj_base_pose", tbase); out.F32("traj_link_velocity", ttwist);
            out.F32("traj_body_pose", tbody); out.U32("traj_status", tstatus); out.U32("traj_status_any", tstatusany); out.F32("traj_solver_residual", tresidual); out.U32("traj_solver_sweeps", tsweeps);
            if (a.taps) {
                out.F32("traj_qdot_pseudo", tpseudo); out.F32("traj_link_velocity_pseudo", tlinkpseudo);
                out.F32("traj_body_pseudo_linear", tbodypl); out.F32("traj_body_pseudo_angular", tbodypa);
                out.F32("traj_joint_limit_impulse", tlimit); out.F32("traj_contact_depth", tdepth);
            } out.U32("traj_pair_count", tpaircount);
            out.U32("traj_candidate_pairs", tpairs); out.U32("traj_contact_count", tcount);
            if (!out.Write(a.dump)) { std::fprintf(stderr, "cannot write %s\n", a.dump.c_str()); return 1; }
        }
        if (a.timed > 0) {
            // wall clock between two synchronisations, as the reference's own gate measures it
            // (tests/perf/test_go2_4096env_step_time.cpp:4-12)
            std::printf("{\"impl\": \"reference-gpu\", \"scene\": \"%s\", \"envs\": %u, \"dt\": %g, \"vel_iters\": %u", a.scene.c_str(), E, a.dt, a.vel_iters);
            for (int mode = 0; mode < 2; ++mode) {
                if (world.SetExecutionMode(mode == 0 ? nk::World::ExecutionMode::Eager : nk::World::ExecutionMode::Graph) != nphi::Status::Ok) {
                    std::printf(", \"%s\": null", mode == 0 ? "eager_ms_per_step" : "graph_ms_per_step");
                    continue;
                }
                std::vector<float> ms;
                bool ok = true;
                for (int rep = 0; rep < a.repeats && ok; ++rep) {
                    uint32_t submitted = 0;
                    ok = world.StepConfigured(static_cast<uint32_t>(a.warm), &submitted) == nphi::Status::Ok && world.Synchronize() == nphi::Status::Ok;
                    const auto t0 = std::chrono::steady_clock::now();
                    ok = ok && world.StepConfigured(static_cast<uint32_t>(a.timed), &submitted) == nphi::Status::Ok;
                    ok = ok && world.Synchronize() == nphi::Status::Ok;
                    const double wall = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
                    ms.push_back(static_cast<float>(wall / a.timed));
                }
                std::sort(ms.begin(), ms.end());
                if (ok && !ms.empty()) std::printf(", \"%s\": %.5f", mode == 0 ? "eager_ms_per_step" : "graph_ms_per_step", ms[ms.size() / 2]);
                else std::printf(", \"%s\": null", mode == 0 ? "eager_ms_per_step" : "graph_ms_per_step");
            }
            if (a.active_sigma > 0.0f && L != 0u) {
                // fresh targets every step: one host-to-device copy of E x L floats, then one eager step
                world.SetExecutionMode(nk::World::ExecutionMode::Eager);
                const std::vector<float> hold = Download<float>(world, nk::FieldId::DriveTarget, size_t{E} * L);
                std::vector<std::vector<float>> pool(16, hold);
                uint64_t rng = 0x9e3779b97f4a7c15ull;
                auto uniform = [&]() { rng ^= rng << 13; rng ^= rng >> 7; rng ^= rng << 17; return static_cast<float>((rng >> 11) * (1.0 / 9007199254740992.0)); };
                for (auto& set : pool)
                    for (size_t i = 0; i < set.size(); ++i) {
                        if (i % L == 0u) continue;                                           // slot 0 is the root
                        const float u1 = std::max(uniform(), 1.0e-7f), u2 = uniform();
                        set[i] += a.active_sigma * std::sqrt(-2.0f * std::log(u1)) * std::cos(6.2831853f * u2);
                    }
                bool ok = true;
                uint32_t submitted = 0;
                auto one = [&](int k) {
                    ok = ok && world.GetData().UploadField(nk::FieldId::DriveTarget, pool[k % 16].data(), pool[k % 16].size() * 4) &&
                         world.StepConfigured(1u, &submitted) == nphi::Status::Ok;
                };
                for (int k = 0; k < std::max(a.warm / 10, 10); ++k) one(k);
                world.Synchronize();
                const auto t0 = std::chrono::steady_clock::now();
                for (int k = 0; k < a.timed; ++k) one(k);
                ok = ok && world.Synchronize() == nphi::Status::Ok;
                const double wall = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
                if (ok) std::printf(", \"active_sigma\": %g, \"active_eager_ms_per_step\": %.5f", a.active_sigma, wall / a.timed);
                else std::printf(", \"active_eager_ms_per_step\": null");
            }
            const auto status = Download<uint32_t>(world, nk::FieldId::EnvStatus, E);
            uint32_t any = 0; for (uint32_t s : status) any |= s;
            std::printf(", \"status_or\": %u, \"timed_steps\": %d, \"warmup_steps\": %d, \"repeats\": %d}\n", any, a.timed, a.warm, a.repeats);
        }
        return 0;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_driver: %s\n", e.what());
        return 1;
    }
}

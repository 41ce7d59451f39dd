// Device code of the fused step kernel: one warp advances one env through the whole pipeline (kinematics, drives,
// dynamics, collision, row assembly, block-descent solve, integration) with every intermediate in the warp's
// shared-memory slice; global memory sees only the env's state.
// The stage order is the reference's nk::Pipeline::BuildInterval (src/nk/pipeline/pipeline.cpp:367-986).
// Each instantiation of step_kernel is compiled in a translation unit of its own (nkb_step_*.cu) so that the
// variants build in parallel; NKB_STEP_VARIANT defines the host-side handle of one.
#pragma once
#include <cuda_runtime.h>
#include <cstdlib>
#include <mutex>
#include "nkb_solver.cuh"
#include "nkb_lbvh.cuh"
#include "nkb_manifold.cuh"
#include "nkb_launch.h"

namespace nkb {

// Torque-free rotation of a free rigid body over one step, in its principal frame (the quantity of the reference's
// SolveFreeRotation, ops/rigid_types.cuh:39-122, used by ops/articulation.cu:1059-1116): the implicit-midpoint form of
// Euler's equations for the scaled angular momentum u,
//     g(u) = u - u0 + c * (m_y m_z, m_z m_x, m_x m_y) = 0,   m = (u0 + u) / 2,   c = dt (a_y - a_z, a_z - a_x, a_x - a_y),
// with a the scaled inverse principal inertias.  Newton's method: the Jacobian is the identity plus three off-diagonal
// pairs, small enough to invert through its column triple products; a step is halved (at most 8 times) until the
// residual's largest component drops; at most 12 steps to 1e-6.  `mid_out` is the midpoint angular velocity.
struct FreeRotation {
    V3 u0, c;
    NKB_DEV V3 midpoint(V3 u) const { return (u0 + u) * 0.5f; }
    NKB_DEV V3 residual(V3 u) const {
        const V3 m = midpoint(u);
        return mk3(u.x - u0.x + c.x * m.y * m.z, u.y - u0.y + c.y * m.z * m.x, u.z - u0.z + c.z * m.x * m.y);
    }
    NKB_DEV static float largest(V3 r) { return fmaxf(fabsf(r.x), fmaxf(fabsf(r.y), fabsf(r.z))); }
    // Newton direction d with (dg/du) d = r at midpoint m, by Cramer's rule on the Jacobian's columns; false when singular
    NKB_DEV bool direction(V3 m, V3 r, V3& d) const {
        const V3 col0 = mk3(1.0f, 0.5f * c.y * m.z, 0.5f * c.z * m.y);
        const V3 col1 = mk3(0.5f * c.x * m.z, 1.0f, 0.5f * c.z * m.x);
        const V3 col2 = mk3(0.5f * c.x * m.y, 0.5f * c.y * m.x, 1.0f);
        const V3 c12 = cross(col1, col2);
        const float det = dot(col0, c12);
        if (!isfinite(det) || fabsf(det) < 1.0e-12f) return false;
        d = mk3(dot(r, c12), dot(col0, cross(r, col2)), dot(col0, cross(col1, r))) * (1.0f / det);
        return true;
    }
};

NKB_DEV bool solve_free_rotation(V3 w0, V3 inv_i, float dt, V3& mid_out) {
    mid_out = mk3(0.f, 0.f, 0.f);
    const V3 momentum = mk3(w0.x / inv_i.x, w0.y / inv_i.y, w0.z / inv_i.z);
    const float scale = FreeRotation::largest(momentum);
    if (scale == 0.0f) return true;                     // at rest
    const V3 a = inv_i * scale;
    FreeRotation eq;
    eq.u0 = momentum * (1.0f / scale);
    eq.c = mk3(dt * (a.y - a.z), dt * (a.z - a.x), dt * (a.x - a.y));
    V3 u = eq.u0;
    for (int newton = 0; newton <= 12; ++newton) {
        const V3 r = eq.residual(u);
        const float size = FreeRotation::largest(r);
        if (!isfinite(size)) return false;
        if (size <= 1.0e-6f) {
            const V3 m = eq.midpoint(u);
            mid_out = mk3(a.x * m.x, a.y * m.y, a.z * m.z);
            return true;
        }
        V3 d;
        if (newton == 12 || !eq.direction(eq.midpoint(u), r, d)) return false;
        float fraction = 1.0f;
        bool improved = false;
        for (int halving = 0; halving < 8 && !improved; ++halving, fraction *= 0.5f) {
            const V3 trial = u - d * fraction;
            const float trial_size = FreeRotation::largest(eq.residual(trial));
            if (isfinite(trial_size) && trial_size < size) { u = trial; improved = true; }
        }
        if (!improved) return false;
    }
    return false;
}

NKB_DEV void stage_integrate_bodies(Env& e, bool use_pseudo) {
    const TemplateView& t = *e.t;
    const float dt = t.cfg.dt;
    for (uint32_t b = e.lane; b < t.B; b += 32u) {
        if (!(__ldg(t.inv_mass + b) > 0.f) || __ldg(t.body_to_link + b) != kNoLink) continue;
        float* pose = sm_bpose(e, b);
        float* bv = sm_bvel(e, b);
        const V3 inv_i = ld3(t.inv_inertia + 3u * b);
        const Q4 iq = ldq(t.inertial_quat + 4u * b);
        const Q4 principal = qnorm_le(qmul(ldq(pose + 3), iq), 1.0e-12f);
        const V3 w0 = qrot(mkq(principal.w, -principal.x, -principal.y, -principal.z), ld3(bv + 3));
        V3 midpoint;
        if (!solve_free_rotation(w0, inv_i, dt, midpoint)) { e.status |= kStatusGyroFailure; continue; }
        const V3 momentum = qrot(principal, mk3(w0.x / inv_i.x, w0.y / inv_i.y, w0.z / inv_i.z));
        V3 v = ld3(bv);
        const V3 w = qrot(principal, midpoint);
        const V3 ipos = ld3(t.inertial_pos + 3u * b);
        const V3 center = ld3(pose) + qrot(ldq(pose + 3), ipos);
        Q4 q = qnorm_le(qmul(mkq(1.0f, 0.5f * dt * w.x, 0.5f * dt * w.y, 0.5f * dt * w.z), ldq(pose + 3)), 1.0e-12f);
        if (use_pseudo) {
            const float* ps = sm_bpseudo(e, b);
            v = v + ld3(ps);
            q = qnorm_le(qmul(mkq(1.0f, 0.5f * dt * ps[3], 0.5f * dt * ps[4], 0.5f * dt * ps[5]), q), 1.0e-12f);
        }
        stq(pose + 3, q);
        st3(pose, center + v * dt - qrot(q, ipos));
        float winv[6];
        world_inv_inertia(q, iq, inv_i, winv);
        st3(bv + 3, sym_mulv(winv, momentum));
    }
    __syncwarp();
}

// Applied drive efforts from the solved drive multipliers (ops/articulation.cu:999-1016).
NKB_DEV void stage_readout_drives(Env& e, uint32_t nheads) {
    const TemplateView& t = *e.t;
    float* tmp = sm_vec(e, kVecTmp);
    tmp[e.lane] = 0.f;
    uint32_t* has = reinterpret_cast<uint32_t*>(sm_vec(e, kVecTmp2));
    has[e.lane] = 0u;
    __syncwarp();
    for (uint32_t h = e.lane; h < nheads; h += 32u) {
        const uint32_t fl = hu(e, HF_FLAGS, h);
        if (fl & kHeadDrive) { const uint32_t link = hu(e, HF_REF, h); tmp[link] = hf(e, HF_LAM, h); has[link] = 1u; }
        // a limit row's slot keeps the multiplier of the velocity solve for the next step (block_descent_tile.cuh:2556)
        if (fl & kHeadLimit) e.s->limit_lambda[((size_t)e.env * t.L + hu(e, HF_REF, h)) * 2u + (hf(e, HF_UNITV, h) < 0.f ? 1u : 0u)] = hf(e, HF_LAM, h);
    }
    __syncwarp();
    float applied = 0.f;
    if (e.lane < t.L && has[e.lane]) { applied = tmp[e.lane] / t.cfg.dt - e.drive_dissipation * e.qd; e.tau += applied; }
    if (e.lane < t.L) e.s->actuator[(size_t)e.env * t.L + e.lane] = applied;
    __syncwarp();
}

NKB_DEV void stage_store_bodies(Env& e, bool velocities) {
    const TemplateView& t = *e.t;
    float* gp = e.s->body_pose + (size_t)e.env * t.B * 7u;
    const float* sp = e.sm + e.lay->bpose;
    for (uint32_t k = e.lane; k < t.B * 7u; k += 32u) gp[k] = sp[k];
    if (!velocities) return;
    for (uint32_t b = e.lane; b < t.B; b += 32u) {
        if (__ldg(t.body_to_link + b) != kNoLink || !(__ldg(t.inv_mass + b) > 0.f)) continue;     // only free dynamic bodies move
        const size_t gb = (size_t)e.env * t.B + b;
        st3(e.s->body_linvel + gb * 3u, ld3(sm_bvel(e, b)));
        st3(e.s->body_angvel + gb * 3u, ld3(sm_bvel(e, b) + 3));
    }
}

// Register cap: measured on the 4096-env quadruped, the kernel runs fastest with about 150 registers and 12 warps per
// SM; tighter caps (144 or 128 registers, 14 warps per SM) slow every warp by more than the extra residency returns.
// NR = coordinates per lane: 1 for articulations of up to 32 coordinates, 2 for up to 64.
// kRigid = the world has free rigid bodies; without them the rigid-block solver code is compiled out.
// Worlds with free bodies are held to fewer resident warps by shared memory than by registers (38 KB per env and more),
// so their variants take a wider cap: no spills, and a team of 8 warps still fits the register file.
#ifndef NKB_MAXNREG
#define NKB_MAXNREG 176
#endif
#ifndef NKB_MAXNREG_RIGID
#define NKB_MAXNREG_RIGID 224
#endif
// The slim build of the same kernel: at 128 registers a fourth warp fits each scheduler partition, so small envs (15 KB
// of shared memory) reach 15 resident warps per SM instead of 12 and 4096 envs need two rounds instead of 2.3.  It
// spills about 200 bytes; a world takes it only where the extra residency is really there (World::BuildLayout).
#ifndef NKB_MAXNREG_SLIM
#define NKB_MAXNREG_SLIM 128
#endif
template <int NR, bool kRigid, bool kControl>
NKB_DEV void advance_env(const StepParams& p, float* sm, uint32_t env, uint32_t lane) {
    const TemplateView& t = p.t;
    const bool has_artic = t.L != 0u, has_bodies = t.B != 0u;
    const bool has_collidables = has_bodies && t.cfg.max_contacts != 0u;
    const bool use_pseudo = t.cfg.pos_iters != 0u && (t.cfg.max_contacts != 0u || t.L != 0u);
    for (uint32_t step = 0u; step < p.steps; ++step) {
        Env e;
        env_begin<NR>(e, p, sm, env, lane);
        if (p.mode == kModeRefresh) {
            if (has_artic) { stage_fk(e); }
            if (has_bodies) { stage_bodies(e, false); stage_store_bodies(e, false); }
            if (has_artic) {
                float* gp = p.s.link_pose + (size_t)env * t.L * 7u;
                for (uint32_t k = lane; k < t.L * 7u; k += 32u) gp[k] = sm[p.sm.pose + k];
            }
            return;
        }
        tick(e, 0);
        if (has_artic) {
            stage_fk(e); tick(e, 1); stage_drives(e);
            // computed torque and operational-space control (pipeline.cpp:406-426) take two passes: a force-free one on the current kinematics, the
            // controller on its mass response and accelerations, then the step's own pass
            // the controllers are compiled into the kControl builds of the kernel only (they would cost every other world registers)
            const bool two_passes = kControl && (t.cfg.control_mode == 3u || t.cfg.control_mode == 4u) && p.mode != kModeDynamicsOnly;
#pragma unroll 1
            for (int pass = two_passes ? 0 : 1; pass < 2; ++pass) {
                stage_dynamics<NR>(e, pass == 1 && p.mode != kModeDynamicsOnly);
                if constexpr (kControl) { if (pass == 0) stage_computed_torque<NR>(e); }
            }
            tick(e, 2);
        }
        if (p.mode == kModeDynamicsOnly) {
            if (lane < t.L) p.s.qddot[(size_t)env * t.L + lane] = e.qdd;
            return;
        }
        uint32_t pair_count = 0u, nheads = 0u;
        if (has_bodies) stage_bodies(e, true);
        if (has_collidables) {
            stage_aabbs(e);
            pair_count = t.broadphase_tree != 0u ? stage_pairs_lbvh(e) : stage_pairs(e);
            tick(e, 3);
            narrowphase_frames(e);
            if constexpr (kRigid) team_fork(e, kTeamNarrowphase, pair_count, [&](uint32_t first, uint32_t stride) { narrowphase_range(e, pair_count, first, stride); });
            else narrowphase_range(e, pair_count, 0u, 1u);
            tick(e, 4);
            stage_store_contacts(e, pair_count);
            tick(e, 5);
        }
        if (p.mode == kModeCollideOnly) {
            if (has_bodies) stage_store_bodies(e, false);
            uint32_t st = e.status;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) st |= __shfl_xor_sync(NKB_FULL, st, o);
            if (lane == 0u) p.s.status[env] |= st;
            return;
        }
        nheads = stage_rows<NR>(e, pair_count);
        tick(e, 6);
        if constexpr (kRigid) team_fork(e, kTeamWarmStart, nheads, [&](uint32_t first, uint32_t stride) { warm_start_range(e, nheads, first, stride); });
        else warm_start_range(e, nheads, 0u, 1u);
        __syncwarp();
        tick(e, 7);
        stage_solve<NR, kRigid>(e, nheads);
        if (has_collidables) {
            stage_cache_commit(e, nheads, [&](uint32_t ncontact) {
                if constexpr (kRigid) team_fork(e, kTeamCacheOwners, ncontact, [&](uint32_t first, uint32_t stride) { cache_owners_range(e, ncontact, first, stride); });
                else cache_owners_range(e, ncontact, 0u, 1u);
            });
        }
        if (has_artic) stage_readout_drives(e, nheads);
        tick(e, 12);
        if (has_artic) { stage_integrate_links(e, use_pseudo); }
        if (has_bodies) stage_integrate_bodies(e, use_pseudo);
        __syncwarp();
        if (has_artic) { stage_fk(e); stage_link_velocities(e); stage_store_links(e); }
        if (has_bodies) {
            // link mirrors follow the new link poses; free bodies keep their integrated pose
            for (uint32_t b = lane; b < t.B; b += 32u) {
                const uint32_t link = __ldg(t.body_to_link + b);
                if (link == kNoLink) continue;
                float* bp = sm_bpose(e, b);
                const float* lp = sm_pose(e, link);
                if (__ldg(t.body_geom_kind + b) != 0u) {
                    const Q4 pq = ldq(lp + 3);
                    st3(bp, ld3(lp) + qrot(pq, ld3(t.body_geom_pos + 3u * b)));
                    stq(bp + 3, qmul(pq, ldq(t.body_geom_quat + 4u * b)));
                } else {
#pragma unroll
                    for (int k = 0; k < 7; ++k) bp[k] = lp[k];
                }
            }
            __syncwarp();
            stage_store_bodies(e, true);
        }
        uint32_t st = e.status;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) st |= __shfl_xor_sync(NKB_FULL, st, o);
        // The gyro bit describes the latest step only (the reference clears it before every body integration,
        // ops/articulation.cu:1053-1056, 1810-1812); every other bit stays until the env is reset.
        if (lane == 0u && (st != 0u || has_bodies)) {
            const uint32_t before = p.s.status[env];
            const uint32_t after = (has_bodies ? before & ~kStatusGyroFailure : before) | st;
            if (after != before) p.s.status[env] = after;
        }
        __syncwarp();
        tick(e, 13);
    }
}

// A helper warp's life: wait for a command, do its share (rigid blocks of a colour on private Newton scratch, or a slice of
// a stage's outer loop), answer, until told to leave (or until a wait runs out).
template <bool kRigid>
NKB_DEV void team_helper(float* sm, const SmemLayout& shared_layout, const TemplateView& t, const StateView& state, uint32_t env,
                         uint32_t member, uint32_t lane, uint32_t vstride) {
    // private copies of the regions a block descent scratches in (same arrangement as the env's own: Newton matrix, block
    // mass, staged rows; then the solver vectors); everything else is the env's own
    const uint32_t newton_span = shared_layout.rjac + 24u * shared_layout.rjac_heads - shared_layout.chol;
    const uint32_t base = shared_layout.team_area + kTeamCommandWords + ((4u * shared_layout.team + 3u) & ~3u) + (member - 1u) * shared_layout.helper_words;
    const uint32_t newton_shift = base - shared_layout.chol, vec_shift = base + newton_span - shared_layout.vecs;
    const TeamCommand* cmd = team_command(sm, shared_layout);
    uint32_t* answer = reinterpret_cast<uint32_t*>(team_result(sm, shared_layout, member));
    uint32_t last = 0u;
#pragma unroll 1
    for (uint32_t trips = 0u; trips < (1u << 24); ++trips) {
        // every lane polls the same word, so the warp never splits over the wait
        uint32_t seq = last;
        {
            const long long begin = clock64();
            while ((seq = team_peek(&cmd->seq)) == last) {
                if (clock64() - begin > kTeamPatience) break;
                __nanosleep(100);
            }
        }
        seq = __shfl_sync(NKB_FULL, seq, 0);
        __syncwarp();
        if (seq == last) {                                   // the lead never called: leave, and say so
            if (lane == 0u) atomicOr(state.status + env, kStatusTeamTimeout);
            return;
        }
        __threadfence_block();
        last = seq;
        const uint32_t op = team_peek(&cmd->op);
        if (op == kTeamExit) return;
        if ((shared_layout.team_drill & 2u) != 0u) continue;          // drill: a helper that never answers
        RigidResult r = {0.f, 0.f, 0u};
        const uint32_t k_begin = cmd->k_begin, k_end = cmd->k_end, nblocks = cmd->nblocks;
        if (op == kTeamDescend && k_begin < k_end && k_end <= nblocks && nblocks <= t.B + 1u) {
            RigidRun run;
            run.sm = sm; run.lay = &shared_layout; run.t = &t; run.lane = lane; run.vstride = vstride;
            run.newton_shift = newton_shift; run.vec_shift = vec_shift;
            run.nheads = cmd->nheads; run.nblocks = nblocks; run.iteration = cmd->iteration; run.tol = cmd->tol;
#ifdef NKB_STAGE_TAPS
            const long long tap0 = clock64();
#endif
            r = descend_rigid_run<kRigid>(run, k_begin, k_end, member, shared_layout.team, cmd->position != 0u);
#ifdef NKB_STAGE_TAPS
            if (state.dbg_cycles != nullptr && lane == 0u && member == 1u) {
                uint32_t* cyc = state.dbg_cycles + (size_t)env * 32u;
                cyc[30] += (uint32_t)(clock64() - tap0); cyc[31] += 1u;
            }
#endif
        }
        else if (op == kTeamNarrowphase || op == kTeamWarmStart || op == kTeamCacheOwners) {
            Env e = bare_env(sm, &shared_layout, &t, &state, env, lane, vstride);
            if (op == kTeamNarrowphase) narrowphase_range(e, k_begin, member, shared_layout.team);
            else if (op == kTeamWarmStart) warm_start_range(e, k_begin, member, shared_layout.team);
            else cache_owners_range(e, k_begin, member, shared_layout.team);
            r.status = e.status;
        }
        __syncwarp();
        if (lane == 0u) {
            float* out = team_result(sm, shared_layout, member);
            out[0] = r.momentum; out[1] = r.residual; answer[2] = r.status;
            __threadfence_block();
            team_poke(answer + 3, seq);
        }
        __syncwarp();
    }
}

// Block layout: blockDim.x / 32 warps, `team` consecutive warps per env (one unless the world runs in team mode); an
// env's shared-memory slice is shared by its team.
template <int NR, bool kRigid, bool kSlim, bool kControl>
__global__ void __maxnreg__(kRigid ? NKB_MAXNREG_RIGID : (kSlim ? NKB_MAXNREG_SLIM : NKB_MAXNREG)) step_kernel(const __grid_constant__ StepParams p) {
    extern __shared__ __align__(16) float smem[];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t team = kRigid ? p.sm.team : 1u;
    const uint32_t slot = warp / team, member = warp - slot * team;
    uint32_t env = blockIdx.x * ((blockDim.x >> 5) / team) + slot;
    float* sm = smem + (size_t)slot * p.sm.words;
    if constexpr (kRigid) {
        // team mode: every lead zeroes its team's sequence numbers before any helper looks (the one block-wide barrier of
        // the kernel, passed by every thread before any leaves)
        if (team > 1u) {
            if (member == 0u) team_open(sm, p.sm, lane);
            __syncthreads();
        }
    }
    if (p.sel_ids != nullptr) env = env < p.sel_count ? p.sel_ids[env] : 0xffffffffu;
    if (env >= p.s.env_count) return;                       // the whole team leaves together
    if (p.sel_mask != nullptr && p.sel_mask[env] == 0u) return;
    if constexpr (kRigid) {
        if (member != 0u) { team_helper<kRigid>(sm, p.sm, p.t, p.s, env, member, lane, 32u * NR); return; }
    }
    advance_env<NR, kRigid, kControl>(p, sm, env, lane);
    if constexpr (kRigid) { if ((p.sm.team_drill & 1u) == 0u) team_dismiss(sm, p.sm, lane); }
}

// Raises the kernel's dynamic shared-memory limit to `bytes` if it is not there yet.  The limit is per function and
// per device and only ever grows, so worlds of different sizes stepped from different threads cannot undo each other's
// setting between the attribute call and the launch.
template <int NR, bool kRigid, bool kSlim, bool kControl>
static cudaError_t variant_reserve_shared(size_t bytes) {
    static std::mutex lock;
    static size_t reserved[64] = {0};
    if (bytes <= 48u * 1024u) return cudaSuccess;
    int device = 0;
    cudaError_t err = cudaGetDevice(&device);
    if (err != cudaSuccess) return err;
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> hold(lock);
    if (bytes <= reserved[device]) return cudaSuccess;
    err = cudaFuncSetAttribute(step_kernel<NR, kRigid, kSlim, kControl>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (err == cudaSuccess) reserved[device] = bytes;
    return err;
}

template <int NR, bool kRigid, bool kSlim, bool kControl>
static int variant_resident_blocks(uint32_t warps_per_block, size_t shared_bytes) {
    if (variant_reserve_shared<NR, kRigid, kSlim, kControl>(shared_bytes) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    int blocks = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, step_kernel<NR, kRigid, kSlim, kControl>, (int)(warps_per_block * 32u), shared_bytes) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return blocks;
}

template <int NR, bool kRigid, bool kSlim, bool kControl>
static int variant_registers() {
    cudaFuncAttributes attr{};
    if (cudaFuncGetAttributes(&attr, step_kernel<NR, kRigid, kSlim, kControl>) != cudaSuccess) { cudaGetLastError(); return 0; }
    return attr.numRegs;
}

template <int NR, bool kRigid, bool kSlim, bool kControl>
static cudaError_t variant_launch(const StepParams& p, uint32_t warps_per_block, cudaStream_t stream) {
    const uint32_t team = kRigid ? p.sm.team : 1u;
    const uint32_t envs_per_block = warps_per_block / team;
    if (envs_per_block == 0u || envs_per_block * team != warps_per_block || envs_per_block > 15u) return cudaErrorInvalidConfiguration;
    const size_t bytes = (size_t)envs_per_block * p.sm.words * sizeof(float);
    const cudaError_t err = variant_reserve_shared<NR, kRigid, kSlim, kControl>(bytes);
    if (err != cudaSuccess) return err;
    const uint32_t envs = p.sel_ids != nullptr ? p.sel_count : p.s.env_count;
    if (envs == 0u) return cudaSuccess;
    const uint32_t blocks = (envs + envs_per_block - 1u) / envs_per_block;
    step_kernel<NR, kRigid, kSlim, kControl><<<blocks, warps_per_block * 32u, bytes, stream>>>(p);
    return cudaGetLastError();
}

#define NKB_STEP_VARIANT(name, NR, RIGID, SLIM, CONTROL) \
    extern const StepVariant name = {variant_resident_blocks<NR, RIGID, SLIM, CONTROL>, variant_registers<NR, RIGID, SLIM, CONTROL>, variant_launch<NR, RIGID, SLIM, CONTROL>};

}  // namespace nkb

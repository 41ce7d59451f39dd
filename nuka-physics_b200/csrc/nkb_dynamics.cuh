// Warp-per-env articulation stages: forward kinematics, implicit PD drives, joint-space dynamics
// (bias forces + composite-inertia mass matrix + L D L^T solve), position integration and link velocities.
// One lane owns one link in the tree sweeps and one coordinate in the mass-matrix work; per-env intermediates
// live in the warp's shared-memory slice.  The computed quantities are those of the reference's
// ops/articulation.cu:505-645 (ArticulationDynamicsKernel), :836-940 (ApplyAffineDriveKernel), :732-791
// (position integration), :647-689 (link velocities), :1561-1596 (world poses) and
// ops/articulation_mass.cuh:124-396 (mass matrix, factor, solve).
#pragma once
#include "nkb_math.cuh"
#include "nkb_types.h"

namespace nkb {

// Per-warp view of one env: template, state, shared-memory slice and this lane's registers.
struct Env {
    const TemplateView* t;
    const StateView* s;
    const SmemLayout* lay;
    float* sm;
    uint32_t env, lane;
    // lane = link
    uint32_t parent, jtype, depth, link_dof;
    float q, qd, qdd, tau;
    V3 axis;                 // unit joint axis in the link frame
    float drive_command, drive_dissipation, drive_lower, drive_upper;
    // lane = dof: a lane owns coordinates lane and lane + 32 (the second only when the articulation has more than 32)
    uint32_t dof_link[2], dof_comp[2];   // comp == kNoLink for scalar joints
    float vel0[2];           // step-start coordinate velocity
    uint32_t status;
    uint32_t vstride;        // words per shared-memory vector: 32 x coordinates per lane
    // team mode: word offsets from the env's Newton scratch (matrix, block mass, staged rows) and solver vectors to this
    // warp's private copies; zero for the env's lead warp
    uint32_t newton_shift, vec_shift;
#ifdef NKB_STAGE_TAPS
    uint32_t* cyc;           // stage cycle counters of this env, or null
    long long t0;
#endif
};

// Stage cycle counters are a build-time instrument (-DNKB_STAGE_TAPS); the shipped kernel carries none of it.
#ifdef NKB_STAGE_TAPS
// Adds the cycles since the last tick to stage counter k.
NKB_DEV void tick(Env& e, int k) {
    if (e.cyc == nullptr) return;
    const long long now = clock64();
    if (e.lane == 0u) e.cyc[k] += (uint32_t)(now - e.t0);
    e.t0 = now;
}
NKB_DEV void tick_count(Env& e, int k) { if (e.cyc != nullptr && e.lane == 0u) e.cyc[k] += 1u; }
#else
NKB_DEV void tick(Env&, int) {}
NKB_DEV void tick_count(Env&, int) {}
#endif

NKB_DEV float* sm_pose(const Env& e, uint32_t l) { return e.sm + e.lay->pose + 7u * l; }
NKB_DEV float* sm_xrot(const Env& e, uint32_t l) { return e.sm + e.lay->xrot + 9u * l; }
NKB_DEV float* sm_xtr(const Env& e, uint32_t l) { return e.sm + e.lay->xtr + 3u * l; }
NKB_DEV float* sm_vel(const Env& e, uint32_t l) { return e.sm + e.lay->vel + 6u * l; }
NKB_DEV float* sm_acc(const Env& e, uint32_t l) { return e.sm + e.lay->acc + 6u * l; }
NKB_DEV float* sm_pbias(const Env& e, uint32_t l) { return e.sm + e.lay->pbias + 6u * l; }
NKB_DEV float* sm_ic(const Env& e, uint32_t l) { return e.sm + e.lay->ic + 10u * l; }
NKB_DEV float* sm_mass(const Env& e) { return e.sm + e.lay->mass; }
NKB_DEV float* sm_factor(const Env& e) { return e.sm + e.lay->factor; }
NKB_DEV float* sm_vec(const Env& e, uint32_t k) { return e.sm + e.lay->vecs + e.vec_shift + e.vstride * k; }   // 32 or 64 words per vector
// value of coordinate j from per-lane registers x[r] (coordinate lane + 32 r)
template <int NR>
NKB_DEV float coord_bcast(const float (&x)[NR], uint32_t j) {
    if (NR == 1) return __shfl_sync(NKB_FULL, x[0], j);
    return __shfl_sync(NKB_FULL, j < 32u ? x[0] : x[NR - 1], j & 31u);
}
// vector slots
enum { kVecAcc = 0, kVecFree = 1, kVecU = 2, kVecPseudo = 3, kVecTmp = 4, kVecTmp2 = 5,
       // Newton-loop scratch shares slots whose other users run before or after the solve
       kVecS0 = kVecTmp, kVecS1 = kVecTmp2, kVecS2 = kVecAcc,
       // the Newton direction is staged after the last read of S0 in an iteration and consumed before the next write
       kVecD = kVecS0, kVecCount = 6 };

NKB_DEV uint32_t joint_dofs(uint32_t t) { return (t == kRevolute || t == kPrismatic) ? 1u : t == kFloating ? 6u : t == kSpherical ? 3u : 0u; }

template <int NR>
NKB_DEV void env_begin(Env& e, const StepParams& p, float* sm, uint32_t env, uint32_t lane) {
    e.t = &p.t; e.s = &p.s; e.lay = &p.sm; e.sm = sm; e.env = env; e.lane = lane;
    const TemplateView& t = p.t;
    const bool link = lane < t.L;
    e.parent = link ? __ldg(t.parent + lane) : kNoLink;
    e.jtype = link ? __ldg(t.jtype + lane) : (uint32_t)kFixed;
    e.depth = link ? __ldg(t.depth + lane) : 0xffffu;
    e.link_dof = link ? __ldg(t.link_dof + lane) : 0u;
    e.axis = mk3(0.f, 0.f, 0.f);
    if (link) {
        V3 a = ld3(t.axis + 3u * lane);
        const float ls = dot(a, a);
        e.axis = ls > 1.0e-12f ? a * rsqrtf(ls) : mk3(0.f, 0.f, 0.f);
    }
    const size_t at = (size_t)env * t.L + lane;
    e.q = link ? p.s.q[at] : 0.f;
    e.qd = link ? p.s.qdot[at] : 0.f;
    e.qdd = 0.f; e.tau = 0.f;
    e.drive_command = e.drive_dissipation = e.drive_lower = e.drive_upper = 0.f;
    e.vstride = 32u * NR; e.newton_shift = 0u; e.vec_shift = 0u;
    e.dof_link[1] = 0u; e.dof_comp[1] = kNoLink; e.vel0[1] = 0.f;
#pragma unroll
    for (uint32_t r = 0u; r < (uint32_t)NR; ++r) {
        const uint32_t c = lane + 32u * r;
        const bool dof = c < t.ndof;
        e.dof_link[r] = dof ? __ldg(t.dof_link + c) : 0u;
        e.dof_comp[r] = kNoLink;
        if (dof && __ldg(t.jtype + e.dof_link[r]) == kFloating) e.dof_comp[r] = c - __ldg(t.link_dof + e.dof_link[r]);
        e.vel0[r] = 0.f;
    }
    e.status = 0u;
#ifdef NKB_STAGE_TAPS
    e.cyc = p.s.dbg_cycles != nullptr ? p.s.dbg_cycles + (size_t)env * 32u : nullptr;
    e.t0 = clock64();
#endif
}

// World poses of every link, ops/articulation.cu:1561-1596 with kinematics.cuh:25-42 joint frames.
NKB_DEV void stage_fk(Env& e) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane;
    const bool link = l < t.L;
    V3 rpos = mk3(0.f, 0.f, 0.f);
    Q4 rrot = mkq(1.f, 0.f, 0.f, 0.f);
    if (link) {
        rpos = ld3(t.offset + 3u * l);
        rrot = ldq(t.local_quat + 4u * l);
        if (e.jtype == kRevolute) {
            float s, c;
            sincos_joint(0.5f * e.q, s, c);
            rrot = qnorm_le(qmul(rrot, mkq(c, e.axis.x * s, e.axis.y * s, e.axis.z * s)), 1.0e-12f);
        } else if (e.jtype == kPrismatic) {
            rpos = rpos + qrot(rrot, e.axis * e.q);
        }
    }
    for (uint32_t d = 0; d <= t.max_depth; ++d) {
        if (link && e.depth == d) {
            float* out = sm_pose(e, l);
            if (e.parent == kNoLink) {
                if (e.jtype == kFloating) {
                    const float* bp = e.s->base_pose + (size_t)e.env * 7u;
#pragma unroll
                    for (int k = 0; k < 7; ++k) out[k] = bp[k];
                } else { st3(out, rpos); stq(out + 3, rrot); }
            } else {
                const float* pp = sm_pose(e, e.parent);
                const Q4 pq = ldq(pp + 3);
                st3(out, ld3(pp) + qrot(pq, rpos));
                stq(out + 3, qnorm_le(qmul(pq, rrot), 1.0e-12f));
            }
        }
        __syncwarp();
    }
}

// Joint transform (E, r) of this lane's link, ops/articulation.cu:259-277.
NKB_DEV void joint_xform(const Env& e, float* E, V3& r) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane;
    if (e.parent == kNoLink && e.jtype == kFloating) {
        const M3 I = m3_ident();
#pragma unroll
        for (int k = 0; k < 9; ++k) E[k] = I.m[k];
        r = mk3(0.f, 0.f, 0.f);
        return;
    }
    M3 jr = m3_ident();
    r = ld3(t.offset + 3u * l);
    const Q4 lq = ldq(t.local_quat + 4u * l);
    if (e.jtype == kRevolute) jr = m3_axis_angle(ld3(t.axis + 3u * l), e.q);
    else if (e.jtype == kPrismatic) r = r + qrot(lq, e.axis * e.q);
    const M3 rot = m3_mul(m3_from_quat(lq), jr);
#pragma unroll
    for (int a = 0; a < 3; ++a)
#pragma unroll
        for (int b = 0; b < 3; ++b) E[a * 3 + b] = rot.m[b * 3 + a];
}

// Affine joint drives, ops/articulation.cu:836-940: implicit PD position (mode 0), direct torque (1), velocity (2),
// actuator (5: torque command inside a signed torque-speed envelope).
NKB_DEV void stage_drives(Env& e) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane;
    e.drive_command = e.drive_dissipation = e.drive_lower = e.drive_upper = 0.f;
    e.tau = 0.f;
    if (l >= t.L || joint_dofs(e.jtype) != 1u) return;
    const size_t at = (size_t)e.env * t.L + l;
    const float target = e.s->drive_target[at], kp = e.s->kp[at], kd = e.s->kd[at], vt = e.s->vel_target[at];
    const float limit = e.s->force_limit[at], ff = e.s->feedforward[at];
    const uint32_t mode = t.cfg.control_mode;
    const bool inverse_dynamics = mode == 3u || mode == 4u;          // computed torque, operational space: the command comes from stage_computed_torque
    const bool position_control = mode == 0u || inverse_dynamics, velocity_control = mode == 2u;
    if ((position_control && (!isfinite(target) || !isfinite(kp) || kp < 0.f || !isfinite(kd) || kd < 0.f)) ||
        ((position_control || velocity_control) && !isfinite(vt)) || (velocity_control && (!isfinite(kp) || kp < 0.f)) ||
        (mode == 3u && !isfinite(e.s->acc_target[at]))) {
        e.status |= kStatusControlFailure; return;
    }
    const float noload = mode == 5u ? e.s->noload_speed[at] : 0.f;
    if (!isfinite(noload)) { e.status |= kStatusControlFailure; return; }
    float lower = limit > 0.f ? -limit : -FLT_MAX, upper = limit > 0.f ? limit : FLT_MAX;
    float damping = 0.f, bias = target;                       // torque mode: the target field carries the commanded effort
    if (inverse_dynamics) bias = 0.f;
    else if (position_control) { damping = kd + t.cfg.dt * kp; bias = kp * (target - e.q) + damping * vt; }
    else if (velocity_control) { damping = kp; bias = damping * vt; }
    else if (mode == 5u && limit > 0.f && noload > 0.f) {
        const float speed_bias = limit * e.qd / noload;
        lower = fminf(fmaxf(-limit - speed_bias, -limit), limit);
        upper = fminf(fmaxf(limit - speed_bias, -limit), limit);
    }
    const float effort = bias - damping * e.qd;
    if (effort < lower || effort > upper) { bias = effort; damping = 0.f; }
    else { lower += damping * e.qd; upper += damping * e.qd; }
    if (!isfinite(bias) || !isfinite(damping) || damping < 0.f || !isfinite(limit) || !isfinite(ff) || !isfinite(e.qd) || !isfinite(e.q)) {
        e.status |= kStatusControlFailure; return;
    }
    if (inverse_dynamics) { lower = limit > 0.f ? -limit : -FLT_MAX; upper = limit > 0.f ? limit : FLT_MAX; }
    e.drive_command = bias; e.drive_dissipation = damping; e.drive_lower = lower; e.drive_upper = upper;
    e.tau = inverse_dynamics ? 0.f : ff;
}

// Bias forces, mass matrix, factor and unconstrained acceleration; optionally the semi-implicit velocity
// update.  Leaves M and its L D L^T factor in shared memory for the constraint solve.
template <int NR>
NKB_DEV void stage_dynamics(Env& e, bool integrate_velocity) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane, L = t.L, n = t.ndof, ld = e.lay->ld;
    const bool link = l < L;
    const bool froot = link && e.parent == kNoLink && e.jtype == kFloating;
    const V3 g = mk3(t.cfg.gravity[0], t.cfg.gravity[1], t.cfg.gravity[2]);
    const float dt = t.cfg.dt;
    float E[9]; V3 r = mk3(0.f, 0.f, 0.f);
    if (link) {
        joint_xform(e, E, r);
        float* xe = sm_xrot(e, l);
#pragma unroll
        for (int k = 0; k < 9; ++k) xe[k] = E[k];
        st3(sm_xtr(e, l), r);
    }
    // joint velocity S qd in the link frame
    V3 jw = mk3(0.f, 0.f, 0.f), jv = mk3(0.f, 0.f, 0.f);
    if (e.jtype == kRevolute) jw = e.axis * e.qd; else if (e.jtype == kPrismatic) jv = e.axis * e.qd;
    V3 vw = mk3(0.f, 0.f, 0.f), vv = mk3(0.f, 0.f, 0.f), cw = vw, cv = vv;
    if (froot) {
        const float* lv = e.s->link_vel + ((size_t)e.env * L + l) * 6u;
        vw = ld3(lv); vv = ld3(lv + 3);
        st3(sm_vel(e, l), vw); st3(sm_vel(e, l) + 3, vv);
    }
    __syncwarp();
    for (uint32_t d = 0; d <= t.max_depth; ++d) {
        if (link && e.depth == d && !froot) {
            V3 pw = mk3(0.f, 0.f, 0.f), pv = pw;
            if (e.parent != kNoLink) { pw = ld3(sm_vel(e, e.parent)); pv = ld3(sm_vel(e, e.parent) + 3); }
            V3 tw, tv;
            xf_motion(E, r, pw, pv, tw, tv);
            vw = tw + jw; vv = tv + jv;
            st3(sm_vel(e, l), vw); st3(sm_vel(e, l) + 3, vv);
            motion_cross(vw, vv, jw, jv, cw, cv);
        }
        __syncwarp();
    }
    // p = v x* (I v)
    const float* I10 = t.inertia10 + 10u * (link ? l : 0u);
    V3 pn = mk3(0.f, 0.f, 0.f), pf = pn;
    if (link) {
        V3 in_, if_;
        rbi_mulv(I10, vw, vv, in_, if_);
        force_cross(vw, vv, in_, if_, pn, pf);
    }
    // accelerations root to leaf with gravity injected at the root
    V3 aw = mk3(0.f, 0.f, 0.f), av = aw;
    for (uint32_t d = 0; d <= t.max_depth; ++d) {
        if (link && e.depth == d) {
            if (e.parent != kNoLink) xf_motion(E, r, ld3(sm_acc(e, e.parent)), ld3(sm_acc(e, e.parent) + 3), aw, av);
            else if (e.jtype == kFloating) {
                const V3 gl = qrot_inv(ldq(e.s->base_pose + (size_t)e.env * 7u + 3), g);
                aw = mk3(0.f, 0.f, 0.f); av = -gl;
            } else xf_motion(E, r, mk3(0.f, 0.f, 0.f), -g, aw, av);
            aw = aw + cw; av = av + cv;
            st3(sm_acc(e, l), aw); st3(sm_acc(e, l) + 3, av);
        }
        __syncwarp();
    }
    if (link) {
        V3 in_, if_;
        rbi_mulv(I10, aw, av, in_, if_);
        pn = pn + in_; pf = pf + if_;
        st3(sm_pbias(e, l), pn); st3(sm_pbias(e, l) + 3, pf);
        float* ic = sm_ic(e, l);
#pragma unroll
        for (int k = 0; k < 10; ++k) ic[k] = __ldg(I10 + k);
    }
    __syncwarp();
    // leaf to root: bias forces and composite inertias, children in list order
    for (uint32_t rem = t.max_depth + 1u; rem > 0u; --rem) {
        if (link && e.depth == rem - 1u) {
            const uint32_t cb = __ldg(t.child_begin + l), ce = __ldg(t.child_begin + l + 1u);
            float* ic = sm_ic(e, l);
            for (uint32_t c = cb; c < ce; ++c) {
                const uint32_t child = __ldg(t.children + c);
                V3 cn, cf;
                xf_force_t(sm_xrot(e, child), ld3(sm_xtr(e, child)), ld3(sm_pbias(e, child)), ld3(sm_pbias(e, child) + 3), cn, cf);
                pn = pn + cn; pf = pf + cf;
                float add[10];
                rbi_to_parent(sm_xrot(e, child), ld3(sm_xtr(e, child)), sm_ic(e, child), add);
#pragma unroll
                for (int k = 0; k < 10; ++k) ic[k] += add[k];
            }
            st3(sm_pbias(e, l), pn); st3(sm_pbias(e, l) + 3, pf);
        }
        __syncwarp();
    }
    // generalized bias and right-hand side, lane = coordinate
    float rhs[NR];
    bool dof[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const uint32_t c = l + 32u * r;
        const float diss_of_link = __shfl_sync(NKB_FULL, e.drive_dissipation, e.dof_link[r]);
        const float tau_of_link = __shfl_sync(NKB_FULL, e.tau, e.dof_link[r]);
        const float qd_of_link = __shfl_sync(NKB_FULL, e.qd, e.dof_link[r]);
        const float q_of_link = __shfl_sync(NKB_FULL, e.q, e.dof_link[r]);
        rhs[r] = 0.f;
        dof[r] = c < n;
        if (dof[r]) {
            const uint32_t dl = e.dof_link[r];
            const float* pb = sm_pbias(e, dl);
            float bias;
            if (e.dof_comp[r] == kNoLink) {
                V3 a = ld3(t.axis + 3u * dl);
                const float ls = dot(a, a);
                if (ls > 1.0e-12f) a = a * rsqrtf(ls);
                const uint32_t jt = __ldg(t.jtype + dl);
                bias = jt == kRevolute ? dot(a, ld3(pb)) : dot(a, ld3(pb + 3));
                e.vel0[r] = qd_of_link;
                const float damping = __ldg(t.damping + dl) + diss_of_link;
                const float spring = __ldg(t.stiffness + dl) * (q_of_link - __ldg(t.spring_ref + dl));
                rhs[r] = tau_of_link - bias - damping * e.vel0[r] - spring;
            } else {
                bias = pb[e.dof_comp[r]];
                e.vel0[r] = sm_vel(e, dl)[e.dof_comp[r]];
                rhs[r] = -bias;
            }
        }
    }
    // mass matrix, ops/articulation_mass.cuh:124-253
    float* M = sm_mass(e);
    for (uint32_t k = l; k < n * ld; k += 32u) M[k] = 0.f;
    __syncwarp();
    if (t.floating_root && l < 6u) {
        const float* ic = sm_ic(e, 0u);
        const float m = ic[0]; const V3 h = ld3(ic + 1);
        const float Ib[9] = {ic[4], ic[7], ic[8], ic[7], ic[5], ic[9], ic[8], ic[9], ic[6]};
        const float hx[9] = {0.f, -h.z, h.y, h.z, 0.f, -h.x, -h.y, h.x, 0.f};
        float* row = M + l * ld;
        if (l < 3u) {
#pragma unroll
            for (int c = 0; c < 3; ++c) { row[c] = Ib[l * 3 + c]; row[3 + c] = hx[l * 3 + c]; }
        } else {
#pragma unroll
            for (int c = 0; c < 3; ++c) { row[c] = -hx[(l - 3) * 3 + c]; row[3 + c] = (int)(l - 3) == c ? m : 0.f; }
        }
    }
    if (link && !froot && joint_dofs(e.jtype) == 1u) {
        const uint32_t di = e.link_dof;
        const float* ic = sm_ic(e, l);
        V3 fn, ff;
        if (e.jtype == kRevolute) rbi_mulv(ic, e.axis, mk3(0.f, 0.f, 0.f), fn, ff); else rbi_mulv(ic, mk3(0.f, 0.f, 0.f), e.axis, fn, ff);
        float diag = e.jtype == kRevolute ? dot(e.axis, fn) : dot(e.axis, ff);
        diag += __ldg(t.armature + l);
        diag += dt * e.drive_dissipation;
        M[di * ld + di] = diag;
        uint32_t walk = l;
        for (;;) {
            const uint32_t p = __ldg(t.parent + walk);
            if (p == kNoLink) break;
            V3 pn2, pf2;
            xf_force_t(sm_xrot(e, walk), ld3(sm_xtr(e, walk)), fn, ff, pn2, pf2);
            fn = pn2; ff = pf2;
            walk = p;
            const uint32_t wt = __ldg(t.jtype + walk);
            if (joint_dofs(wt) == 0u) continue;
            const uint32_t dj = __ldg(t.link_dof + walk);
            if (wt == kFloating) {
                const float f6[6] = {fn.x, fn.y, fn.z, ff.x, ff.y, ff.z};
#pragma unroll
                for (int b = 0; b < 6; ++b) { M[di * ld + b] = f6[b]; M[b * ld + di] = f6[b]; }
                continue;
            }
            V3 a = ld3(t.axis + 3u * walk);
            const float ls = dot(a, a);
            if (ls > 1.0e-12f) a = a * rsqrtf(ls);
            const float entry = wt == kRevolute ? dot(a, fn) : dot(a, ff);
            M[di * ld + dj] = entry; M[dj * ld + di] = entry;
        }
    }
    __syncwarp();
    if (e.s->dbg_mass != nullptr) {
        float* out = e.s->dbg_mass + (size_t)e.env * n * n;
        for (uint32_t k = l; k < n * n; k += 32u) out[k] = M[(k / n) * ld + k % n];
    }
    // L D L^T, unit lower triangle with D on the diagonal and pivot floor 1e-6 (articulation_mass.cuh:269-335).
    // Column by column, lane = row: entry (row, k) = (M[row][k] - sum_{j<k} L[row][j] L[k][j] d_j) / d_k, the terms
    // subtracted in ascending j exactly as the reference's in-place elimination subtracts them, but with both rows
    // and the pivots read ahead of one short dependent chain instead of a read-modify-write per term.
    float* F = sm_factor(e);
    float* piv = sm_vec(e, kVecTmp);
    for (uint32_t k = l; k < n * ld; k += 32u) F[k] = M[k];
    __syncwarp();
#pragma unroll 1
    for (uint32_t k = 0; k < n; ++k) {
        const float* Fk = F + k * ld;
        float v[NR];
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint32_t row = l + 32u * r;
            v[r] = 0.f;
            if (row >= k && row < n) {
                const float* Fr = F + row * ld;
                const float4* Fr4 = reinterpret_cast<const float4*>(Fr);
                const float4* Fk4 = reinterpret_cast<const float4*>(Fk);
                const float4* piv4 = reinterpret_cast<const float4*>(piv);
                float acc = Fr[k];
                const uint32_t full = k >> 2;
#pragma unroll 1
                for (uint32_t c = 0u; c < full; ++c) {
                    const float4 a = Fr4[c], b4 = Fk4[c], p = piv4[c];
                    acc -= a.x * b4.x * p.x; acc -= a.y * b4.y * p.y; acc -= a.z * b4.z * p.z; acc -= a.w * b4.w * p.w;
                }
                for (uint32_t j = full << 2; j < k; ++j) acc -= Fr[j] * Fk[j] * piv[j];
                v[r] = acc;
            }
        }
        const float dk = fmaxf(coord_bcast<NR>(v, k), 1.0e-6f);
        __syncwarp();
#pragma unroll
        for (int r = 0; r < NR; ++r) {
            const uint32_t row = l + 32u * r;
            if (row == k) { F[row * ld + k] = dk; piv[k] = dk; }
            else if (row > k && row < n) F[row * ld + k] = v[r] / dk;
        }
        __syncwarp();
    }
    // the strict upper triangle keeps M's entries; only the lower triangle and the diagonal are read below
    // solve L D L^T x = rhs, lane = coordinate (articulation_mass.cuh:357-396)
    float x[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) x[r] = dof[r] ? rhs[r] : 0.f;
    for (uint32_t j = 0; j < n; ++j) {
        const float xj = coord_bcast<NR>(x, j);
#pragma unroll
        for (int r = 0; r < NR; ++r) { const uint32_t row = l + 32u * r; if (row > j && row < n) x[r] -= F[row * ld + j] * xj; }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) { const uint32_t row = l + 32u * r; if (dof[r]) x[r] /= F[row * ld + row]; }
    for (uint32_t jj = n; jj > 0u; --jj) {
        const uint32_t j = jj - 1u;
        const float xj = coord_bcast<NR>(x, j);
#pragma unroll
        for (int r = 0; r < NR; ++r) { const uint32_t row = l + 32u * r; if (row < j) x[r] -= F[j * ld + row] * xj; }
    }
#pragma unroll
    for (int r = 0; r < NR; ++r) if (dof[r]) sm_vec(e, kVecAcc)[l + 32u * r] = x[r];
    __syncwarp();
    // accelerations back to links, velocity update (articulation.cu:597-615)
    const float acc_of_mine = link && joint_dofs(e.jtype) == 1u ? sm_vec(e, kVecAcc)[e.link_dof] : 0.f;
    e.qdd = acc_of_mine;
    if (integrate_velocity) {
        if (link && joint_dofs(e.jtype) == 1u) e.qd = e.qd + dt * acc_of_mine;
        // the floating base's six coordinates come first, so they sit in register slot 0
        const bool base_coord = dof[0] && e.dof_comp[0] != kNoLink;
        float nv = 0.f;
        if (base_coord) {
            const uint32_t c = e.dof_comp[0], i = c % 3u, j = (i + 1u) % 3u, k = (i + 2u) % 3u;
            const float* rv = sm_vel(e, e.dof_link[0]);
            const float transport = c < 3u ? 0.f : rv[j] * rv[3u + k] - rv[k] * rv[3u + j];
            nv = e.vel0[0] + dt * (x[0] + transport);
        }
        __syncwarp();
        if (base_coord) sm_vel(e, e.dof_link[0])[e.dof_comp[0]] = nv;
        __syncwarp();
    }
}

// Computed-torque control (control mode 3), the quantities of the reference's ApplyDynamicsDriveKernel
// (ops/articulation.cu:1315-1418).  Runs between a force-free dynamics pass (which leaves M's factor in shared memory and
// the free accelerations in the lanes) and the step's dynamics pass.  With S the selector of the scalar joints,
// H = (S M^-1 S^T)^-1 is the inertia the actuators see, a floating base's reaction included; the command is
// H (a* + kp (q* - q) + kd (qd* - qd)) - H qdd_free - d qd (bias compensation without the passive joint damping).
// Lane c owns column c of each small matrix and runs the reference's serial column loops (same operation order, double
// accumulators where the reference has them); the matrices live in regions that are idle between the two dynamics passes:
// the Newton matrix holds S M^-1 S^T and its factors, the head records' region holds H, the solver vectors the small
// tables.
// Out of line, with its inputs by value: the controller runs in one control mode only and must not weigh on the register
// allocation of the step kernel's common path.
struct TorqueIn {
    float* sm; const SmemLayout* lay; const TemplateView* t; const StateView* s;
    uint32_t env, lane, jtype, link_dof, mode;
    float q, qd, qdd, lower, upper;
};
struct TorqueOut { float tau, command; uint32_t status; uint32_t applied; };

// Pseudoinverse of the symmetric n x n task metric (n = 3 or 6, row stride 6, in shared memory) by cyclic Jacobi rotations
// in the reference's pair order and with its rotation formulas (ops/articulation.cu:1234-1288); directions whose
// eigenvalue is within 8 eps of the largest are dropped.  The whole warp takes part: every lane follows the pivots, lane
// k < n carries row k of the matrix and of the eigenvector table through each rotation, lane 0 closes the 2 x 2 block,
// and the n x n entries of the result are spread over the lanes.  `vectors` is 36 words of scratch beside the matrix.
static __device__ __noinline__ void task_metric_pseudoinverse(float* a, float* vectors, uint32_t n, float* inverse, uint32_t lane) {
    for (uint32_t i = lane; i < 36u; i += 32u) vectors[i] = (i / 6u == i % 6u && i / 6u < n) ? 1.0f : 0.f;
    __syncwarp();
    for (uint32_t sweep = 0u; sweep < 24u; ++sweep) {
        bool changed = false;
        for (uint32_t p = 0u; p < n; ++p) for (uint32_t q = p + 1u; q < n; ++q) {
            const float app = a[p * 6u + p], aqq = a[q * 6u + q], apq = a[p * 6u + q];
            if (fabsf(apq) <= FLT_EPSILON * (fabsf(app) + fabsf(aqq))) continue;       // the same words in every lane: a uniform branch
            changed = true;
            const double theta = ((double)aqq - app) / (2.0 * apq);
            const float tangent = (float)(copysign(1.0, theta) / (fabs(theta) + sqrt(1.0 + theta * theta)));
            const float cosine = rsqrtf(1.0f + tangent * tangent), sine = tangent * cosine;
            __syncwarp();
            if (lane < n) {
                const uint32_t k = lane;
                if (k != p && k != q) {
                    const float kp = a[k * 6u + p], kq = a[k * 6u + q];
                    const float turned_p = cosine * kp - sine * kq, turned_q = sine * kp + cosine * kq;
                    a[k * 6u + p] = turned_p; a[p * 6u + k] = turned_p; a[k * 6u + q] = turned_q; a[q * 6u + k] = turned_q;
                }
                const float vp = vectors[k * 6u + p], vq = vectors[k * 6u + q];
                vectors[k * 6u + p] = cosine * vp - sine * vq;
                vectors[k * 6u + q] = sine * vp + cosine * vq;
            }
            if (lane == 0u) {
                a[p * 6u + p] = app - tangent * apq;
                a[q * 6u + q] = aqq + tangent * apq;
                a[p * 6u + q] = 0.f; a[q * 6u + p] = 0.f;
            }
            __syncwarp();
        }
        if (!changed) break;
    }
    float largest = 0.f;
    for (uint32_t i = 0u; i < n; ++i) largest = fmaxf(largest, a[i * 6u + i]);
    const float tolerance = largest * (8.0f * FLT_EPSILON);
    for (uint32_t i = lane; i < n * n; i += 32u) {
        const uint32_t r = i / n, c = i % n;
        double v = 0.0;
        for (uint32_t k = 0u; k < n; ++k) {
            const float eigenvalue = a[k * 6u + k];
            if (eigenvalue > tolerance) v += (double)vectors[r * 6u + k] * vectors[c * 6u + k] / eigenvalue;
        }
        inverse[r * 6u + c] = (float)v;
    }
    __syncwarp();
}

// The task frame's velocity and acceleration in the world from the task link's twist and force-free acceleration (link
// frame, angular first) plus J q'', the pose error, and from them kp x_err - kd v - a (ops/articulation.cu:1490-1513).
static __device__ __noinline__ void task_right_hand_side(TorqueIn e, const float* acc0, const float* J, const float* qdd, float* trhs, uint32_t rows,
                                                         V3 task_pos, Q4 task_q, Q4 link_q, V3 offset, Q4 desired) {
    const TemplateView& t = *e.t;
    const uint32_t n = t.ndof, L = t.L, tl = t.cfg.task_link;
    const float* vel = e.sm + e.lay->vel + 6u * tl;
    const V3 omega = ld3(vel), linear = ld3(vel + 3);
    const V3 alpha = mk3(acc0[0], acc0[1], acc0[2]), linear_accel = mk3(acc0[3], acc0[4], acc0[5]);
    const V3 g = mk3(t.cfg.gravity[0], t.cfg.gravity[1], t.cfg.gravity[2]);
    const V3 task_velocity = qrot(link_q, linear + cross(omega, offset));
    const V3 task_angular = qrot(link_q, omega);
    V3 task_accel = qrot(link_q, (linear_accel + cross(omega, linear)) + (cross(alpha, offset) + cross(omega, cross(omega, offset)))) + g;
    V3 task_angular_accel = qrot(link_q, alpha);
    float jq[6];
    for (uint32_t r = 0u; r < 6u; ++r) {
        float sum = 0.f;
        for (uint32_t i = 0u; i < n; ++i) sum += J[r * n + i] * qdd[i];
        jq[r] = sum;
    }
    task_accel = task_accel + mk3(jq[0], jq[1], jq[2]);
    task_angular_accel = task_angular_accel + mk3(jq[3], jq[4], jq[5]);
    const V3 position_error = ld3(e.s->task_target + (size_t)e.env * 3u) - task_pos;
    V3 orientation_error = mk3(0.f, 0.f, 0.f);
    if (rows == 6u) {
        const Q4 current = qnorm_le(task_q, 1.0e-12f), wanted = qnorm_le(desired, 1.0e-12f);
        const Q4 err = qmul(wanted, mkq(current.w, -current.x, -current.y, -current.z));
        const float sign = err.w < 0.f ? -1.0f : 1.0f;
        const float length = sqrtf(err.x * err.x + err.y * err.y + err.z * err.z);
        const float scale = length > 1.0e-7f ? sign * 2.0f * atan2f(length, fabsf(err.w)) / length : sign * 2.0f;
        orientation_error = mk3(err.x * scale, err.y * scale, err.z * scale);
    }
    const float kp = e.s->kp[(size_t)e.env * L + tl], kd = e.s->kd[(size_t)e.env * L + tl];
    trhs[0] = kp * position_error.x - kd * task_velocity.x - task_accel.x;
    trhs[1] = kp * position_error.y - kd * task_velocity.y - task_accel.y;
    trhs[2] = kp * position_error.z - kd * task_velocity.z - task_accel.z;
    trhs[3] = kp * orientation_error.x - kd * task_angular.x - task_angular_accel.x;
    trhs[4] = kp * orientation_error.y - kd * task_angular.y - task_angular_accel.y;
    trhs[5] = kp * orientation_error.z - kd * task_angular.z - task_angular_accel.z;
}

// Operational-space control (control mode 4), the Osc branch of ApplyDynamicsDriveKernel (ops/articulation.cu:1419-1550),
// entered with H = (S M^-1 S^T)^-1 in `H`, the actuated joints' table in `dofs` and their force-free accelerations,
// passive terms and inputs in the solver vectors.  J (6 x n, linear rows first) is the Jacobian of the task frame in the
// world, B = J M^-1 S^T (`resp`), the task force F = (B H B^T)^+ (kp x_err - kd v - a_free - B (bias + damping + posture))
// acts through H B^T (`tmap`).  Joints on the chain from the task link to the root hold their posture through the
// nullspace gains, the others through their own drive gains.  Lanes share the work: lane = link for the Jacobian columns,
// lane = task row for the mass solves, lane = actuated joint for the products, lane = matrix row inside the pseudoinverse's rotations.
// The task link's acceleration is the force-free pass's velocity-product acceleration (q'' = 0, `acc0`, read before the
// actuated-inertia matrix overwrites the link scratch) plus J q''.
struct OscIn { uint32_t active, rank, joints; float acc0[6]; };
template <int NR>
static __device__ __noinline__ float osc_command(TorqueIn e, OscIn o, uint32_t* status) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane, L = t.L, n = t.ndof, ld = e.lay->ld, active = o.active, tl = t.cfg.task_link;
    const bool scalar = l < L && joint_dofs(e.jtype) == 1u;
    const bool column = l < active;
    float* vecs = e.sm + e.lay->vecs;
    constexpr uint32_t vs = 32u * NR;
    const float* free_acc = vecs + vs * kVecFree;
    const float* passive = vecs + vs * kVecU;
    float* prhs = vecs + vs * kVecPseudo;                    // posture accelerations of the chain joints
    const uint32_t* dofs = reinterpret_cast<const uint32_t*>(vecs + vs * kVecTmp);
    float* command = vecs + vs * kVecTmp2;
    float* own = vecs + vs * kVecAcc;                        // off-chain joints: their own PD effort (the LDL^T diagonal is dead)
    const float* F = e.sm + e.lay->factor;
    float* H = e.sm + e.lay->heads;
    float* qdd = H + active * active;                        // all n force-free accelerations (saved by the caller)
    float* J = qdd + n;                                      // 6 x n
    float* resp = J + 6u * n;                                // 6 x active
    float* tmap = resp + 6u * active;                        // 6 x active
    float* metric = tmap + 6u * active;                      // 6 x 6
    float* inverse = metric + 36u;                           // 6 x 6
    float* bias = inverse + 36u;                             // active
    float* posture = bias + active;                          // active
    float* chain = posture + active;                         // n flags
    float* trhs = chain + n;                                 // 6
    float* force = trhs + 6u;                                // 6
    float* eigenvectors = force + 6u;                        // 6 x 6 scratch of the pseudoinverse
    const size_t at = (size_t)e.env * L + l;
    const float* pose_t = e.sm + e.lay->pose + 7u * tl;
    const float* frame = e.s->task_frame + (size_t)e.env * 7u;
    const Q4 frame_q = qnorm_le(ldq(frame + 3), 1.0e-12f);
    const V3 offset = ld3(frame);
    const Q4 link_q = ldq(pose_t + 3);
    const V3 task_pos = ld3(pose_t) + qrot(link_q, offset);
    const Q4 task_q = qnorm_le(qmul(link_q, frame_q), 1.0e-12f);
    // bias = -d qd - H qdd_free, lane = actuated joint
    if (column) {
        double b = passive[l];
        for (uint32_t c = 0u; c < active; ++c) b -= (double)H[l * active + c] * free_acc[c];
        bias[l] = (float)b;
    }
    for (uint32_t i = l; i < 6u * n; i += 32u) J[i] = 0.f;
    for (uint32_t i = l; i < n; i += 32u) chain[i] = 0.f;
    __syncwarp();
    // Jacobian columns, lane = link on the chain from the task link to the root
    const bool on_chain = l < L && ((__ldg(t.anc_mask + tl) >> l) & 1u) != 0u;
    if (on_chain) {
        const float* pose_l = e.sm + e.lay->pose + 7u * l;
        const V3 lever = task_pos - ld3(pose_l);
        const uint32_t dof = e.link_dof;
        if (e.jtype == kFloating) {
            const Q4 base_q = ldq(e.s->base_pose + (size_t)e.env * 7u + 3);
#pragma unroll
            for (uint32_t c = 0u; c < 3u; ++c) {
                const V3 axis = qrot(base_q, mk3(c == 0u ? 1.f : 0.f, c == 1u ? 1.f : 0.f, c == 2u ? 1.f : 0.f));
                const V3 lin = cross(axis, lever);
                J[dof + c] = lin.x; J[n + dof + c] = lin.y; J[2u * n + dof + c] = lin.z;
                J[3u * n + dof + c] = axis.x; J[4u * n + dof + c] = axis.y; J[5u * n + dof + c] = axis.z;
                J[dof + 3u + c] = axis.x; J[n + dof + 3u + c] = axis.y; J[2u * n + dof + 3u + c] = axis.z;
            }
        } else if (joint_dofs(e.jtype) == 1u) {
            const V3 axis = qrot(ldq(pose_l + 3), ld3(t.axis + 3u * l));
            const bool revolute = e.jtype == kRevolute;
            const V3 lin = revolute ? cross(axis, lever) : axis, ang = revolute ? axis : mk3(0.f, 0.f, 0.f);
            J[dof] = lin.x; J[n + dof] = lin.y; J[2u * n + dof] = lin.z;
            J[3u * n + dof] = ang.x; J[4u * n + dof] = ang.y; J[5u * n + dof] = ang.z;
            chain[dof] = 1.f;
        }
    }
    __syncwarp();
    const Q4 desired = ldq(e.s->task_rotation + (size_t)e.env * 4u);
    const uint32_t rows = desired.w * desired.w + desired.x * desired.x + desired.y * desired.y + desired.z * desired.z > 1.0e-12f ? 6u : 3u;
    // B: M x = J_r^T through the L D L^T factor, lane = task row
    if (l < rows) {
        float x[32 * NR];
        for (uint32_t i = 0u; i < n; ++i) x[i] = J[l * n + i];
        for (uint32_t j = 0u; j < n; ++j)
            for (uint32_t i = j + 1u; i < n; ++i) x[i] -= F[i * ld + j] * x[j];
        for (uint32_t i = 0u; i < n; ++i) x[i] /= F[i * ld + i];
        for (uint32_t end = n; end > 0u; --end) {
            const uint32_t i = end - 1u;
            float sum = x[i];
            for (uint32_t j = i + 1u; j < n; ++j) sum -= F[j * ld + i] * x[j];
            x[i] = sum;
        }
        for (uint32_t c = 0u; c < active; ++c) resp[l * active + c] = x[dofs[c]];
    }
    __syncwarp();
    if (column)
        for (uint32_t r = 0u; r < rows; ++r) {
            double v = 0.0;
            for (uint32_t a = 0u; a < active; ++a) v += (double)H[l * active + a] * resp[r * active + a];
            tmap[r * active + l] = (float)v;
        }
    for (uint32_t i = l; i < 72u; i += 32u) metric[i] = 0.f;      // metric and inverse
    __syncwarp();
    for (uint32_t i = l; i < rows * rows; i += 32u) {
        const uint32_t r = i / rows, c = i % rows;
        double v = 0.0;
        for (uint32_t a = 0u; a < active; ++a) v += (double)resp[r * active + a] * tmap[c * active + a];
        metric[r * 6u + c] = (float)v;
    }
    __syncwarp();
    task_metric_pseudoinverse(metric, eigenvectors, rows, inverse, l);
    // the task frame's velocity and force-free acceleration in the world, the task-space right-hand side: lane 0
    if (l == 0u) task_right_hand_side(e, o.acc0, J, qdd, trhs, rows, task_pos, task_q, link_q, offset, desired);
    // posture: nullspace gains on the chain's joints (as accelerations through H), own gains elsewhere
    if (scalar) {
        const float pd_error = e.s->drive_target[at] - e.q, rate_error = e.s->vel_target[at] - e.qd;
        const bool mine_on_chain = chain[e.link_dof] != 0.f;
        prhs[o.rank] = mine_on_chain ? e.s->null_kp[e.env] * pd_error + e.s->null_kd[e.env] * rate_error : 0.f;
        own[o.rank] = mine_on_chain ? 0.f : e.s->kp[at] * pd_error + e.s->kd[at] * rate_error;
    }
    __syncwarp();
    if (column) {
        double v = 0.0;
        for (uint32_t c = 0u; c < active; ++c) v += (double)H[l * active + c] * prhs[c];
        const bool off_chain = chain[dofs[l]] == 0.f;
        if (off_chain) v += own[l];
        posture[l] = (float)v;
    }
    __syncwarp();
    if (l < rows) {
        float rhs = trhs[l];
        for (uint32_t a = 0u; a < active; ++a) rhs -= resp[l * active + a] * (bias[a] - passive[a] + posture[a]);
        trhs[l] = rhs;
    }
    __syncwarp();
    if (l < rows) {
        float sum = 0.f;
        for (uint32_t c = 0u; c < rows; ++c) sum += inverse[l * 6u + c] * trhs[c];
        force[l] = sum;
    }
    __syncwarp();
    float value = 0.f;
    if (column) {
        double v = bias[l] + posture[l];
        for (uint32_t r = 0u; r < rows; ++r) v += (double)tmap[r * active + l] * force[r];
        value = (float)v;
    }
    const bool finite = __all_sync(NKB_FULL, !column || isfinite(value));
    if (column) command[l] = finite ? value : 0.f;
    __syncwarp();
    if (!finite) *status = kStatusControlFailure;
    const float mine = scalar ? command[o.rank] : 0.f;
    __syncwarp();
    return mine;
}

template <int NR>
__device__ __noinline__ TorqueOut computed_torque(TorqueIn e) {
    const TemplateView& t = *e.t;
    TorqueOut out;
    out.tau = 0.f; out.command = 0.f; out.status = 0u; out.applied = 0u;
    const uint32_t l = e.lane, L = t.L, n = t.ndof, ld = e.lay->ld;
    const bool scalar = l < L && joint_dofs(e.jtype) == 1u;
    // a drive the affine stage rejected (bounds left at zero) switches the controller off for the env
    if (__any_sync(NKB_FULL, scalar && e.lower == 0.f && e.upper == 0.f)) return out;
    const bool osc = e.mode == 4u;
    if (osc) {          // ops/articulation.cu:1341-1360: every task input finite, gains non-negative
        const uint32_t tl = t.cfg.task_link;
        const float* in3 = e.s->task_target + (size_t)e.env * 3u;
        const float* in4 = e.s->task_rotation + (size_t)e.env * 4u;
        const float* in7 = e.s->task_frame + (size_t)e.env * 7u;
        const float gains[4] = {e.s->kp[(size_t)e.env * L + tl], e.s->kd[(size_t)e.env * L + tl], e.s->null_kp[e.env], e.s->null_kd[e.env]};
        bool ok = true;
        for (int k = 0; k < 3; ++k) ok &= isfinite(in3[k]);
        for (int k = 0; k < 4; ++k) ok &= isfinite(in4[k]);
        for (int k = 0; k < 7; ++k) ok &= isfinite(in7[k]);
        for (int k = 0; k < 4; ++k) ok &= isfinite(gains[k]) && gains[k] >= 0.f;
        if (!ok) { out.status = kStatusControlFailure; return out; }
    }
    const uint32_t joints = __ballot_sync(NKB_FULL, scalar);
    const uint32_t active = (uint32_t)__popc(joints);
    if (active == 0u) return out;
    const uint32_t rank = (uint32_t)__popc(joints & ((1u << l) - 1u));        // this lane's joint among the active ones
    const size_t at = (size_t)e.env * L + l;
    float* vecs = e.sm + e.lay->vecs;
    constexpr uint32_t vs = 32u * NR;
    float* diag = vecs + vs * kVecAcc;
    float* free_acc = vecs + vs * kVecFree;
    float* passive = vecs + vs * kVecU;
    float* rhs = vecs + vs * kVecPseudo;
    uint32_t* dofs = reinterpret_cast<uint32_t*>(vecs + vs * kVecTmp);
    float* command = vecs + vs * kVecTmp2;
    float* A = e.sm + e.lay->chol;                         // active x active, row stride `active`
    float* H = e.sm + e.lay->heads;
    const float* F = e.sm + e.lay->factor;
    out.applied = 1u;
    OscIn osc_in;
    osc_in.active = active; osc_in.rank = rank; osc_in.joints = joints;
    if (osc) {
        // before the actuated-inertia matrix overwrites the link scratch and the solver vectors: the task link's force-free
        // acceleration and all n force-free coordinate accelerations
        const float* a0 = e.sm + e.lay->acc + 6u * t.cfg.task_link;
#pragma unroll
        for (int k = 0; k < 6; ++k) osc_in.acc0[k] = a0[k];
        float* keep = H + active * active;
        for (uint32_t i = l; i < n; i += 32u) keep[i] = vecs[vs * kVecAcc + i];
    }
    __syncwarp();
    if (scalar) {
        out.tau = e.s->feedforward[at];
        dofs[rank] = e.link_dof;
        free_acc[rank] = e.qdd;
        passive[rank] = -__ldg(t.damping + l) * e.qd;
        rhs[rank] = e.s->acc_target[at] + e.s->kp[at] * (e.s->drive_target[at] - e.q) + e.s->kd[at] * (e.s->vel_target[at] - e.qd);
    }
    __syncwarp();
    const bool column = l < active;
    float x[32 * NR];
    // S M^-1 S^T, column by column: M x = e_dof(c) through the L D L^T factor (articulation_mass.cuh:357-411)
    if (column) {
        for (uint32_t i = 0u; i < n; ++i) x[i] = i == dofs[l] ? 1.0f : 0.0f;
        for (uint32_t j = 0u; j < n; ++j)
            for (uint32_t i = j + 1u; i < n; ++i) x[i] -= F[i * ld + j] * x[j];
        for (uint32_t i = 0u; i < n; ++i) x[i] /= F[i * ld + i];
        for (uint32_t end = n; end > 0u; --end) {
            const uint32_t i = end - 1u;
            float s = x[i];
            for (uint32_t j = i + 1u; j < n; ++j) s -= F[j * ld + i] * x[j];
            x[i] = s;
        }
        for (uint32_t r = 0u; r < active; ++r) A[r * active + l] = x[dofs[r]];
    }
    __syncwarp();
    if (column)
        for (uint32_t c = 0u; c < l; ++c) {
            const float v = 0.5f * (A[l * active + c] + A[c * active + l]);
            A[l * active + c] = v; A[c * active + l] = v;
        }
    __syncwarp();
    // L D L^T of the actuated block (FactorControlMass): every lane follows the pivots, lane i owns row i
    bool definite = true;
    for (uint32_t j = 0u; j < active; ++j) {
        double pivot = A[j * active + j];
        for (uint32_t k = 0u; k < j; ++k) { const double v = A[j * active + k]; pivot -= v * v * diag[k]; }
        if (!(pivot > 0.0) || !isfinite(pivot)) { definite = false; break; }
        __syncwarp();
        if (l == 0u) diag[j] = (float)pivot;
        if (column && l > j) {
            double v = A[l * active + j];
            for (uint32_t k = 0u; k < j; ++k) v -= (double)A[l * active + k] * A[j * active + k] * diag[k];
            A[l * active + j] = (float)(v / pivot);
        }
        __syncwarp();
    }
    if (!definite) { out.status = kStatusControlFailure; return out; }
    // H = inverse, column by column (SolveControlMass on unit vectors)
    if (column) {
        for (uint32_t i = 0u; i < active; ++i) {
            double v = i == l ? 1.0 : 0.0;
            for (uint32_t j = 0u; j < i; ++j) v -= (double)A[i * active + j] * x[j];
            x[i] = (float)v;
        }
        for (uint32_t i = 0u; i < active; ++i) x[i] /= diag[i];
        for (uint32_t ii = active; ii > 0u; --ii) {
            const uint32_t i = ii - 1u;
            double v = x[i];
            for (uint32_t j = i + 1u; j < active; ++j) v -= (double)A[j * active + i] * x[j];
            x[i] = (float)v;
        }
        for (uint32_t r = 0u; r < active; ++r) H[r * active + l] = x[r];
    }
    __syncwarp();
    if (osc) {
        uint32_t failed = 0u;
        out.command = osc_command<NR>(e, osc_in, &failed);
        out.status = failed;
        return out;
    }
    // command = bias + H rhs, bias = -d qd - H qdd_free; lane r owns row r
    float value = 0.f;
    if (column) {
        double b = passive[l];
        for (uint32_t c = 0u; c < active; ++c) b -= (double)H[l * active + c] * free_acc[c];
        double v = (double)(float)b;
        for (uint32_t c = 0u; c < active; ++c) v += (double)H[l * active + c] * rhs[c];
        value = (float)v;
    }
    const bool finite = __all_sync(NKB_FULL, !column || isfinite(value));
    if (column) command[l] = finite ? value : 0.f;
    __syncwarp();
    if (scalar) out.command = command[rank];
    if (!finite) out.status = kStatusControlFailure;
    __syncwarp();
    return out;
}

template <int NR>
NKB_DEV void stage_computed_torque(Env& e) {
    TorqueIn in;
    in.sm = e.sm; in.lay = e.lay; in.t = e.t; in.s = e.s; in.env = e.env; in.lane = e.lane; in.jtype = e.jtype; in.link_dof = e.link_dof;
    in.mode = e.t->cfg.control_mode;
    in.q = e.q; in.qd = e.qd; in.qdd = e.qdd; in.lower = e.drive_lower; in.upper = e.drive_upper;
    const TorqueOut out = computed_torque<NR>(in);
    e.status |= out.status;
    if (out.applied != 0u && e.lane < e.t->L && joint_dofs(e.jtype) == 1u) {
        e.tau = out.tau;
        if (out.status == 0u) e.drive_command = out.command;
    }
}

// q += dt (qdot + pseudo); floating base pose; ops/articulation.cu:732-791.
NKB_DEV void stage_integrate_links(Env& e, bool use_pseudo) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane;
    if (l >= t.L) return;
    const float dt = t.cfg.dt;
    const float* ps = sm_vec(e, kVecPseudo);
    if (joint_dofs(e.jtype) == 1u) e.q += (e.qd + (use_pseudo ? ps[e.link_dof] : 0.f)) * dt;
    else e.q += e.qd * dt;
    if (e.parent == kNoLink && e.jtype == kFloating) {
        float* rv = sm_vel(e, l);
        float v[6];
#pragma unroll
        for (int i = 0; i < 6; ++i) v[i] = rv[i] + (use_pseudo ? ps[i] : 0.f);
        float* bp = e.s->base_pose + (size_t)e.env * 7u;
        const Q4 rot = ldq(bp + 3);
        const V3 vw = qrot(rot, mk3(v[3], v[4], v[5]));
        st3(bp, ld3(bp) + vw * dt);
        const Q4 dq = mkq(1.0f, 0.5f * v[0] * dt, 0.5f * v[1] * dt, 0.5f * v[2] * dt);
        stq(bp + 3, qnorm_lt(qmul(rot, dq), 1.0e-24f));
        const V3 turned = qrot_inv(qnorm_lt(dq, 1.0e-24f), mk3(rv[3], rv[4], rv[5]));
        rv[3] = turned.x; rv[4] = turned.y; rv[5] = turned.z;
    }
}

// Link spatial velocities after the solve, ops/articulation.cu:647-689.
NKB_DEV void stage_link_velocities(Env& e) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane;
    const bool link = l < t.L;
    const bool froot = link && e.parent == kNoLink && e.jtype == kFloating;
    float E[9]; V3 r = mk3(0.f, 0.f, 0.f);
    if (link) joint_xform(e, E, r);
    V3 jw = mk3(0.f, 0.f, 0.f), jv = jw;
    if (e.jtype == kRevolute) jw = e.axis * e.qd; else if (e.jtype == kPrismatic) jv = e.axis * e.qd;
    for (uint32_t d = 0; d <= t.max_depth; ++d) {
        if (link && e.depth == d && !froot) {
            V3 pw = mk3(0.f, 0.f, 0.f), pv = pw;
            if (e.parent != kNoLink) { pw = ld3(sm_vel(e, e.parent)); pv = ld3(sm_vel(e, e.parent) + 3); }
            V3 tw, tv;
            xf_motion(E, r, pw, pv, tw, tv);
            st3(sm_vel(e, l), tw + jw); st3(sm_vel(e, l) + 3, tv + jv);
        }
        __syncwarp();
    }
}

// Writes the articulation's public state back to global memory.
NKB_DEV void stage_store_links(Env& e) {
    const TemplateView& t = *e.t;
    const uint32_t l = e.lane, L = t.L;
    if (l < L) {
        const size_t at = (size_t)e.env * L + l;
        e.s->q[at] = e.q; e.s->qdot[at] = e.qd; e.s->qddot[at] = e.qdd; e.s->tau[at] = e.tau;
    }
    float* gp = e.s->link_pose + (size_t)e.env * L * 7u;
    const float* sp = e.sm + e.lay->pose;
    for (uint32_t k = l; k < L * 7u; k += 32u) gp[k] = sp[k];
    float* gv = e.s->link_vel + (size_t)e.env * L * 6u;
    const float* sv = e.sm + e.lay->vel;
    for (uint32_t k = l; k < L * 6u; k += 32u) gv[k] = sv[k];
}

}  // namespace nkb

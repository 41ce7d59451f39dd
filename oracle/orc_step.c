/* Oracle (test infrastructure): template blob parsing, world state, the step sequence and field access.
 * The step order restates the reference's nk::Pipeline::BuildInterval (src/nk/pipeline/pipeline.cpp:367-986). */
#include <stdlib.h>
#include <stdio.h>
#include "orc.h"
#include "orc_math.h"
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---- template blob: "NKT1", count, then {name[32], dtype u32, pad u32, n u64, data padded to 8} ---- */
typedef struct { const char *name; uint32_t dtype; uint64_t n; const void *data; } blob_entry;
static int blob_find(const uint8_t *blob, size_t bytes, const char *name, blob_entry *out) {
    if (bytes < 8 || memcmp(blob, "NKT1", 4) != 0) return 0;
    uint32_t count; memcpy(&count, blob + 4, 4);
    size_t at = 8;
    for (uint32_t i = 0; i < count; ++i) {
        if (at + 48 > bytes) return 0;
        const char *nm = (const char *)(blob + at);
        uint32_t dtype; uint64_t n;
        memcpy(&dtype, blob + at + 32, 4); memcpy(&n, blob + at + 40, 8);
        const size_t esz = dtype == 3u ? 8u : 4u;
        const size_t payload = (size_t)((n * esz + 7u) & ~(uint64_t)7u);
        if (at + 48 + payload > bytes) return 0;
        if (strncmp(nm, name, 32) == 0) { out->name = nm; out->dtype = dtype; out->n = n; out->data = blob + at + 48; return 1; }
        at += 48 + payload;
    }
    return 0;
}
static void *blob_arr(const uint8_t *blob, size_t bytes, const char *name, uint64_t expect, int *ok) {
    blob_entry e;
    if (!blob_find(blob, bytes, name, &e) || (expect != (uint64_t)-1 && e.n != expect)) { fprintf(stderr, "[oracle] template field %s missing or mis-sized\n", name); *ok = 0; return NULL; }
    return (void *)e.data;
}

static uint32_t joint_dofs(uint32_t t) { return (t == ORC_JOINT_REVOLUTE || t == ORC_JOINT_PRISMATIC) ? 1u : t == ORC_JOINT_FLOATING ? 6u : t == ORC_JOINT_SPHERICAL ? 3u : 0u; }

static float *falloc(size_t n) { return (float *)calloc(n ? n : 1u, sizeof(float)); }

static void env_alloc(const orc_model *m, orc_env *e) {
    const uint32_t L = m->L, B = m->B, n = m->ndof, S = m->cfg.max_contacts;
    memset(e, 0, sizeof *e);
    e->q = falloc(L); e->qdot = falloc(L); e->qddot = falloc(L); e->tau = falloc(L);
    e->link_pose = falloc(7 * L); e->link_vel = falloc(6 * L); e->link_acc = falloc(6 * L);
    e->link_vbias = falloc(6 * L); e->link_pbias = falloc(6 * L); e->link_S = falloc(6 * L);
    e->link_xup = falloc(36 * L); e->link_ic = falloc(36 * L);
    e->drive_target = falloc(L); e->vel_target = falloc(L); e->kp = falloc(L); e->kd = falloc(L); e->noload_speed = falloc(L); e->acc_target = falloc(L);
    e->force_limit = falloc(L); e->feedforward = falloc(L); e->limit_lambda = falloc(2 * L);
    e->drive_command = falloc(L); e->drive_dissipation = falloc(L); e->drive_lower = falloc(L); e->drive_upper = falloc(L);
    e->actuator_applied = falloc(L);
    e->M = falloc((size_t)n * n); e->Mfactor = falloc((size_t)n * n); e->bias = falloc(n);
    e->body_pose = falloc(7 * B); e->body_linvel = falloc(3 * B); e->body_angvel = falloc(3 * B);
    e->body_winv = falloc(6 * B); e->aabb_lo = falloc(3 * B); e->aabb_hi = falloc(3 * B);
    e->pairs = (uint32_t *)calloc(2 * S + 1, 4); e->ccount = (uint32_t *)calloc(S + 1, 4);
    e->cpoint = falloc(12 * S); e->cnormal = falloc(12 * S); e->cdepth = falloc(4 * S);
    e->cid_pair = (uint64_t *)calloc(4 * S + 1, 8); e->cid_feature = (uint64_t *)calloc(4 * S + 1, 8);
    e->row_cap = S * 12u + 4u * L;
    e->rows = (orc_row *)calloc(e->row_cap + 1, sizeof(orc_row));
    e->jac_pool = falloc((size_t)e->row_cap * 2u * (n ? n : 1u));
    e->artic_vel = falloc(n); e->artic_free = falloc(n); e->qdot_pseudo = falloc(n);
    e->rigid_vel = falloc(6 * B); e->rigid_free = falloc(6 * B); e->body_pseudo = falloc(6 * B);
    e->cache = (orc_cache_entry *)calloc(4 * S + 1, sizeof(orc_cache_entry));
    e->cache_next = (orc_cache_entry *)calloc(4 * S + 1, sizeof(orc_cache_entry));
}
static void env_free(orc_env *e) {
    void *p[] = {e->q, e->qdot, e->qddot, e->tau, e->link_pose, e->link_vel, e->link_acc, e->link_vbias, e->link_pbias, e->link_S,
                 e->link_xup, e->link_ic, e->drive_target, e->vel_target, e->kp, e->kd, e->force_limit, e->feedforward, e->noload_speed, e->acc_target,
                 e->drive_command, e->drive_dissipation, e->drive_lower, e->drive_upper, e->actuator_applied, e->M, e->Mfactor, e->bias,
                 e->body_pose, e->body_linvel, e->body_angvel, e->body_winv, e->aabb_lo, e->aabb_hi, e->pairs, e->ccount,
                 e->cpoint, e->cnormal, e->cdepth, e->cid_pair, e->cid_feature, e->rows, e->jac_pool, e->artic_vel, e->artic_free,
                 e->qdot_pseudo, e->rigid_vel, e->rigid_free, e->body_pseudo, e->cache, e->cache_next, e->limit_lambda};
    for (size_t i = 0; i < sizeof p / sizeof p[0]; ++i) free(p[i]);
}

/* reference src/nk/pipeline/world.cpp:289-654 SeedInitialState: every env starts from the template */
static void env_seed(const orc_model *m, orc_env *e) {
    const uint32_t L = m->L, B = m->B, n = m->ndof, S = m->cfg.max_contacts;
    for (uint32_t l = 0; l < L; ++l) {
        e->q[l] = m->q0[l]; e->qdot[l] = 0.0f; e->qddot[l] = 0.0f; e->tau[l] = 0.0f;
        e->drive_target[l] = m->q0[l]; e->vel_target[l] = 0.0f; e->feedforward[l] = 0.0f; e->acc_target[l] = 0.0f;
        e->kp[l] = m->kp0[l]; e->kd[l] = m->kd0[l]; e->force_limit[l] = m->force_limit0[l];
    }
    memset(e->link_vel, 0, sizeof(float) * 6 * L);
    memset(e->limit_lambda, 0, sizeof(float) * 2 * L);
    memset(e->task_target, 0, sizeof e->task_target); memset(e->task_rotation, 0, sizeof e->task_rotation);
    memset(e->task_frame, 0, sizeof e->task_frame); e->task_frame[3] = 1.0f; e->null_kp = e->null_kd = 0.0f;
    if (L) memcpy(e->base_pose, m->base_pose0, 28);
    if (B) memcpy(e->body_pose, m->body_pose0, sizeof(float) * 7 * B);
    memset(e->body_linvel, 0, sizeof(float) * 3 * B); memset(e->body_angvel, 0, sizeof(float) * 3 * B);
    memset(e->artic_vel, 0, sizeof(float) * n); memset(e->artic_free, 0, sizeof(float) * n);
    memset(e->rigid_vel, 0, sizeof(float) * 6 * B); memset(e->rigid_free, 0, sizeof(float) * 6 * B);
    memset(e->cache, 0, sizeof(orc_cache_entry) * 4 * S); memset(e->cache_next, 0, sizeof(orc_cache_entry) * 4 * S);
    e->status = 0; e->nrows = 0; e->pair_count = 0; e->contact_points = 0;
    orc_fk(m, e);
    orc_sync_bodies(m, e);
}

orc_world *orc_world_create(const void *blob_in, size_t bytes, uint32_t env_count) {
    orc_world *w = (orc_world *)calloc(1, sizeof *w);
    w->blob_copy = malloc(bytes);
    memcpy(w->blob_copy, blob_in, bytes);
    const uint8_t *blob = (const uint8_t *)w->blob_copy;
    orc_model *m = &w->m;
    int ok = 1;
    const float *cf = (const float *)blob_arr(blob, bytes, "cfg_f", 10, &ok);
    const uint32_t *cu = (const uint32_t *)blob_arr(blob, bytes, "cfg_u", 6, &ok);
    if (!ok) { orc_world_destroy(w); return NULL; }
    m->cfg.dt = cf[0]; m->cfg.gravity[0] = cf[1]; m->cfg.gravity[1] = cf[2]; m->cfg.gravity[2] = cf[3];
    m->cfg.pos_beta = cf[4]; m->cfg.pos_slop = cf[5]; m->cfg.contact_margin = cf[6];
    m->cfg.baumgarte_max_velocity = cf[7]; m->cfg.overlap_recovery_velocity = cf[8]; m->cfg.velocity_tolerance = cf[9];
    m->cfg.vel_iters = cu[0]; m->cfg.pos_iters = cu[1]; m->cfg.max_contacts = cu[2]; m->cfg.max_pairs = cu[3];
    m->L = cu[4]; m->B = cu[5];
    const uint32_t L = m->L, B = m->B;
#define F(name, cnt) (float *)blob_arr(blob, bytes, name, (uint64_t)(cnt), &ok)
#define U(name, cnt) (uint32_t *)blob_arr(blob, bytes, name, (uint64_t)(cnt), &ok)
    m->parent = U("parent", L); m->jtype = U("jtype", L); m->link_body = U("link_body", L); m->geom_kind = U("geom_kind", L);
    m->limit_flags = U("limit_flags", L);
    m->axis = F("axis", 3 * L); m->local_pos = F("local_pos", 3 * L); m->local_quat = F("local_quat", 4 * L);
    m->parent_offset = F("parent_offset", 3 * L); m->com = F("com", 3 * L); m->inertia = F("inertia", 36 * L);
    m->damping = F("damping", L); m->armature = F("armature", L); m->frictionloss = F("frictionloss", L);
    m->stiffness = F("stiffness", L); m->spring_ref = F("spring_ref", L);
    m->limit_lower = F("limit_lower", L); m->limit_upper = F("limit_upper", L);
    m->geom_pos = F("geom_pos", 3 * L); m->geom_quat = F("geom_quat", 4 * L);
    m->q0 = F("q0", L); m->base_pose0 = F("base_pose0", 7);
    m->kp0 = F("kp0", L); m->kd0 = F("kd0", L); m->force_limit0 = F("force_limit0", L);
    m->shape_kind = U("shape_kind", B); m->contype = U("contype", B); m->conaffinity = U("conaffinity", B);
    m->group = U("group", B); m->body_to_link = U("body_to_link", B); m->body_id = (int32_t *)U("body_id", B);
    m->shape_params = F("shape_params", 4 * B); m->mu = F("mu", B); m->inv_mass = F("inv_mass", B);
    m->inv_inertia = F("inv_inertia", 3 * B); m->inertial_pos = F("inertial_pos", 3 * B); m->inertial_quat = F("inertial_quat", 4 * B);
    m->body_pose0 = F("body_pose0", 7 * B);
    blob_entry ex;
    if (blob_find(blob, bytes, "excluded", &ex)) { m->excluded = (uint64_t *)ex.data; m->n_excluded = (uint32_t)ex.n; }
    if (!ok || m->cfg.max_contacts > 1024u) { orc_world_destroy(w); return NULL; }
    /* shape frames per collidable row: the template's own, or each link's single shape frame */
    m->body_geom_kind = (uint32_t *)calloc(B + 1, 4); m->body_geom_pos = (float *)calloc(3 * B + 3, 4); m->body_geom_quat = (float *)calloc(4 * B + 4, 4);
    {
        blob_entry gk, gp, gq;
        const int own = blob_find(blob, bytes, "body_geom_kind", &gk) && gk.n == B && blob_find(blob, bytes, "body_geom_pos", &gp) && gp.n == 3u * B &&
                        blob_find(blob, bytes, "body_geom_quat", &gq) && gq.n == 4u * B;
        for (uint32_t b = 0; b < B; ++b) {
            const uint32_t l = m->body_to_link[b];
            if (own) {
                m->body_geom_kind[b] = ((const uint32_t *)gk.data)[b];
                memcpy(m->body_geom_pos + 3 * b, (const float *)gp.data + 3 * b, 12); memcpy(m->body_geom_quat + 4 * b, (const float *)gq.data + 4 * b, 16);
            } else if (l != ORC_NOLINK && l < L) {
                m->body_geom_kind[b] = m->geom_kind[l];
                memcpy(m->body_geom_pos + 3 * b, m->geom_pos + 3 * l, 12); memcpy(m->body_geom_quat + 4 * b, m->geom_quat + 4 * l, 16);
            } else m->body_geom_quat[4 * b] = 1.0f;
        }
    }
    /* derived tree tables (reference model.link_tree_depth / link_child_range / link_children) */
    m->depth = (uint32_t *)calloc(L + 1, 4); m->child_begin = (uint32_t *)calloc(L + 2, 4);
    m->children = (uint32_t *)calloc(L + 1, 4); m->link_dof = (uint32_t *)calloc(L + 1, 4);
    m->max_depth = 0; m->ndof = 0;
    for (uint32_t l = 0; l < L; ++l) {
        m->depth[l] = m->parent[l] == ORC_NOLINK ? 0u : m->depth[m->parent[l]] + 1u;
        if (m->depth[l] > m->max_depth) m->max_depth = m->depth[l];
        m->link_dof[l] = m->ndof; m->ndof += joint_dofs(m->jtype[l]);
    }
    uint32_t at = 0;
    for (uint32_t l = 0; l < L; ++l) {
        m->child_begin[l] = at;
        for (uint32_t c = 0; c < L; ++c) if (m->parent[c] == l) m->children[at++] = c;
    }
    m->child_begin[L] = at;
    if (m->ndof > ORC_MAX_DOF) { orc_world_destroy(w); return NULL; }
    w->E = env_count;
    w->m.env_count = env_count;
    w->m.broadphase = 0u;
    w->env = (orc_env *)calloc(env_count ? env_count : 1u, sizeof(orc_env));
    for (uint32_t i = 0; i < env_count; ++i) { env_alloc(m, &w->env[i]); env_seed(m, &w->env[i]); }
    return w;
}

void orc_world_destroy(orc_world *w) {
    if (!w) return;
    if (w->env) { for (uint32_t i = 0; i < w->E; ++i) env_free(&w->env[i]); free(w->env); }
    free(w->m.depth); free(w->m.child_begin); free(w->m.children); free(w->m.link_dof);
    free(w->m.body_geom_kind); free(w->m.body_geom_pos); free(w->m.body_geom_quat);
    free(w->blob_copy); free(w);
}

/* control mode of every env: 0 PD position, 1 torque, 2 velocity; other values are ignored */
void orc_world_set_control_mode(orc_world *w, uint32_t mode) { if (mode <= 5u) w->m.cfg.control_mode = mode; }
void orc_world_set_task_link(orc_world *w, uint32_t link) { w->m.cfg.task_link = link; }

void orc_world_set_broadphase(orc_world *w, uint32_t mode) { if (mode <= 2u) w->m.broadphase = mode; }

void orc_world_reset(orc_world *w) { for (uint32_t i = 0; i < w->E; ++i) env_seed(&w->m, &w->env[i]); }
void orc_world_refresh(orc_world *w) { for (uint32_t i = 0; i < w->E; ++i) { orc_fk(&w->m, &w->env[i]); orc_sync_bodies(&w->m, &w->env[i]); } }

/* pipeline.cpp:367-986 */
void orc_step_env(const orc_model *m, orc_env *e) {
    const int has_artic = m->L > 0u, has_bodies = m->B > 0u;
    const int has_contacts = e->row_cap > 0u;
    const int has_collidables = has_bodies && m->cfg.max_contacts > 0u;
    if (has_artic) {
        orc_fk(m, e); orc_apply_drives(m, e);
        if (m->cfg.control_mode == 3u || m->cfg.control_mode == 4u) {
            /* pipeline.cpp:406-426: a force-free dynamics pass on the current kinematics, the inverse-dynamics controller on
             * its mass response and acceleration, then the step's dynamics pass (the same mass matrix) */
            orc_dynamics(m, e, 0);
            orc_apply_dynamics_drives(m, e);
        }
        orc_dynamics(m, e, 1);
    }
    orc_body_integrate_velocity(m, e);
    if (has_bodies) orc_sync_bodies(m, e);
    if (has_collidables) { orc_build_aabbs(m, e); orc_find_pairs(m, e); orc_narrowphase(m, e); }
    if (has_contacts) { orc_assemble_rows(m, e); orc_warm_start_prepare(m, e); }
    orc_solve(m, e);
    /* a limit row's slot keeps the multiplier of the velocity solve for the next step's row (block_descent_tile.cuh:2556) */
    for (uint32_t r = 0; r < e->nrows; ++r)
        if (e->rows[r].tag == 1u) e->limit_lambda[2u * e->rows[r].link + ((e->rows[r].flags & ORC_ROW_LIMIT_UPPER) ? 1u : 0u)] = e->rows[r].lambda;
    if (has_contacts) { orc_warm_start_commit(m, e); orc_readout_drives(m, e); }
    orc_integrate_position(m, e);
    if (has_artic) { orc_fk(m, e); orc_fk_link_velocities(m, e); }
    if (has_bodies) orc_sync_bodies(m, e);
}

int orc_hw_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();      /* the cores this process may run on, whatever OMP_NUM_THREADS says */
#else
    return 1;
#endif
}

void orc_world_step(orc_world *w, uint32_t n, int threads) {
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    (void)threads;
#endif
    for (uint32_t s = 0; s < n; ++s) {
#ifdef _OPENMP
#pragma omp parallel for schedule(dynamic, 8) num_threads(threads)
#endif
        for (int64_t i = 0; i < (int64_t)w->E; ++i) orc_step_env(&w->m, &w->env[i]);
    }
}

void orc_stage_dynamics(orc_world *w, int integrate_velocity) {
    for (uint32_t i = 0; i < w->E; ++i) { orc_fk(&w->m, &w->env[i]); orc_apply_drives(&w->m, &w->env[i]); orc_dynamics(&w->m, &w->env[i], integrate_velocity); }
}
void orc_stage_collide(orc_world *w) {
    for (uint32_t i = 0; i < w->E; ++i) {
        orc_env *e = &w->env[i];
        orc_fk(&w->m, e); orc_body_integrate_velocity(&w->m, e); orc_sync_bodies(&w->m, e);
        orc_build_aabbs(&w->m, e); orc_find_pairs(&w->m, e); orc_narrowphase(&w->m, e);
    }
}

/* ---- field access ---- */
typedef struct { const char *name; size_t per_env; size_t elem; int kind; } field_desc;
static void *field_ptr(const orc_model *m, orc_env *e, const char *f, size_t *count, size_t *esz) {
    const uint32_t L = m->L, B = m->B, n = m->ndof, S = m->cfg.max_contacts;
    *esz = 4;
#define R(nm, p, c) if (strcmp(f, nm) == 0) { *count = (c); return (void *)(p); }
    R("q", e->q, L) R("qdot", e->qdot, L) R("qddot", e->qddot, L) R("tau", e->tau, L)
    R("base_pose", e->base_pose, 7) R("link_pose", e->link_pose, 7 * L) R("link_velocity", e->link_vel, 6 * L)
    R("link_acceleration", e->link_acc, 6 * L)
    R("drive_target", e->drive_target, L) R("velocity_target", e->vel_target, L) R("noload_speed", e->noload_speed, L) R("acceleration_target", e->acc_target, L) R("drive_stiffness", e->kp, L)
    R("drive_damping", e->kd, L) R("drive_force_limit", e->force_limit, L) R("joint_feedforward", e->feedforward, L)
    R("actuator_applied", e->actuator_applied, L)
    R("mass_matrix", e->M, (size_t)n * n) R("mass_factor", e->Mfactor, (size_t)n * n) R("bias", e->bias, n)
    R("body_pose", e->body_pose, 7 * B) R("body_linear_velocity", e->body_linvel, 3 * B) R("body_angular_velocity", e->body_angvel, 3 * B)
    R("aabb_lo", e->aabb_lo, 3 * B) R("aabb_hi", e->aabb_hi, 3 * B)
    R("pair_count", &e->pair_count, 1) R("candidate_pairs", e->pairs, 2 * S) R("contact_count", e->ccount, S)
    R("contact_point", e->cpoint, 12 * S) R("contact_normal", e->cnormal, 12 * S) R("contact_depth", e->cdepth, 4 * S)
    R("env_status", &e->status, 1) R("solver_residual", e->solver_residual, 4) R("solver_sweeps", &e->sweeps, 1)
    R("limit_multiplier", e->limit_lambda, 2 * L) R("task_target", e->task_target, 3) R("task_rotation_target", e->task_rotation, 4)
    R("task_local_pose", e->task_frame, 7) R("task_nullspace_stiffness", &e->null_kp, 1) R("task_nullspace_damping", &e->null_kd, 1) R("contact_points", &e->contact_points, 1) R("qdot_pseudo", e->qdot_pseudo, n) R("dof_velocity", e->artic_vel, n)
#undef R
    *count = 0;
    return NULL;
}
int orc_get(orc_world *w, const char *field, void *out, size_t bytes) {
    for (uint32_t i = 0; i < w->E; ++i) {
        size_t count, esz;
        void *p = field_ptr(&w->m, &w->env[i], field, &count, &esz);
        if (!p) return 1;
        if (bytes != (size_t)w->E * count * esz) return 2;
        memcpy((uint8_t *)out + (size_t)i * count * esz, p, count * esz);
    }
    return 0;
}
int orc_set(orc_world *w, const char *field, const void *in, size_t bytes) {
    for (uint32_t i = 0; i < w->E; ++i) {
        size_t count, esz;
        void *p = field_ptr(&w->m, &w->env[i], field, &count, &esz);
        if (!p) return 1;
        if (bytes != (size_t)w->E * count * esz) return 2;
        memcpy(p, (const uint8_t *)in + (size_t)i * count * esz, count * esz);
    }
    return 0;
}

/*
 * CPU oracle for the batched articulated-robot step: TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's step algorithm (kry4r/Nuka-Physics),
 * one function per pipeline stage, each citing the reference file:line it follows.
 * Nothing in the shipped library links or calls this code; the tests, the smoke
 * entry and the bench's CPU-baseline leg use it as the checker.
 *
 * Pin status: the reference has no CPU implementation of this path and its MJX
 * golden trajectories are Git-LFS pointers only, so this restatement is pinned on
 * the closed-form expectations of the reference's own tests (see tests/): analytic
 * manifold cases, the friction-cone / relaxation / momentum-restart cases of
 * tests/math/test_contact_tangent.cpp, the contact-identity rules of
 * tests/constraint/test_contact_identity.cpp, brute-force pair sets, momentum
 * exchange, resting contact, rotated-gravity covariance, M qdd == tau - bias.
 * Numerical agreement with MuJoCo itself is "parity unpinned".
 *
 * Conventions (reference src/math/cuda_spatial_ops.cuh:1-30, nuka.h:498):
 *   spatial vectors are angular-first [w(3); v(3)]; quaternions are wxyz;
 *   poses are xyz then wxyz (7 floats).
 */
#ifndef ORC_H
#define ORC_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ORC_NOLINK 0xffffffffu

/* reference src/phi/articulation_contract.hpp joint codes */
enum { ORC_JOINT_REVOLUTE = 0, ORC_JOINT_PRISMATIC = 1, ORC_JOINT_FIXED = 2,
       ORC_JOINT_FLOATING = 3, ORC_JOINT_SPHERICAL = 4 };
/* reference src/collision/shape_kind.hpp:10-19 */
enum { ORC_SHAPE_SPHERE = 0, ORC_SHAPE_CAPSULE = 1, ORC_SHAPE_BOX = 2, ORC_SHAPE_PLANE = 3, ORC_SHAPE_CYLINDER = 7 };
/* reference src/phi/op_schema.hpp:36-52 */
enum { ORC_STATUS_PAIR_OVERFLOW = 1u << 0, ORC_STATUS_DOF_OVERFLOW = 1u << 2,
       ORC_STATUS_GYRO_FAILURE = 1u << 5, ORC_STATUS_CONTROL_FAILURE = 1u << 10,
       ORC_STATUS_SOLVER_FAILURE = 1u << 13 };

/* row flags, reference src/nk/solve/nk_row.hpp:42-58 */
enum { ORC_ROW_ACTIVE = 1u << 0, ORC_ROW_BLOCK_NORMAL = 1u << 2, ORC_ROW_BLOCK_TANGENT = 1u << 3,
       ORC_ROW_LIMIT_LOWER = 1u << 4, ORC_ROW_LIMIT_UPPER = 1u << 5, ORC_ROW_CONTACT_NORMAL = 1u << 6,
       ORC_ROW_VELOCITY_ONLY = 1u << 7, ORC_ROW_SPECULATIVE = 1u << 8 };

enum { ORC_SIDE_RIGID = 0, ORC_SIDE_ARTIC = 1, ORC_SIDE_STATIC = 3 };

#define ORC_MAX_DOF 64
#define ORC_PTS_PER_SLOT 4

typedef struct orc_config {
    float dt;
    float gravity[3];
    uint32_t vel_iters;
    uint32_t pos_iters;
    float pos_beta, pos_slop;
    float contact_margin;
    float baumgarte_max_velocity;
    float overlap_recovery_velocity;
    float velocity_tolerance;
    uint32_t max_contacts;      /* candidate slots per env */
    uint32_t max_pairs;         /* 0: same as max_contacts */
    uint32_t control_mode;      /* 0 PD position, 1 torque, 2 velocity, 3 computed torque, 4 operational space, 5 actuator (phi/articulation_contract.hpp:16-23) */
    uint32_t task_link;         /* mode 4: the link that carries the task frame */
} orc_config;

/* One env's cooked template (reference src/nk/model/model.hpp:175-244, 488-548). */
typedef struct orc_model {
    uint32_t L;                 /* links per env (0: no articulation) */
    uint32_t B;                 /* collidable body rows per env */
    uint32_t ndof;
    /* links */
    uint32_t *parent, *jtype, *link_body, *geom_kind, *limit_flags, *depth;
    uint32_t max_depth;
    uint32_t *child_begin, *children;   /* children of link i: children[child_begin[i]..child_begin[i+1]) */
    uint32_t *link_dof;                 /* first dof of each link */
    float *axis, *local_pos, *local_quat, *parent_offset, *com, *inertia;
    float *damping, *armature, *frictionloss, *stiffness, *spring_ref;
    float *limit_lower, *limit_upper;
    float *geom_pos, *geom_quat;
    /* per collidable row: frame of the shape in its link (derived from the link arrays when the template has no
     * body_geom_* fields); lets one link carry several shapes */
    uint32_t *body_geom_kind; float *body_geom_pos, *body_geom_quat;
    float *q0, *base_pose0;
    float *kp0, *kd0, *force_limit0;
    /* bodies */
    uint32_t *shape_kind, *contype, *conaffinity, *group, *body_to_link;
    int32_t *body_id;
    float *shape_params, *mu, *inv_mass, *inv_inertia, *inertial_pos, *inertial_quat, *body_pose0;
    /* sorted excluded pair keys (a<<32|b) */
    uint64_t *excluded;
    uint32_t n_excluded;
    orc_config cfg;
    uint32_t env_count;         /* envs of the world this model serves (the reference's route choice depends on it) */
    uint32_t broadphase;        /* 0: the reference's rule (all-pairs while B^2 E <= 2^20, else the tree), 1: all-pairs, 2: tree */
} orc_model;

/* one solver row; reference src/nk/solve/nk_row.hpp:73-101 */
typedef struct orc_side { uint32_t kind, index; float jlin[3], jang[3]; } orc_side;
typedef struct orc_row {
    uint32_t flags, group_first, group_normal_count;
    float rhs, compliance, lower, upper, mu, mu2;
    orc_side a, b;
    float penetration;
    float lambda;
    uint32_t contact_slot, contact_point; /* for position bias; ORC_NOLINK on joint rows */
    uint32_t tag, link;                   /* 0 contact, 1 limit, 2 joint friction, 3 drive */
    float *ja, *jb;                       /* chain jacobians (ndof) or NULL */
} orc_row;

typedef struct orc_cache_entry {
    uint64_t pair, feature;
    float lambda[4];
    float normal[3];
    uint32_t age;
    uint32_t valid;
} orc_cache_entry;

/* Per-env state. */
typedef struct orc_env {
    float *q, *qdot, *qddot, *tau;          /* L */
    float base_pose[7];
    float *link_pose;                        /* L*7 */
    float *link_vel;                         /* L*6 */
    float *link_acc, *link_vbias, *link_pbias, *link_S;  /* L*6 */
    float *link_xup, *link_ic;               /* L*36 */
    float *drive_target, *vel_target, *kp, *kd, *force_limit, *feedforward, *noload_speed, *acc_target;
    float task_target[3], task_rotation[4], task_frame[7], null_kp, null_kd;     /* mode 4 inputs: world target, optional orientation (zero = position only), local frame on the task link, posture gains */
    float *limit_lambda;      /* 2 x L: the joint-limit multipliers the last velocity solve left (lower, upper per link) */
    float *drive_command, *drive_dissipation, *drive_lower, *drive_upper;
    float *actuator_applied;                 /* L */
    float *M, *Mfactor, *bias;               /* ndof^2, ndof^2, ndof */
    /* bodies */
    float *body_pose;                        /* B*7 */
    float *body_linvel, *body_angvel;        /* B*3 */
    float *body_winv;                        /* B*6 symmetric xx yy zz xy xz yz */
    float *aabb_lo, *aabb_hi;                /* B*3 */
    /* contacts */
    uint32_t pair_count;
    uint32_t *pairs;                         /* S*2 */
    uint32_t *ccount;                        /* S */
    float *cpoint, *cnormal, *cdepth;        /* S*4*3, S*4*3, S*4 */
    uint64_t *cid_pair, *cid_feature;        /* S*4 */
    /* rows */
    uint32_t nrows, row_cap;
    orc_row *rows;
    float *jac_pool;
    uint32_t contact_points;                 /* live points this step */
    /* solver carried state */
    float *artic_vel, *artic_free;           /* ndof */
    float *rigid_vel, *rigid_free;           /* B*6 */
    float *qdot_pseudo;                      /* ndof */
    float *body_pseudo;                      /* B*6 */
    orc_cache_entry *cache, *cache_next;     /* S*4 */
    float solver_residual[4];
    uint32_t sweeps;
    uint32_t status;
} orc_env;

typedef struct orc_world {
    orc_model m;
    uint32_t E;
    orc_env *env;
    void *blob_copy;
} orc_world;

/* ---- API (all return 0 on success) ---- */
orc_world *orc_world_create(const void *blob, size_t bytes, uint32_t env_count);
void orc_world_destroy(orc_world *w);
void orc_world_reset(orc_world *w);
/* threads <= 0: all cores */
void orc_world_step(orc_world *w, uint32_t n, int threads);
void orc_world_refresh(orc_world *w);           /* FK + body poses after state upload */
/* single stages, for per-stage parity */
void orc_stage_dynamics(orc_world *w, int integrate_velocity);
void orc_stage_collide(orc_world *w);
/* field access: copies E*count floats (or u32) in env-major order */
int orc_get(orc_world *w, const char *field, void *out, size_t bytes);
int orc_set(orc_world *w, const char *field, const void *in, size_t bytes);
int orc_hw_threads(void);

/* internal stages (per env) */
void orc_fk(const orc_model *m, orc_env *e);
void orc_apply_drives(const orc_model *m, orc_env *e);
void orc_factor_mass(const float *M, float *F, uint32_t n);
void orc_solve_mass(const float *F, float *x, uint32_t n);
void orc_apply_dynamics_drives(const orc_model *m, orc_env *e);
void orc_dynamics(const orc_model *m, orc_env *e, int integrate_velocity);
void orc_body_integrate_velocity(const orc_model *m, orc_env *e);
void orc_sync_bodies(const orc_model *m, orc_env *e);
void orc_build_aabbs(const orc_model *m, orc_env *e);
void orc_find_pairs(const orc_model *m, orc_env *e);
void orc_find_pairs_lbvh(const orc_model *m, orc_env *e);
uint32_t orc_lbvh_pair_set(uint32_t n, const float *lo, const float *hi, uint64_t *out, uint32_t capacity);
void orc_world_set_broadphase(orc_world *w, uint32_t mode);
void orc_narrowphase(const orc_model *m, orc_env *e);
void orc_assemble_rows(const orc_model *m, orc_env *e);
void orc_warm_start_prepare(const orc_model *m, orc_env *e);
void orc_solve(const orc_model *m, orc_env *e);
void orc_warm_start_commit(const orc_model *m, orc_env *e);
void orc_readout_drives(const orc_model *m, orc_env *e);
void orc_integrate_position(const orc_model *m, orc_env *e);
void orc_fk_link_velocities(const orc_model *m, orc_env *e);
void orc_step_env(const orc_model *m, orc_env *e);

#ifdef __cplusplus
}
#endif
#endif

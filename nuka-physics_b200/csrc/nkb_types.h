// Plain-data views shared by the host runtime and the CUDA kernels of the batched articulated step.
// One "template" describes a single environment (the role of the reference's cooked nk::Model,
// src/nk/model/model.hpp:175-244); per-env state lives in env-major arrays whose public members keep the
// layouts of the reference's state fields (src/nk/model/fields.yaml): q/qdot per link, poses as
// xyz + wxyz (7 floats), spatial velocities angular-first (6 floats).
#pragma once
#include <cstdint>

namespace nkb {

constexpr uint32_t kNoLink = 0xffffffffu;
constexpr uint32_t kMaxLinks = 32u;     // one warp lane per link
constexpr uint32_t kMaxDof = 64u;       // a warp lane owns coordinates lane and lane + 32
constexpr uint32_t kMaxBodies = 256u;   // collidable rows per env (the env's shared-memory slice is the practical limit)
constexpr uint32_t kPtsPerSlot = 4u;

enum JointType : uint32_t { kRevolute = 0, kPrismatic = 1, kFixed = 2, kFloating = 3, kSpherical = 4 };
enum ShapeKind : uint32_t { kSphere = 0, kCapsule = 1, kBox = 2, kPlane = 3, kCylinder = 7 };      // the reference's collision/shape_kind.hpp:10-17
// env status bits, reference src/phi/op_schema.hpp:36-52
enum : uint32_t { kStatusPairOverflow = 1u << 0, kStatusDofOverflow = 1u << 2, kStatusGyroFailure = 1u << 5,
                  kStatusControlFailure = 1u << 10, kStatusSolverFailure = 1u << 13,
                  kStatusHeadOverflow = 1u << 20,
                  kStatusTeamTimeout = 1u << 21 };     // a warp of an env's team gave up waiting for another (team mode)
// head flags
enum : uint32_t { kHeadContact = 1u << 0, kHeadContactNormal = 1u << 1, kHeadSpeculative = 1u << 2,
                  kHeadVelocityOnly = 1u << 3, kHeadDrive = 1u << 4, kHeadLimit = 1u << 5, kHeadFriction = 1u << 6,
                  kHeadScalar = 1u << 7 /* position pass: only the normal axis */ };
constexpr uint32_t kHeadWords = 64u;
constexpr uint32_t kHeadStride = kHeadWords + 1u;   // odd record stride in shared memory    // words of shared memory per solver head

// Scratch words of the tree broadphase for B collidable rows (nkb_lbvh.cuh): sorted keys, internal nodes (children, range,
// box), split table, ready flags and one partner bit row per body.
#ifdef __CUDACC__
#define NKB_HOST_DEVICE __host__ __device__
#else
#define NKB_HOST_DEVICE
#endif
NKB_HOST_DEVICE inline uint32_t lbvh_pow2(uint32_t b) { uint32_t p = 2u; while (p < b) p <<= 1u; return p; }
NKB_HOST_DEVICE inline uint32_t lbvh_scratch_words(uint32_t B) {
    if (B < 2u) return 0u;
    return 2u * lbvh_pow2(B) + (B - 1u) * 10u + 4u * B + B * ((B + 31u) / 32u);
}

// Scratch words of the narrowphase (nkb_manifold.cuh): one world frame per collidable row and two polygon staging areas
// per warp that works on the env.
NKB_HOST_DEVICE inline uint32_t manifold_scratch_words(uint32_t B, uint32_t warps) { return 12u * B + 64u * warps; }

struct Config {
    float dt;
    float gravity[3];
    float pos_beta, pos_slop, contact_margin, baumgarte_max_velocity, overlap_recovery_velocity, velocity_tolerance;
    uint32_t vel_iters, pos_iters, max_contacts, max_pairs;
    uint32_t control_mode;      // 0 PD position, 1 torque, 2 velocity, 3 computed torque, 4 operational space, 5 actuator (reference phi/articulation_contract.hpp:16-23)
    uint32_t task_link;         // mode 4: the link that carries the task frame (nuka_world_desc_t.osc_task_link)
};

// Device pointers to the template tables (read-only during a step).
struct TemplateView {
    uint32_t L, B, ndof, max_depth, n_excluded, floating_root;
    uint32_t head_cap;          // solver heads per env held in shared memory
    uint32_t point_cap;         // contact points per env that get rows
    uint32_t slot_cap;          // candidate slots one step can fill: min(max_contacts, admissible pairs)
    const uint32_t *parent, *jtype, *depth, *child_begin, *children, *link_dof, *link_body, *geom_kind, *limit_flags;
    const uint32_t *dof_link, *anc_mask;
    const float *axis, *offset, *local_quat, *inertia10, *damping, *armature, *frictionloss, *stiffness, *spring_ref;
    const float *limit_lower, *limit_upper, *geom_pos, *geom_quat;
    const uint32_t *body_geom_kind;     // B: nonzero when the row's shape has its own frame in the link
    const float *body_geom_pos, *body_geom_quat;   // 3B, 4B
    const uint32_t *shape_kind, *contype, *conaffinity, *group, *body_to_link;
    const int32_t *body_id;
    const float *shape_params, *mu, *inv_mass, *inv_inertia, *inertial_pos, *inertial_quat;
    const unsigned long long *excluded;
    // body-row pairs (a << 16 | b, a < b, ascending) that pass the template-constant filters: not both
    // static, bitmask/group admitted, not excluded.  Only these need an AABB test each step.
    const uint32_t *adm_pairs;
    // the same admissibility as one bit row per body: bit b of row a (ceil(B / 32) words per row) for a < b
    const uint32_t *adm_mask;
    uint32_t broadphase_tree;           // 1: candidate pairs come from the per-env tree, 0: from the admissible-pair table
    const uint32_t *free_slot;         // B: slot of a free dynamic body in the solver's rigid-block arrays; others share slot n_free
    uint32_t n_free;
    uint32_t n_adm;
    Config cfg;
};

struct CacheEntry {             // one cached contact point (warm start)
    unsigned long long feature;
    uint32_t pair;              // (a << 16) | b, 0xffffffff when empty
    uint32_t age;
    float lambda[3];
    float normal[3];
};

// Device pointers to the per-env state, env-major.
struct StateView {
    uint32_t env_count;
    float *q, *qdot, *qddot, *tau, *actuator;                   // E x L
    float *base_pose;                                           // E x 7
    float *link_pose;                                           // E x L x 7
    float *link_vel;                                            // E x L x 6
    float *drive_target, *vel_target, *kp, *kd, *force_limit, *feedforward, *noload_speed, *acc_target;   // E x L
    float *body_pose;                                           // E x B x 7
    float *body_linvel, *body_angvel;                           // E x B x 3
    float *carry_artic;                                         // E x ndof  (solved - free velocity of the last step)
    float *carry_rigid;                                         // E x B x 6
    float *task_target, *task_rotation, *task_frame, *null_kp, *null_kd;   // E x 3, E x 4 (wxyz, zero = position only), E x 7 (xyz + wxyz on the task link), E, E: mode 4 inputs
    float *limit_lambda;                                        // E x L x 2  (joint-limit multipliers of the last velocity solve: lower, upper)
    CacheEntry *cache;                                          // E x S x 4
    uint32_t *status;                                           // E
    float *solver_residual;                                     // E x 4
    uint32_t *solver_sweeps;                                    // E
    // contact read-out (public CONTACT_* style fields and parity taps)
    uint32_t *pair_count;                                       // E
    uint32_t *pairs;                                            // E x S x 2
    uint32_t *contact_count;                                    // E x S
    float *contact_point, *contact_normal;                      // E x S x 4 x 3
    float *contact_depth;                                       // E x S x 4
    // optional parity taps (null unless requested)
    float *dbg_mass;                                            // E x ndof x ndof
    float *dbg_qdot_pseudo;                                     // E x ndof
    uint32_t *dbg_cycles;                                       // E x 32 stage cycle counters
};

// Shared-memory layout of one env (offsets in 4-byte words), filled by the host.
struct SmemLayout {
    uint32_t pose, xrot, xtr, vel, vbias, acc, pbias, ic;       // per link
    uint32_t mass, factor, vecs, vstride;                       // articulation (vstride: words per vector, 32 or 64)
    uint32_t bpose, bvel, bwinv, aabb, bmass, bfree, bpseudo;   // bodies
    uint32_t pairs, ccount, cpoint, cnormal, cdepth, cfeat;     // contacts
    uint32_t cstage;                                            // cache rebuild staging (shares the Jacobian pool, dead by then)
    uint32_t heads, jpool, binfo, chol, bm6;                    // solver (chol: Newton matrix; bm6: rigid block mass + head rows)
    uint32_t rjac, rjac_heads;                                  // staged Jacobian rows of one rigid block's heads (24 words each)
    // Team mode: `team` warps advance one env; warp 0 leads, the others wait for work (rigid blocks of one colour).
    // team_area: 12 command words, 4 result words per member, then helper_words of private Newton scratch per helper.
    uint32_t team, team_area, helper_words;
    // Fault drills for the team's bounded waits (tests only): bit 0 = the lead leaves without dismissing its helpers,
    // bit 1 = helpers never answer a command.  Either way every wait runs out, a status bit is set and the kernel ends.
    uint32_t team_drill;
    uint32_t words;                                             // total per env
    uint32_t ld;                                                // leading dimension of mass/factor (ndof | 1)
};

enum StepMode : uint32_t { kModeStep = 0, kModeDynamicsOnly = 1, kModeCollideOnly = 2, kModeRefresh = 3 };

struct StepParams {
    TemplateView t;
    StateView s;
    SmemLayout sm;
    uint32_t mode;
    uint32_t steps;
    // Env selection of a refresh launch (null: every env).  sel_ids lists sel_count envs, one warp each; sel_mask is
    // an E-word device array whose non-zero entries pick the envs of a full-size launch.
    const uint32_t* sel_ids;
    uint32_t sel_count;
    const uint32_t* sel_mask;
};

}  // namespace nkb

/*
 * C ABI of the B200-native batched articulated-robot step.
 *
 * The entry points, handle types, result codes, descriptor layouts and state-field ids below are the ones
 * the reference exposes for this path in src/include/nuka/nuka.h, so a caller bound to the reference's
 * world/step interface (C, C++ via nuka.hpp, or the Python module) can bind this library instead.
 * Each declaration cites the reference declaration it replaces.  Entry points of the reference outside the
 * step path (rendering, sensors, checkpoints, scene export, IK, telemetry) are not provided.
 *
 * Additions that have no counterpart in the reference are grouped at the end and prefixed nuka_b200_ or
 * documented as such.
 */
#ifndef NUKA_B200_H
#define NUKA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* nuka.h:11-12 opaque handles (integer ids in pointer clothing, as in src/c_abi/handle_table.hpp:13-60) */
typedef struct nuka_device_t* nuka_device_handle;
typedef struct nuka_world_t* nuka_world_handle;
typedef struct nuka_checkpoint_t* nuka_checkpoint_handle;     /* nuka.h:14 */

/* nuka.h:20 */
#define NUKA_MAX_CONTACT_SLOTS_PER_ENV 4u

/* nuka.h:22-32 */
typedef enum nuka_result_t {
    NUKA_RESULT_OK = 0,
    NUKA_RESULT_INVALID_ARG = 1,
    NUKA_RESULT_NULL_HANDLE = 2,
    NUKA_RESULT_CUDA_ERROR = 3,
    NUKA_RESULT_FILE_NOT_FOUND = 4,
    NUKA_RESULT_PARSE_ERROR = 5,
    NUKA_RESULT_OUT_OF_MEMORY = 6,
    NUKA_RESULT_NOT_SUPPORTED = 7,
    NUKA_RESULT_INTERNAL = 100
} nuka_result_t;

/* nuka.h:34-41 */
typedef struct nuka_version_t { uint16_t major, minor, patch; } nuka_version_t;
nuka_version_t nuka_get_version(void);
const char* nuka_result_message(nuka_result_t result);
/* nuka.h:42-44: thread-local text of the last failure; reading clears it. */
const char* nuka_last_error_message(void);

/* nuka.h:46-55 */
typedef struct nuka_device_desc_t {
    uint32_t gpu_index;
    void* cuda_stream;                 /* borrowed cudaStream_t, or NULL for an owned stream */
    uint8_t backend_selection_layer_enabled;
} nuka_device_desc_t;
nuka_result_t nuka_device_create(const nuka_device_desc_t* desc, nuka_device_handle* out);
void nuka_device_destroy(nuka_device_handle device);

/* nuka.h:57-173: same member order and types.  Members this library does not act on must be zero,
 * otherwise creation returns NUKA_RESULT_NOT_SUPPORTED (terrain/heightfield/curriculum, instancing,
 * cloth, OGC, substeps > 1). */
typedef struct nuka_world_desc_t {
    const char* scene_path;            /* path of a ".nks" scene file (cooked on load) or a ".nkt" cooked template file */
    uint32_t env_count;
    float fixed_dt;
    uint8_t determinism;               /* 0 or 1; larger values are INVALID_ARG */
    uint8_t control_mode;              /* 0 PD position, 1 torque, 2 velocity, 3 computed torque, 4 operational space, 5 actuator */
    uint32_t osc_task_link;            /* control mode 4: the link (index in the articulation) that carries the task frame; must be 0 in other modes */
    float terrain_step_height, terrain_step_width, terrain_platform_width, terrain_grid_width, terrain_grid_height_max;
    uint32_t instance_count;
    float instance_spacing;
    uint32_t contact_family;
    uint32_t heightfield_terrain_type, heightfield_nrow, heightfield_ncol;
    float heightfield_cell;
    const char* heightfield_image_path;
    float heightfield_radius_x, heightfield_radius_y, heightfield_elevation_z, heightfield_base_z;
    float gravity_x, gravity_y, gravity_z;   /* all zero selects (0, 0, -9.81) */
    uint32_t curric_levels, curric_types;
    float terrain_feature_cell;
    uint32_t solver_vel_iters;         /* 0 keeps the template's value */
    uint32_t solver_pos_iters;
    float solver_contact_margin;
    uint32_t solver_max_pairs;
    float solver_baumgarte_max_velocity;
    uint32_t cloth_integrator;
    uint32_t ogc_contact_capacity;
    float solver_overlap_recovery_velocity;
    uint32_t solver_substeps;
    uint32_t contact_detection_substeps;
} nuka_world_desc_t;

/* nuka.h:175 */
nuka_result_t nuka_world_create_from_scene(nuka_device_handle device, const nuka_world_desc_t* desc, nuka_world_handle* out);
/* nuka.h:253-255: step and step_n enqueue on the device stream and return before completion. */
void nuka_world_destroy(nuka_world_handle world);
nuka_result_t nuka_world_step(nuka_world_handle world);
nuka_result_t nuka_world_step_n(nuka_world_handle world, uint32_t step_count);

/* nuka.h:256-279 */
typedef enum nuka_execution_mode_t { NUKA_EXECUTION_EAGER = 0, NUKA_EXECUTION_GRAPH = 1 } nuka_execution_mode_t;
nuka_result_t nuka_world_set_execution_mode(nuka_world_handle world, nuka_execution_mode_t mode);
/* nuka.h:285 */
nuka_result_t nuka_world_set_gravity_z(nuka_world_handle world, float gravity_z);
/* nuka.h:289-290: 1..65535 */
nuka_result_t nuka_world_set_velocity_iterations(nuka_world_handle world, uint32_t iterations);
nuka_result_t nuka_world_get_velocity_iterations(nuka_world_handle world, uint32_t* out_iterations);
/* nuka.h:376 */
nuka_result_t nuka_world_synchronize(nuka_world_handle world);
/* nuka.h:380-385: reset keeps drive targets; an invalid id is INVALID_ARG with no env changed. */
nuka_result_t nuka_world_reset(nuka_world_handle world);
nuka_result_t nuka_world_reset_envs(nuka_world_handle world, const uint32_t* env_ids, uint32_t count);
/* nuka.h:387-404, src/c_abi/checkpoint.cpp:442-635.  A checkpoint holds the world's persistent state on the host
 * (coordinates, velocities, poses, carried constraint velocities, the contact cache, status words, drive targets and
 * gains) plus gravity, the velocity-iteration count and the number of steps taken.  capture synchronises the
 * world's stream.  restore accepts only a checkpoint of the same world (else INVALID_ARG), keeps every buffer-view
 * address, and refreshes link and body poses; contact read-out fields keep their last values until the next step.
 * A restored world repeats the steps that followed the capture bit for bit.
 * write/read use this library's own file layout (magic, layout hash, step count, byte count, bytes, host settings);
 * read validates the hash and byte count against the reading world (mismatch or a short file: INVALID_ARG) and
 * returns a checkpoint owned by that world.  equal compares layout, step count and bytes.  state_hash is FNV-1a 64
 * over the same bytes and settings in fixed order. */
nuka_result_t nuka_world_checkpoint_capture(nuka_world_handle world, nuka_checkpoint_handle* out);
nuka_result_t nuka_world_checkpoint_restore(nuka_world_handle world, nuka_checkpoint_handle checkpoint);
void nuka_checkpoint_destroy(nuka_checkpoint_handle checkpoint);
nuka_result_t nuka_checkpoint_write(nuka_checkpoint_handle checkpoint, const char* path);
nuka_result_t nuka_world_checkpoint_read(nuka_world_handle world, const char* path, nuka_checkpoint_handle* out);
nuka_result_t nuka_checkpoint_byte_size(nuka_checkpoint_handle checkpoint, uint64_t* out_bytes);
nuka_result_t nuka_checkpoint_equal(nuka_checkpoint_handle a, nuka_checkpoint_handle b, uint32_t* out_equal);
nuka_result_t nuka_world_state_hash(nuka_world_handle world, uint64_t* out_hash);
/* nuka.h:434 */
nuka_result_t nuka_world_forward_kinematics(nuka_world_handle world);
/* nuka.h:479-481 */
nuka_result_t nuka_world_get_stream(nuka_world_handle world, void** out_stream);
nuka_result_t nuka_world_record_event(nuka_world_handle world, void* cuda_event);

/* nuka.h:496-964: state field ids (values as in the reference) for the fields this path serves.  The reference's
 * CONTACT_POINTS (5) and CONTACT_NORMAL (17) views are not served; contacts are read through the tap fields below. */
typedef enum nuka_state_field_t {
    NUKA_FIELD_RIGID_BODY_TRANSFORM = 0,      /* E x B x 7 f32 */
    NUKA_FIELD_ARTICULATION_LINK_POSE = 1,    /* E x L x 7 f32 */
    NUKA_FIELD_JOINT_POSITION = 2,            /* E x L f32, slot 0 = root */
    NUKA_FIELD_JOINT_VELOCITY = 3,            /* E x L f32 */
    NUKA_FIELD_DRIVE_TARGET = 6,              /* E x L f32, writable */
    NUKA_FIELD_LINK_VELOCITY = 7,             /* E x L x 6 f32, angular first */
    NUKA_FIELD_DRIVE_STIFFNESS = 8,           /* E x L f32, writable */
    NUKA_FIELD_DRIVE_DAMPING = 9,
    NUKA_FIELD_DRIVE_FORCE_LIMIT = 10,
    NUKA_FIELD_BASE_POSE = 11,                /* E x 7 f32 */
    NUKA_FIELD_TORQUE_INPUT = 12,             /* E x L f32, writable; the same memory as DRIVE_TARGET (nuka.h:587-589) */
    NUKA_FIELD_VELOCITY_TARGET = 13,          /* E x L f32, writable */
    NUKA_FIELD_ACTUATOR_NOLOAD_SPEED = 14,    /* E x L f32, writable; actuator mode's torque-speed envelope, <= 0 disables it */
    NUKA_FIELD_JOINT_FEEDFORWARD = 22,        /* E x L f32, writable */
    NUKA_FIELD_ACCELERATION_TARGET = 56,      /* E x L f32, writable; computed-torque control's feed-forward acceleration */
    /* operational-space control (control_mode 4, nuka.h:596-598, 748-751, 789-790): one task per env on link osc_task_link.
       The task link's DRIVE_STIFFNESS / DRIVE_DAMPING are the task gains; joints off the chain from that link to the root
       hold DRIVE_TARGET through their own gains, joints on it through the nullspace gains.  Kept across resets. */
    NUKA_FIELD_TASK_TARGET = 15,              /* E x 3 f32, writable: world position the task frame reaches for */
    NUKA_FIELD_TASK_ROTATION_TARGET = 31,     /* E x 4 f32 (w, x, y, z), writable: world orientation; all zero = position-only task */
    NUKA_FIELD_TASK_LOCAL_POSE = 32,          /* E x 7 f32 (x, y, z, qw, qx, qy, qz), writable: the task frame on the task link */
    NUKA_FIELD_TASK_NULLSPACE_STIFFNESS = 57, /* E f32, writable */
    NUKA_FIELD_TASK_NULLSPACE_DAMPING = 58,   /* E f32, writable */
    NUKA_FIELD_BODY_LINEAR_VELOCITY = 25,     /* E x B x 3 f32 */
    NUKA_FIELD_BODY_ANGULAR_VELOCITY = 26,    /* E x B x 3 f32 */
    NUKA_FIELD_JOINT_LIMIT_IMPULSE = 27,      /* E x L x 2 f32, read-only: the multipliers (lower, upper) the latest velocity solve left on
                                                 each link's authored limit rows; the next step's limit rows start from them, as in the
                                                 reference, whose assembly clears only the slots of links without that limit
                                                 (src/phi/backend_cuda/ops/assemble_rows.cu:826-879); zeroed by a reset */
    NUKA_FIELD_ACTUATOR_EFFORT = 29,          /* E x L f32 */
    NUKA_FIELD_ENV_STATUS = 39,               /* E u32: sticky bits, the reference's (src/phi/op_schema.hpp:36-50): 1<<0 candidate
                                                 pairs dropped, 1<<2 coordinate overflow, 1<<5 free-rotation solve not converged
                                                 (of the latest step only: cleared before every body integration, as in the
                                                 reference), 1<<10 control input rejected, 1<<13 solver failure; this library's own: 1<<20 contact
                                                 points beyond the solver-row capacity dropped, 1<<21 a warp of an env's team gave
                                                 up waiting for another (the env's state is void) */
    NUKA_FIELD_SOLVER_RESIDUAL = 109,         /* E x 4 f32: normal, tangent, joint, momentum */
    /* fields without a counterpart in the reference's public enum (parity taps of this library) */
    NUKA_B200_FIELD_JOINT_ACCELERATION = 0x10000,   /* E x L f32 */
    NUKA_B200_FIELD_MASS_MATRIX = 0x10001,          /* E x n x n f32, filled by the dynamics stage when tapped */
    NUKA_B200_FIELD_PAIR_COUNT = 0x10002,           /* E u32 */
    NUKA_B200_FIELD_CANDIDATE_PAIRS = 0x10003,      /* E x S x 2 u32, ascending (a, b) */
    NUKA_B200_FIELD_CONTACT_COUNT = 0x10004,        /* E x S u32 */
    NUKA_B200_FIELD_CONTACT_POINT = 0x10005,        /* E x S x 4 x 3 f32 */
    NUKA_B200_FIELD_CONTACT_NORMAL = 0x10006,       /* E x S x 4 x 3 f32 */
    NUKA_B200_FIELD_CONTACT_DEPTH = 0x10007,        /* E x S x 4 f32 */
    NUKA_B200_FIELD_SOLVER_SWEEPS = 0x10008,        /* E u32 */
    NUKA_B200_FIELD_JOINT_PSEUDO_VELOCITY = 0x10009 /* E x n f32 */
} nuka_state_field_t;

/* nuka.h:1158-1166 */
typedef struct nuka_buffer_view_t {
    void* device_ptr;
    size_t element_count;
    uint32_t element_stride_bytes;
    uint8_t dtype;                     /* 0 f32, 1 u32, 2 u64, 3 u8 */
} nuka_buffer_view_t;
nuka_result_t nuka_world_get_buffer_view(nuka_world_handle world, nuka_state_field_t field, nuka_buffer_view_t* out);
/* nuka.h:1222-1234.  The name of link `link_index` (links of all envs in a row: index modulo links per env): the joint whose
 * child the link's body is, else the body's own name, as the scene file gives them.  A null `out` asks for the length
 * (*out_len, without the terminator); a buffer too small for name + NUL is INVALID_ARG with *out_len still set.
 * NOT_SUPPORTED for worlds whose template carries no names (the procedural templates). */
nuka_result_t nuka_world_get_dof_name(nuka_world_handle world, uint32_t link_index, char* out, size_t cap, size_t* out_len);
/* nuka.h:1180-1187: host <-> field byte transfer; out-of-range is INVALID_ARG, unknown field NOT_SUPPORTED. */
nuka_result_t nuka_world_upload_field(nuka_world_handle world, nuka_state_field_t field, const void* bytes, size_t nbytes, size_t byte_offset);
nuka_result_t nuka_world_download_field(nuka_world_handle world, nuka_state_field_t field, void* bytes, size_t nbytes, size_t byte_offset);

/* ---- additions (no counterpart in the reference) ---- */

/* Creates a world from an in-memory cooked template (".nkt" bytes).  The reference can only obtain
 * articulated templates by cooking scene files through importers that are outside this path. */
nuka_result_t nuka_world_create_from_template(nuka_device_handle device, const nuka_world_desc_t* desc,
                                              const void* template_bytes, size_t template_size, nuka_world_handle* out);

/* Parses a cooked template as world creation would and reports the same result code (OK, PARSE_ERROR for a malformed
 * or truncated container, NOT_SUPPORTED / INVALID_ARG for a model outside this path's limits), without a device. */
nuka_result_t nuka_b200_template_check(const void* template_bytes, size_t template_size);

/* Scene cooking.  nuka_world_create_from_scene (above) takes the reference's scene file: when scene_path holds a `.nks`
 * document (JSON, src/scene/format/nks.cpp) the library cooks it as the reference's cooker does for the part this path
 * covers (src/scene/cook/cook_to_model.cpp: one articulated tree of revolute / prismatic / fixed joints under a free or
 * static root, sphere / capsule / box shapes, free rigid bodies, ground planes, position actuators as drives, the scene's
 * contype / conaffinity bits, one candidate slot per admissible pair), with fixed_dt and the solver iteration counts of
 * the descriptor; anything else in the scene gives NUKA_RESULT_NOT_SUPPORTED with a message, malformed JSON
 * NUKA_RESULT_PARSE_ERROR.  A cooked template file (`.nkt`) loads as is.
 * nuka_b200_scene_cook exposes the cooker itself (no device needed): scene text in, cooked template bytes out.  Call it
 * with out = NULL to learn the size.  The options default (nuka_b200_cook_options_defaults) to what create_from_scene
 * uses; the other settings serve callers that want a robot-versus-ground template from a scene that has no ground or
 * actuators of its own. */
typedef struct nuka_b200_cook_options_t {
    float dt;
    uint32_t velocity_iterations, position_iterations;
    float default_kp, default_kd;       /* drive gains of scalar joints without an actuator (0 = undriven) */
    uint32_t add_default_ground;        /* add a plane at ground_height when the scene has none */
    float ground_height, ground_mu;
    uint32_t self_collision;            /* robot rows keep their contype / conaffinity (else: they meet the ground only) */
    uint32_t scene_filters;             /* every row keeps the scene's bits, the ground's included; implies self_collision */
    uint32_t max_contacts;              /* candidate slots per env: 0 = one per shape row, 0xffffffff = every admissible pair */
    uint32_t max_points;                /* contact points per env with solver rows: 0 = derived bound, at most 128 */
} nuka_b200_cook_options_t;
void nuka_b200_cook_options_defaults(nuka_b200_cook_options_t* options);
nuka_result_t nuka_b200_scene_cook(const char* scene_json, size_t scene_size, const nuka_b200_cook_options_t* options, void* out,
                                   size_t capacity, size_t* out_size);

typedef struct nuka_b200_world_info_t {
    uint32_t env_count, links_per_env, bodies_per_env, dofs_per_env, contact_slots_per_env;
    uint32_t shared_bytes_per_env, warps_per_block;
    float fixed_dt;                 /* the step the world integrates with (desc->fixed_dt, else the template's) */
} nuka_b200_world_info_t;
nuka_result_t nuka_b200_world_info(nuka_world_handle world, nuka_b200_world_info_t* out);

/* Runs one pipeline stage for per-stage parity checks: 1 = kinematics + drives + dynamics without the
 * velocity update (fills JOINT_ACCELERATION and MASS_MATRIX), 2 = collision only (fills the contact taps). */
nuka_result_t nuka_b200_world_run_stage(nuka_world_handle world, uint32_t stage);

/* Kernel launches enqueued by this world since creation (for throughput reports). */
nuka_result_t nuka_b200_world_launch_count(nuka_world_handle world, uint64_t* out);

/* The observation record of the reference's gym layer, python/nuka/tasks/go2_obs.py:11-20 and :282-305
 * (Go2ObsBuilder.compute_obs), composed by one kernel on the world's stream instead of a chain of tensor ops.  For a
 * floating-base robot with nj = L - 1 actuated joints a record holds, in order:
 *     base linear velocity (base frame) x lin_vel_scale      3      (reference scale 2.0)
 *     base angular velocity (base frame) x ang_vel_scale     3      (0.25)
 *     world (0, 0, -1) rotated into the base frame           3
 *     command x command_scale                                3      ((2.0, 2.0, 0.25))
 *     (q - default_position) x dof_pos_scale                 nj     (1.0), joints in the caller's order
 *     qdot x dof_vel_scale                                   nj     (0.05), joints in the caller's order
 *     last_action                                            nj
 * every value clipped to [-clip, clip] (100), i.e. 12 + 3 nj floats: 48 for a 12-joint quadruped.  With `reward`
 * non-null its value follows the record unclipped, for callers that exchange observation + reward in one buffer.
 * All pointers are device memory read on the world's stream.  Zero-initialise the struct and call
 * nuka_b200_observation_desc_defaults for the reference's scales. */
typedef struct nuka_b200_observation_desc_t {
    const float* command;            /* E x 3, or 3 floats for every env when command_stride is 0 */
    uint32_t command_stride;         /* floats between consecutive envs' commands: 0 or >= 3 */
    const float* last_action;        /* E x nj, NULL = zeros */
    const float* default_position;   /* nj in the caller's joint order, NULL = zeros */
    const uint32_t* joint_order;     /* nj: library joint slot (0-based; slot j is link j + 1) read for the caller's joint i; NULL = identity.
                                        The reference's table of the same meaning is urdf_from_nuka_slot, go2_obs.py:252-262 */
    const float* reward;             /* E, NULL = no reward column */
    float lin_vel_scale, ang_vel_scale, dof_pos_scale, dof_vel_scale;
    float command_scale[3];
    float clip;
    uint32_t row_stride;             /* floats between consecutive records in device_out; 0 = the record width */
} nuka_b200_observation_desc_t;
void nuka_b200_observation_desc_defaults(nuka_b200_observation_desc_t* desc);
/* Writes E records into device_out (caller-owned device memory, e.g. this rank's slice of a gather buffer).
 * device_out == NULL only reports the record width (without the reward column) in *out_width.
 * NUKA_ERR_NOT_SUPPORTED for worlds without a floating-base articulation, INVALID_ARG for a null command, a stride
 * below the record width or a buffer that is too small. */
nuka_result_t nuka_b200_world_pack_observations(nuka_world_handle world, const nuka_b200_observation_desc_t* desc,
                                                float* device_out, size_t capacity_floats, uint32_t* out_width);

/* nuka_world_reset_envs (nuka.h:380-385) with the env set chosen on the device: resets every env whose word in
 * device_mask (E x u32 device memory, read on the world's stream) is non-zero and recomputes their derived poses.
 * Nothing crosses to the host and nothing synchronises, so an episode loop can chain step, termination test and
 * reset on one stream (the reference's gym layer downloads the done ids first, python/nuka/gym/env.py autoreset). */
nuka_result_t nuka_b200_world_reset_envs_masked(nuka_world_handle world, const uint32_t* device_mask);

/* Route of the candidate-pair stage (the reference has the same two: a per-env LBVH, src/collision/lbvh_batched.cuh, and an
 * all-pairs pass for small scenes, ops/broadphase.cu:404-474).  0: chosen by the size of the template's admissible-pair
 * table (the default), 1: the table, 2: the per-env tree.  The pair list is the same either way. */
nuka_result_t nuka_b200_world_set_broadphase(nuka_world_handle world, uint32_t mode);

/* Switches the per-step contact read-out arrays (PAIR_COUNT ... CONTACT_DEPTH below) on (non-zero, the default) or
 * off.  While off the step skips those stores and the arrays keep their last contents. */
nuka_result_t nuka_b200_world_set_contact_readout(nuka_world_handle world, uint32_t enabled);

/* No counterpart in the reference.  nuka_world_reset_envs without any allocation: same validation, set semantics and
 * resulting state, but the env-id list goes through a fixed 16 KB device array built into the library instead of a
 * buffer the world allocates on demand.  Meant for callers that cannot allocate once their episode loop runs: a
 * training process whose framework allocator already owns the rest of the device memory (an allocation for the id
 * list could then fail mid-run), and control loops that cannot afford the device-wide stall an allocation implies.
 *  - at most NUKA_B200_STATIC_RESET_MAX_IDS ids per call (counted before de-duplication); more is
 *    NUKA_ERR_INVALID_ARG and nothing changes;
 *  - the first call on a device also looks up the array's device address; make that first call during set-up,
 *    before any stream capture is started;
 *  - nothing in the array needs clearing: each call overwrites the ids it is about to read;
 *  - all worlds on one device share the array, so two calls must not be in flight at the same time on that device
 *    (different worlds, streams or threads): they would race on the id list.  A call returns after its ids have
 *    been consumed, so calls issued one after another from one thread are safe. */
#define NUKA_B200_STATIC_RESET_MAX_IDS 4096u
nuka_result_t nuka_b200_world_reset_envs_static(nuka_world_handle world, const uint32_t* env_ids, uint32_t count);

#ifdef __cplusplus
}
#endif
#endif

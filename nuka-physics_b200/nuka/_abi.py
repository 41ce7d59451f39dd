"""ctypes declarations of the C ABI (include/nuka_b200.h).  The native library is mandatory: there is no
Python or CPU fallback for the step."""
import ctypes
import os

from . import _build

OK, INVALID_ARG, NULL_HANDLE, CUDA_ERROR, FILE_NOT_FOUND, PARSE_ERROR, OUT_OF_MEMORY, NOT_SUPPORTED, INTERNAL = 0, 1, 2, 3, 4, 5, 6, 7, 100


class DeviceDesc(ctypes.Structure):
    _fields_ = [("gpu_index", ctypes.c_uint32), ("cuda_stream", ctypes.c_void_p), ("backend_selection_layer_enabled", ctypes.c_uint8)]


class WorldDesc(ctypes.Structure):
    _fields_ = [
        ("scene_path", ctypes.c_char_p), ("env_count", ctypes.c_uint32), ("fixed_dt", ctypes.c_float),
        ("determinism", ctypes.c_uint8), ("control_mode", ctypes.c_uint8), ("osc_task_link", ctypes.c_uint32),
        ("terrain_step_height", ctypes.c_float), ("terrain_step_width", ctypes.c_float), ("terrain_platform_width", ctypes.c_float),
        ("terrain_grid_width", ctypes.c_float), ("terrain_grid_height_max", ctypes.c_float),
        ("instance_count", ctypes.c_uint32), ("instance_spacing", ctypes.c_float), ("contact_family", ctypes.c_uint32),
        ("heightfield_terrain_type", ctypes.c_uint32), ("heightfield_nrow", ctypes.c_uint32), ("heightfield_ncol", ctypes.c_uint32),
        ("heightfield_cell", ctypes.c_float), ("heightfield_image_path", ctypes.c_char_p),
        ("heightfield_radius_x", ctypes.c_float), ("heightfield_radius_y", ctypes.c_float),
        ("heightfield_elevation_z", ctypes.c_float), ("heightfield_base_z", ctypes.c_float),
        ("gravity_x", ctypes.c_float), ("gravity_y", ctypes.c_float), ("gravity_z", ctypes.c_float),
        ("curric_levels", ctypes.c_uint32), ("curric_types", ctypes.c_uint32), ("terrain_feature_cell", ctypes.c_float),
        ("solver_vel_iters", ctypes.c_uint32), ("solver_pos_iters", ctypes.c_uint32), ("solver_contact_margin", ctypes.c_float),
        ("solver_max_pairs", ctypes.c_uint32), ("solver_baumgarte_max_velocity", ctypes.c_float), ("cloth_integrator", ctypes.c_uint32),
        ("ogc_contact_capacity", ctypes.c_uint32), ("solver_overlap_recovery_velocity", ctypes.c_float),
        ("solver_substeps", ctypes.c_uint32), ("contact_detection_substeps", ctypes.c_uint32),
    ]


class BufferView(ctypes.Structure):
    _fields_ = [("device_ptr", ctypes.c_void_p), ("element_count", ctypes.c_size_t), ("element_stride_bytes", ctypes.c_uint32), ("dtype", ctypes.c_uint8)]


class WorldInfo(ctypes.Structure):
    _fields_ = [(n, ctypes.c_uint32) for n in ("env_count", "links_per_env", "bodies_per_env", "dofs_per_env", "contact_slots_per_env",
                                                "shared_bytes_per_env", "warps_per_block")] + [("fixed_dt", ctypes.c_float)]


class ObservationDesc(ctypes.Structure):
    _fields_ = [("command", ctypes.c_void_p), ("command_stride", ctypes.c_uint32), ("last_action", ctypes.c_void_p),
                ("default_position", ctypes.c_void_p), ("joint_order", ctypes.c_void_p), ("reward", ctypes.c_void_p),
                ("lin_vel_scale", ctypes.c_float), ("ang_vel_scale", ctypes.c_float), ("dof_pos_scale", ctypes.c_float),
                ("dof_vel_scale", ctypes.c_float), ("command_scale", ctypes.c_float * 3), ("clip", ctypes.c_float),
                ("row_stride", ctypes.c_uint32)]


class CookOptions(ctypes.Structure):
    _fields_ = [("dt", ctypes.c_float), ("velocity_iterations", ctypes.c_uint32), ("position_iterations", ctypes.c_uint32),
                ("default_kp", ctypes.c_float), ("default_kd", ctypes.c_float), ("add_default_ground", ctypes.c_uint32),
                ("ground_height", ctypes.c_float), ("ground_mu", ctypes.c_float), ("self_collision", ctypes.c_uint32),
                ("scene_filters", ctypes.c_uint32), ("max_contacts", ctypes.c_uint32), ("max_points", ctypes.c_uint32)]


EXPORTS = [
    "nuka_get_version", "nuka_result_message", "nuka_last_error_message", "nuka_device_create", "nuka_device_destroy",
    "nuka_world_create_from_scene", "nuka_world_destroy", "nuka_world_step", "nuka_world_step_n", "nuka_world_set_execution_mode",
    "nuka_world_set_gravity_z", "nuka_world_set_velocity_iterations", "nuka_world_get_velocity_iterations", "nuka_world_synchronize",
    "nuka_world_reset", "nuka_world_reset_envs", "nuka_world_forward_kinematics", "nuka_world_get_stream", "nuka_world_record_event",
    "nuka_world_get_buffer_view", "nuka_world_upload_field", "nuka_world_download_field", "nuka_world_create_from_template",
    "nuka_b200_world_info", "nuka_b200_world_run_stage", "nuka_b200_world_launch_count", "nuka_b200_world_reset_envs_static",
    "nuka_b200_world_pack_observations", "nuka_b200_observation_desc_defaults", "nuka_b200_world_reset_envs_masked",
    "nuka_b200_world_set_contact_readout", "nuka_b200_world_set_broadphase", "nuka_b200_template_check", "nuka_b200_cook_options_defaults", "nuka_b200_scene_cook", "nuka_world_checkpoint_capture", "nuka_world_checkpoint_restore", "nuka_checkpoint_destroy",
    "nuka_checkpoint_write", "nuka_world_checkpoint_read", "nuka_checkpoint_byte_size", "nuka_checkpoint_equal", "nuka_world_state_hash",
    "nuka_world_get_dof_name",
]

_LIB = None


def lib():
    """Loads libnuka_b200.so (building it first when the sources are newer)."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = os.environ.get("NUKA_B200_LIBRARY") or _build.LIB_PATH       # the variable selects an alternative build of the library
    if not os.path.exists(path):
        path = _build.build_native()
    L = ctypes.CDLL(path)
    vp, u32, sz = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_size_t
    L.nuka_result_message.restype = ctypes.c_char_p
    L.nuka_result_message.argtypes = [ctypes.c_int]
    L.nuka_last_error_message.restype = ctypes.c_char_p
    L.nuka_device_create.argtypes = [ctypes.POINTER(DeviceDesc), ctypes.POINTER(vp)]
    L.nuka_device_destroy.argtypes = [vp]
    L.nuka_device_destroy.restype = None
    L.nuka_world_create_from_scene.argtypes = [vp, ctypes.POINTER(WorldDesc), ctypes.POINTER(vp)]
    L.nuka_world_create_from_template.argtypes = [vp, ctypes.POINTER(WorldDesc), ctypes.c_char_p, sz, ctypes.POINTER(vp)]
    L.nuka_world_destroy.argtypes = [vp]
    L.nuka_world_destroy.restype = None
    L.nuka_world_step.argtypes = [vp]
    L.nuka_world_step_n.argtypes = [vp, u32]
    L.nuka_world_set_execution_mode.argtypes = [vp, ctypes.c_int]
    L.nuka_world_set_gravity_z.argtypes = [vp, ctypes.c_float]
    L.nuka_world_set_velocity_iterations.argtypes = [vp, u32]
    L.nuka_world_get_velocity_iterations.argtypes = [vp, ctypes.POINTER(u32)]
    L.nuka_world_synchronize.argtypes = [vp]
    L.nuka_world_reset.argtypes = [vp]
    L.nuka_world_reset_envs.argtypes = [vp, ctypes.POINTER(u32), u32]
    L.nuka_b200_world_reset_envs_static.argtypes = [vp, ctypes.POINTER(u32), u32]
    L.nuka_b200_world_pack_observations.argtypes = [vp, ctypes.POINTER(ObservationDesc), vp, sz, ctypes.POINTER(u32)]
    L.nuka_b200_observation_desc_defaults.argtypes = [ctypes.POINTER(ObservationDesc)]
    L.nuka_b200_observation_desc_defaults.restype = None
    L.nuka_b200_world_reset_envs_masked.argtypes = [vp, vp]
    L.nuka_b200_cook_options_defaults.argtypes = [ctypes.POINTER(CookOptions)]
    L.nuka_b200_cook_options_defaults.restype = None
    L.nuka_b200_scene_cook.argtypes = [ctypes.c_char_p, sz, ctypes.POINTER(CookOptions), vp, sz, ctypes.POINTER(sz)]
    L.nuka_b200_world_set_contact_readout.argtypes = [vp, u32]
    L.nuka_b200_world_set_broadphase.argtypes = [vp, u32]
    L.nuka_world_forward_kinematics.argtypes = [vp]
    L.nuka_world_get_stream.argtypes = [vp, ctypes.POINTER(vp)]
    L.nuka_world_record_event.argtypes = [vp, vp]
    L.nuka_world_get_buffer_view.argtypes = [vp, ctypes.c_int, ctypes.POINTER(BufferView)]
    L.nuka_world_get_dof_name.argtypes = [vp, ctypes.c_uint32, ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]
    L.nuka_world_upload_field.argtypes = [vp, ctypes.c_int, vp, sz, sz]
    L.nuka_world_download_field.argtypes = [vp, ctypes.c_int, vp, sz, sz]
    L.nuka_b200_world_info.argtypes = [vp, ctypes.POINTER(WorldInfo)]
    L.nuka_b200_world_run_stage.argtypes = [vp, u32]
    L.nuka_b200_world_launch_count.argtypes = [vp, ctypes.POINTER(ctypes.c_uint64)]
    L.nuka_world_checkpoint_capture.argtypes = [vp, ctypes.POINTER(vp)]
    L.nuka_world_checkpoint_restore.argtypes = [vp, vp]
    L.nuka_checkpoint_destroy.argtypes = [vp]
    L.nuka_checkpoint_destroy.restype = None
    L.nuka_checkpoint_write.argtypes = [vp, ctypes.c_char_p]
    L.nuka_world_checkpoint_read.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(vp)]
    L.nuka_checkpoint_byte_size.argtypes = [vp, ctypes.POINTER(ctypes.c_uint64)]
    L.nuka_checkpoint_equal.argtypes = [vp, vp, ctypes.POINTER(u32)]
    L.nuka_world_state_hash.argtypes = [vp, ctypes.POINTER(ctypes.c_uint64)]
    _LIB = L
    return L

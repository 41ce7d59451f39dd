"""B200-native batched articulated-robot step behind the reference's world/step interface.

The surface mirrors the reference's Python module for this path (python/nuka/__init__.py:27-101,
python/src/nuka_ext.cpp:2546-2600): ``Device.create``, ``World.create_from_scene`` / ``step`` / ``step_n`` /
``synchronize`` / ``reset`` / ``reset_envs`` / ``view`` / ``set_velocity_iterations``; ``FieldView`` exposes
world-owned device memory without a copy (``__cuda_array_interface__`` and ``__dlpack__``).
Every call goes through the C ABI of ``libnuka_b200.so``; nothing here computes physics.
"""
import ctypes
import os
import enum

import numpy as np

from . import _abi, nkt, templates  # noqa: F401


class NukaError(RuntimeError):
    def __init__(self, code, message):
        super().__init__(f"{_abi.lib().nuka_result_message(code).decode()} ({code}): {message}")
        self.code = code


def _check(code):
    if code != _abi.OK:
        raise NukaError(code, _abi.lib().nuka_last_error_message().decode())


class Field(enum.IntEnum):
    """State field ids (reference nuka.h:496-964) plus this library's parity taps."""
    RIGID_BODY_TRANSFORM = 0
    ARTICULATION_LINK_POSE = 1
    JOINT_POSITION = 2
    JOINT_VELOCITY = 3
    DRIVE_TARGET = 6
    LINK_VELOCITY = 7
    DRIVE_STIFFNESS = 8
    DRIVE_DAMPING = 9
    DRIVE_FORCE_LIMIT = 10
    BASE_POSE = 11
    TORQUE_INPUT = 12
    VELOCITY_TARGET = 13
    ACTUATOR_NOLOAD_SPEED = 14
    TASK_TARGET = 15
    JOINT_FEEDFORWARD = 22
    ACCELERATION_TARGET = 56
    TASK_NULLSPACE_STIFFNESS = 57
    TASK_NULLSPACE_DAMPING = 58
    BODY_LINEAR_VELOCITY = 25
    BODY_ANGULAR_VELOCITY = 26
    JOINT_LIMIT_IMPULSE = 27
    TASK_ROTATION_TARGET = 31
    TASK_LOCAL_POSE = 32
    ACTUATOR_EFFORT = 29
    ENV_STATUS = 39
    SOLVER_RESIDUAL = 109
    JOINT_ACCELERATION = 0x10000
    MASS_MATRIX = 0x10001
    PAIR_COUNT = 0x10002
    CANDIDATE_PAIRS = 0x10003
    CONTACT_COUNT = 0x10004
    CONTACT_POINT = 0x10005
    CONTACT_NORMAL = 0x10006
    CONTACT_DEPTH = 0x10007
    SOLVER_SWEEPS = 0x10008
    JOINT_PSEUDO_VELOCITY = 0x10009
    STAGE_CYCLES = 0x1000A      # served only by a library built with NUKA_B200_STAGE_TAPS=1 (profiling builds)


class Device:
    def __init__(self, handle, gpu_index):
        self._h = handle
        self.gpu_index = gpu_index

    @classmethod
    def create(cls, gpu_index=0, cuda_stream=None):
        desc = _abi.DeviceDesc(gpu_index, cuda_stream, 0)
        out = ctypes.c_void_p()
        _check(_abi.lib().nuka_device_create(ctypes.byref(desc), ctypes.byref(out)))
        return cls(out, gpu_index)

    def destroy(self):
        if self._h:
            _abi.lib().nuka_device_destroy(self._h)
            self._h = None


class FieldView:
    """Borrowed view of a world-owned device buffer; valid until the world is destroyed."""

    def __init__(self, world, field, view):
        self._world = world
        self.field = Field(field)
        self.device_ptr = view.device_ptr
        self.element_count = view.element_count
        self.dtype = np.dtype(np.float32 if view.dtype == 0 else np.uint32)
        self.shape = (world.env_count, view.element_count // world.env_count)

    @property
    def __cuda_array_interface__(self):
        return {"shape": self.shape, "typestr": self.dtype.str, "data": (self.device_ptr, False), "version": 3, "strides": None}

    def torch(self):
        import torch
        return torch.as_tensor(self, device=f"cuda:{self._world.device.gpu_index}")

    def __dlpack__(self, stream=None):
        return self.torch().__dlpack__(stream=stream)

    def __dlpack_device__(self):
        return (2, self._world.device.gpu_index)   # kDLCUDA


class Checkpoint:
    """A captured world state (reference nuka.h:387-404)."""

    def __init__(self, handle):
        self._h = handle

    def write(self, path):
        _check(_abi.lib().nuka_checkpoint_write(self._h, os.fsencode(path)))

    @property
    def byte_size(self):
        out = ctypes.c_uint64()
        _check(_abi.lib().nuka_checkpoint_byte_size(self._h, ctypes.byref(out)))
        return out.value

    def __eq__(self, other):
        if not isinstance(other, Checkpoint):
            return NotImplemented
        out = ctypes.c_uint32()
        _check(_abi.lib().nuka_checkpoint_equal(self._h, other._h, ctypes.byref(out)))
        return bool(out.value)

    __hash__ = None

    def destroy(self):
        if self._h:
            _abi.lib().nuka_checkpoint_destroy(self._h)
            self._h = None


class World:
    def __init__(self, device, handle, env_count):
        self.device = device
        self._h = handle
        self.env_count = env_count
        info = _abi.WorldInfo()
        _check(_abi.lib().nuka_b200_world_info(self._h, ctypes.byref(info)))
        self.info = info

    @staticmethod
    def _desc(scene_path, env_count, dt, determinism, control_mode, **solver):
        d = _abi.WorldDesc()
        d.scene_path = scene_path.encode() if scene_path else None
        d.env_count, d.fixed_dt, d.determinism, d.control_mode = env_count, dt, determinism, control_mode
        for k, v in solver.items():
            setattr(d, k, v)
        return d

    @classmethod
    def create_from_scene(cls, device, scene_path, env_count, dt=0.0, determinism=0, control_mode=0, **solver):
        d = cls._desc(scene_path, env_count, dt, determinism, control_mode, **solver)
        out = ctypes.c_void_p()
        _check(_abi.lib().nuka_world_create_from_scene(device._h, ctypes.byref(d), ctypes.byref(out)))
        return cls(device, out, env_count)

    @classmethod
    def create_from_template(cls, device, blob, env_count, dt=0.0, determinism=0, control_mode=0, **solver):
        d = cls._desc(None, env_count, dt, determinism, control_mode, **solver)
        out = ctypes.c_void_p()
        blob = bytes(blob)
        _check(_abi.lib().nuka_world_create_from_template(device._h, ctypes.byref(d), blob, len(blob), ctypes.byref(out)))
        return cls(device, out, env_count)

    def destroy(self):
        if self._h:
            _abi.lib().nuka_world_destroy(self._h)
            self._h = None

    def step(self):
        _check(_abi.lib().nuka_world_step(self._h))

    def step_n(self, n):
        _check(_abi.lib().nuka_world_step_n(self._h, n))

    def synchronize(self):
        _check(_abi.lib().nuka_world_synchronize(self._h))

    def reset(self):
        _check(_abi.lib().nuka_world_reset(self._h))

    def reset_envs(self, env_ids):
        ids = np.ascontiguousarray(env_ids, dtype=np.uint32)
        _check(_abi.lib().nuka_world_reset_envs(self._h, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), ids.size))

    def observation_width(self):
        """Floats per observation record (12 + 3 x actuated joints; 48 for a 12-joint quadruped), reward column excluded."""
        width = ctypes.c_uint32()
        _check(_abi.lib().nuka_b200_world_pack_observations(self._h, None, None, 0, ctypes.byref(width)))
        return width.value

    def observation_desc(self, command, last_action=None, default_position=None, joint_order=None, reward=None, row_stride=0):
        """Descriptor of the reference's observation record (python/nuka/tasks/go2_obs.py:11-20) with its scales; the
        arguments are CUDA tensors (command: 3 floats for every env, or E x 3) that must outlive the pack calls."""
        d = _abi.ObservationDesc()
        _abi.lib().nuka_b200_observation_desc_defaults(ctypes.byref(d))
        d.command = command.data_ptr()
        d.command_stride = 0 if command.numel() == 3 else int(command.stride(0))
        for name, value in (("last_action", last_action), ("default_position", default_position), ("joint_order", joint_order), ("reward", reward)):
            setattr(d, name, value.data_ptr() if value is not None else None)
        d.row_stride = int(row_stride)
        d._keep = (command, last_action, default_position, joint_order, reward)
        return d

    def pack_observations(self, desc, out):
        """Writes one record per env into `out` (CUDA float32 tensor, row stride desc.row_stride or the record width) on the world's stream."""
        _check(_abi.lib().nuka_b200_world_pack_observations(self._h, ctypes.byref(desc), ctypes.c_void_p(out.data_ptr()), out.numel(), None))

    def reset_envs_masked(self, mask):
        """Resets the envs whose word in `mask` (CUDA tensor of E 32-bit words) is non-zero; stays on the world's stream, no host sync."""
        _check(_abi.lib().nuka_b200_world_reset_envs_masked(self._h, ctypes.c_void_p(mask.data_ptr())))

    def set_broadphase(self, mode):
        """0: by the size of the admissible-pair table, 1: the table, 2: the per-env tree (same pair list either way)."""
        _check(_abi.lib().nuka_b200_world_set_broadphase(self._h, int(mode)))

    def set_contact_readout(self, enabled):
        _check(_abi.lib().nuka_b200_world_set_contact_readout(self._h, 1 if enabled else 0))

    def reset_envs_static(self, env_ids):
        """reset_envs without any allocation (at most 4096 ids per call; calls on one device must not overlap)."""
        ids = np.ascontiguousarray(env_ids, dtype=np.uint32)
        _check(_abi.lib().nuka_b200_world_reset_envs_static(self._h, ids.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), ids.size))

    def checkpoint_capture(self):
        """Host copy of the persistent state and settings (reference nuka.h:389); synchronises the stream."""
        h = ctypes.c_void_p()
        _check(_abi.lib().nuka_world_checkpoint_capture(self._h, ctypes.byref(h)))
        return Checkpoint(h)

    def checkpoint_restore(self, checkpoint):
        _check(_abi.lib().nuka_world_checkpoint_restore(self._h, checkpoint._h))

    def checkpoint_read(self, path):
        h = ctypes.c_void_p()
        _check(_abi.lib().nuka_world_checkpoint_read(self._h, os.fsencode(path), ctypes.byref(h)))
        return Checkpoint(h)

    def state_hash(self):
        out = ctypes.c_uint64()
        _check(_abi.lib().nuka_world_state_hash(self._h, ctypes.byref(out)))
        return out.value

    def forward_kinematics(self):
        _check(_abi.lib().nuka_world_forward_kinematics(self._h))

    def set_velocity_iterations(self, n):
        _check(_abi.lib().nuka_world_set_velocity_iterations(self._h, n))

    def get_velocity_iterations(self):
        out = ctypes.c_uint32()
        _check(_abi.lib().nuka_world_get_velocity_iterations(self._h, ctypes.byref(out)))
        return out.value

    def set_execution_mode(self, graph):
        _check(_abi.lib().nuka_world_set_execution_mode(self._h, 1 if graph else 0))

    def run_stage(self, stage):
        _check(_abi.lib().nuka_b200_world_run_stage(self._h, stage))

    def dof_names(self):
        """Names of one env's links in link order (reference python/nuka: World.dof_names): the joint whose child the link
        is, else the body's name; the root's is usually empty or the trunk's."""
        names = []
        for link in range(self.info.links_per_env):
            need = ctypes.c_size_t()
            _check(_abi.lib().nuka_world_get_dof_name(self._h, link, None, 0, ctypes.byref(need)))
            buf = ctypes.create_string_buffer(need.value + 1)
            _check(_abi.lib().nuka_world_get_dof_name(self._h, link, buf, need.value + 1, ctypes.byref(need)))
            names.append(buf.value.decode())
        return names

    def dof_index(self, pattern):
        """Link columns whose name matches the regular expression `pattern` (int32 array, possibly empty), as the reference's
        World.dof_index (python/src/nuka_ext.cpp:3014-3048): a leading 'entity/' is dropped, unnamed links never match.
        Index the per-link buffers with it: ``targets[:, world.dof_index("thigh")]``."""
        import re
        expr = re.compile(pattern.rsplit("/", 1)[-1])
        return np.array([k for k, name in enumerate(self.dof_names()) if name and expr.search(name)], dtype=np.int32)

    @property
    def base_link_count(self):
        """Links per env; the per-link buffers are this wide, slot 0 is the root (nuka_ext.cpp:2772)."""
        return self.info.links_per_env

    @property
    def action_dim(self):
        """Actuated joint columns a policy controls: base_link_count - 1 (nuka_ext.cpp:2777-2783)."""
        return self.info.links_per_env - 1

    def set_drive_targets(self, values):
        """Writes all env_count x base_link_count drive targets from a flat host array (nuka_ext.cpp:3120-3140)."""
        values = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
        if values.size != self.env_count * self.info.links_per_env:
            raise ValueError(f"set_drive_targets: array length {values.size} != DRIVE_TARGET count {self.env_count * self.info.links_per_env}")
        self.upload(Field.DRIVE_TARGET, values.reshape(self.env_count, -1))

    def launch_count(self):
        out = ctypes.c_uint64()
        _check(_abi.lib().nuka_b200_world_launch_count(self._h, ctypes.byref(out)))
        return out.value

    def view(self, field):
        v = _abi.BufferView()
        _check(_abi.lib().nuka_world_get_buffer_view(self._h, int(field), ctypes.byref(v)))
        return FieldView(self, field, v)

    def upload(self, field, array, byte_offset=0):
        a = np.ascontiguousarray(array)
        _check(_abi.lib().nuka_world_upload_field(self._h, int(field), a.ctypes.data, a.nbytes, byte_offset))

    def download(self, field):
        v = self.view(field)
        out = np.zeros(v.shape, dtype=v.dtype)
        _check(_abi.lib().nuka_world_download_field(self._h, int(field), out.ctypes.data, out.nbytes, 0))
        return out


def sync(world):
    world.synchronize()

"""The allocation-free partial reset against nuka_world_reset_envs, through the C ABI, on two calls in a row."""
import ctypes

import numpy as np
import pytest

import nuka
from nuka import Field as F, _abi, templates as T

pytestmark = pytest.mark.gpu

FIELDS = (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.LINK_VELOCITY, F.ARTICULATION_LINK_POSE, F.RIGID_BODY_TRANSFORM,
          F.ENV_STATUS, F.DRIVE_TARGET)


def _state(w):
    return [w.download(f).tobytes() for f in FIELDS]


def _pair(device, E):
    blob = T.quadruped(0).blob()
    st = T.quadruped_state(E, 5)
    worlds = []
    for _ in range(2):
        w = nuka.World.create_from_template(device, blob, E)
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
        w.step_n(6)
        worlds.append(w)
    assert _state(worlds[0]) == _state(worlds[1])
    return worlds


def test_static_reset_matches_reset_envs_on_consecutive_calls(device):
    E = 96
    a, b = _pair(device, E)
    first = np.array([3, 17, 17, 95, 0, 42], np.uint32)           # unsorted, with a duplicate
    second = np.array([42, 7, 8, 9, 64], np.uint32)
    a.reset_envs(first); b.reset_envs_static(first)
    assert _state(a) == _state(b)
    a.step_n(3); b.step_n(3)
    a.reset_envs(second); b.reset_envs_static(second)
    assert _state(a) == _state(b)
    a.step_n(2); b.step_n(2)
    assert _state(a) == _state(b)
    # the reset envs really went back to the creation state, the others did not
    q = b.download(F.JOINT_POSITION)
    fresh = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    q0 = fresh.download(F.JOINT_POSITION)
    b.reset_envs_static(np.arange(E, dtype=np.uint32))
    assert np.array_equal(b.download(F.JOINT_POSITION), q0) and not np.array_equal(q, q0)
    for w in (a, b, fresh):
        w.destroy()


def _free_device_bytes():
    import torch
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_reset_allocates_nothing_and_two_worlds_share_the_array(device):
    """After the set-up call the free device memory does not move across further static resets (the property the entry
    point exists for), and two worlds on the device that call in turn each get exactly their own ids reset: the
    shared id array is rewritten by every call."""
    pytest.importorskip("torch")
    E = 64
    a, b = _pair(device, E)
    fresh = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    q0 = fresh.download(F.JOINT_POSITION)
    a.reset_envs_static(np.array([1], np.uint32))             # set-up call: resolves the array's address once
    before = _free_device_bytes()
    ids_a, ids_b = np.array([5, 6, 7, 50], np.uint32), np.array([9, 60], np.uint32)
    for _ in range(4):
        a.reset_envs_static(ids_a)
        b.reset_envs_static(ids_b)
        assert _free_device_bytes() == before
        a.step_n(2); b.step_n(2)
    assert _free_device_bytes() == before
    a.reset_envs_static(ids_a); b.reset_envs_static(ids_b)
    qa, qb = a.download(F.JOINT_POSITION), b.download(F.JOINT_POSITION)
    reset_a, reset_b = np.zeros(E, bool), np.zeros(E, bool)
    reset_a[ids_a] = True; reset_b[ids_b] = True
    assert np.array_equal(qa[reset_a], q0[reset_a]) and not np.array_equal(qa[~reset_a & (np.arange(E) != 1)], q0[~reset_a & (np.arange(E) != 1)])
    assert np.array_equal(qb[reset_b], q0[reset_b]) and (qb[~reset_b] != q0[~reset_b]).any(axis=1).all()
    for w in (a, b, fresh):
        w.destroy()


def test_static_reset_rejects_bad_requests_without_mutation(device):
    E = 32
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    w.step_n(4)
    before = _state(w)
    lib = _abi.lib()
    too_many = np.zeros(4097, np.uint32)
    rc = lib.nuka_b200_world_reset_envs_static(w._h, too_many.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), too_many.size)
    assert rc == _abi.INVALID_ARG and b"4096" in lib.nuka_last_error_message()
    bad = np.array([1, E], np.uint32)
    assert lib.nuka_b200_world_reset_envs_static(w._h, bad.ctypes.data_as(ctypes.POINTER(ctypes.c_uint32)), bad.size) == _abi.INVALID_ARG
    assert lib.nuka_b200_world_reset_envs_static(w._h, None, 3) == _abi.INVALID_ARG
    assert lib.nuka_b200_world_reset_envs_static(w._h, None, 0) == _abi.OK
    assert lib.nuka_b200_world_reset_envs_static(None, None, 0) == _abi.NULL_HANDLE
    assert _state(w) == before
    w.destroy()

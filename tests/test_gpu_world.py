"""GPU behaviour of the world interface: determinism, reset semantics, views, graph mode, error codes
(the reference's tests/c_abi/test_multi_env_world.cpp:222-300 and python/tests/test_nuka_dlpack.py)."""
import ctypes

import numpy as np
import pytest

import nuka
from nuka import Field as F, _abi, templates as T

pytestmark = pytest.mark.gpu


def quad_world(device, E, seed=None):
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    if seed is not None:
        st = T.quadruped_state(E, seed)
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
    return w


def test_identical_envs_stay_bit_identical_and_runs_repeat(device):
    outs = []
    for _ in range(2):
        w = quad_world(device, 512)
        w.step_n(60)
        q, base = w.download(F.JOINT_POSITION), w.download(F.BASE_POSE)
        assert (q == q[0]).all() and (base == base[0]).all()
        outs.append((q.tobytes(), base.tobytes()))
        w.destroy()
    assert outs[0] == outs[1]


def test_step_n_equals_repeated_steps_and_graph_mode(device):
    a, b, c = quad_world(device, 64, 0), quad_world(device, 64, 0), quad_world(device, 64, 0)
    a.step_n(12)
    for _ in range(12):
        b.step()
    c.set_execution_mode(True)
    c.step_n(12)
    qa, qb, qc = a.download(F.JOINT_VELOCITY), b.download(F.JOINT_VELOCITY), c.download(F.JOINT_VELOCITY)
    assert qa.tobytes() == qb.tobytes() == qc.tobytes()
    for w in (a, b, c):
        w.destroy()


def test_reset_semantics(device):
    w = quad_world(device, 32, 3)
    w.upload(F.DRIVE_TARGET, np.full((32, 13), 0.3, np.float32))
    ref = quad_world(device, 32)
    q0 = ref.download(F.JOINT_POSITION)
    w.step_n(25)
    before = w.download(F.JOINT_POSITION)
    with pytest.raises(nuka.NukaError) as err:
        w.reset_envs([1, 99])
    assert err.value.code == _abi.INVALID_ARG
    assert np.array_equal(w.download(F.JOINT_POSITION), before)          # no env was changed
    w.reset_envs([5, 7, 5])
    after = w.download(F.JOINT_POSITION)
    assert np.array_equal(after[[5, 7]], q0[[5, 7]])
    keep = [i for i in range(32) if i not in (5, 7)]
    assert np.array_equal(after[keep], before[keep])
    assert np.array_equal(w.download(F.DRIVE_TARGET), np.full((32, 13), 0.3, np.float32))   # targets survive a reset
    w.reset()
    assert np.array_equal(w.download(F.JOINT_POSITION), q0)
    assert np.array_equal(w.download(F.JOINT_VELOCITY), np.zeros_like(q0))
    w.destroy(); ref.destroy()


def test_views_are_zero_copy(device):
    torch = pytest.importorskip("torch")
    w = quad_world(device, 16, 0)
    view = w.view(F.DRIVE_TARGET)
    assert view.shape == (16, 13)
    t = view.torch()
    assert t.data_ptr() == view.device_ptr
    t.fill_(0.25)
    torch.cuda.synchronize()
    assert np.array_equal(w.download(F.DRIVE_TARGET), np.full((16, 13), 0.25, np.float32))
    assert torch.from_dlpack(view).data_ptr() == view.device_ptr
    pose = w.view(F.ARTICULATION_LINK_POSE)
    assert pose.shape == (16, 91)
    w.destroy()


def test_error_codes_on_the_device(device):
    lib = _abi.lib()
    w = quad_world(device, 4)
    view = _abi.BufferView()
    assert lib.nuka_world_get_buffer_view(w._h, 4, ctypes.byref(view)) == _abi.NOT_SUPPORTED     # OBSERVATIONS is not on this path
    buf = np.zeros(8, np.float32)
    assert lib.nuka_world_upload_field(w._h, int(F.JOINT_POSITION), buf.ctypes.data, buf.nbytes, 4 * 13 * 4 - 4) == _abi.INVALID_ARG
    assert lib.nuka_world_set_velocity_iterations(w._h, 0) == _abi.INVALID_ARG
    w.set_velocity_iterations(9)
    assert w.get_velocity_iterations() == 9
    desc = _abi.WorldDesc()
    desc.env_count = 0
    out = ctypes.c_void_p()
    blob = T.arm7().blob()
    assert lib.nuka_world_create_from_template(device._h, ctypes.byref(desc), blob, len(blob), ctypes.byref(out)) == _abi.INVALID_ARG
    desc.env_count = 2
    desc.determinism = 2
    assert lib.nuka_world_create_from_template(device._h, ctypes.byref(desc), blob, len(blob), ctypes.byref(out)) == _abi.INVALID_ARG
    desc.determinism = 0
    assert lib.nuka_world_create_from_template(device._h, ctypes.byref(desc), b"junk" * 8, 32, ctypes.byref(out)) == _abi.PARSE_ERROR
    desc.scene_path = b"/nonexistent/robot.nkt"
    assert lib.nuka_world_create_from_scene(device._h, ctypes.byref(desc), ctypes.byref(out)) == _abi.FILE_NOT_FOUND
    desc.scene_path = b"robot.usda"
    assert lib.nuka_world_create_from_scene(device._h, ctypes.byref(desc), ctypes.byref(out)) == _abi.NOT_SUPPORTED
    w.destroy()


def test_nan_input_sets_the_status_bit_without_faulting(device):
    w = quad_world(device, 8, 0)
    target = w.download(F.DRIVE_TARGET)
    target[3, 4] = np.nan
    w.upload(F.DRIVE_TARGET, target)
    w.step()
    status = w.download(F.ENV_STATUS)[:, 0]
    assert status[3] & (1 << 10) and not (status[[0, 1, 2, 4, 5, 6, 7]] & (1 << 10)).any()
    w.destroy()


def test_contact_point_capacity_overflow_sets_the_status_bit_and_drops_the_excess(device):
    """Six boxes landing produce more contact points than a template capacity of 8: the envs that exceed it raise the
    head-overflow status bit (1 << 20), the extra points get no solver rows, and stepping goes on with finite state."""
    E = 32
    tb = T.box_pile(2, count=6)
    tb.max_points = 8
    st = T.box_pile_state(E, 2, count=6)
    w = nuka.World.create_from_template(device, tb.blob(), E)
    w.upload(F.RIGID_BODY_TRANSFORM, st["body_pose"])
    w.forward_kinematics()
    w.step_n(60)
    status = w.download(F.ENV_STATUS)[:, 0]
    points = w.download(F.CONTACT_COUNT).sum(axis=1)
    assert (points > 8).any()
    assert ((status & (1 << 20)) != 0).any()
    assert (((status & (1 << 20)) != 0) | (points <= 8)).all()          # every env over the capacity in the last step is flagged
    assert np.isfinite(w.download(F.RIGID_BODY_TRANSFORM)).all() and np.isfinite(w.download(F.BODY_LINEAR_VELOCITY)).all()
    w.step_n(5)                                                          # and the world keeps stepping
    w.synchronize()
    w.destroy()


def test_scene_path_loads_a_cooked_template_file(device, tmp_path):
    path = tmp_path / "arm.nkt"
    path.write_bytes(T.arm7(0).blob())
    w = nuka.World.create_from_scene(device, str(path), 8, dt=1.0 / 250.0)
    w.step_n(3)
    assert np.isfinite(w.download(F.JOINT_POSITION)).all()
    w.destroy()


def test_pack_observations_matches_the_host_side_layout(device):
    import torch
    from nuka import shard
    E = 33
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    st = T.quadruped_state(E, 2)
    w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
    w.step_n(3)
    assert w.observation_width() == shard.RECORD_FLOATS
    out = torch.zeros((E, shard.RECORD_FLOATS), dtype=torch.float32, device="cuda")
    w.pack_observations(out); w.synchronize()
    views = [w.view(f).torch() for f in (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.LINK_VELOCITY, F.DRIVE_TARGET)]
    want = shard.pack_observations(torch.zeros_like(out), *views)
    assert torch.equal(out, want)
    small = torch.zeros(10, dtype=torch.float32, device="cuda")
    with pytest.raises(nuka.NukaError):
        w.pack_observations(small)
    w.destroy()


def test_device_borrows_the_callers_stream(device):
    """A device created over a caller's stream runs its worlds there (reference python/tests/test_caller_stream.py)
    and produces the same bytes as a device with its own stream."""
    torch = pytest.importorskip("torch")
    stream = torch.cuda.Stream()
    borrowed = nuka.Device.create(0, cuda_stream=stream.cuda_stream)
    w = quad_world(borrowed, 24, 1)
    got = ctypes.c_void_p()
    assert _abi.lib().nuka_world_get_stream(w._h, ctypes.byref(got)) == _abi.OK
    assert got.value == stream.cuda_stream
    ref = quad_world(device, 24, 1)
    w.step_n(7); ref.step_n(7)
    stream.synchronize()                    # the caller's own synchronisation is enough to see the results
    assert w.download(F.JOINT_POSITION).tobytes() == ref.download(F.JOINT_POSITION).tobytes()
    w.destroy(); ref.destroy(); borrowed.destroy()


def test_drive_targets_written_through_a_view_steer_the_next_step(device):
    """DRIVE_TARGET is a writable input picked up by the following step (tests/c_abi/test_drive_target_io.cpp)."""
    torch = pytest.importorskip("torch")
    E = 8
    w = quad_world(device, E, 0)
    w.step_n(50)
    before = w.download(F.JOINT_POSITION)
    targets = w.view(F.DRIVE_TARGET).torch()
    targets[:, 3] += 0.3                    # one thigh joint of every env
    torch.cuda.synchronize()
    w.step_n(60)
    after = w.download(F.JOINT_POSITION)
    moved = after[:, 3] - before[:, 3]
    assert (moved > 0.1).all() and (moved < 0.4).all()
    others = np.delete(after - before, 3, axis=1)
    assert np.abs(others).mean() < 0.1              # the rest of the robot only adjusts its balance
    assert w.download(F.ENV_STATUS).max() == 0
    w.destroy()

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


def test_scene_path_takes_the_scene_file_the_reference_takes(device):
    """nuka_world_create_from_scene on a `.nks` document: the library cooks it itself (reference semantics: the scene's
    actuators, ground and filter bits, one candidate slot per admissible pair), and the world steps bit-identically to
    one created from the Python cooker's template of the same file."""
    import os
    from nuka import nks
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "scene_quadbox.nks")
    E = 16
    a = nuka.World.create_from_scene(device, path, E, dt=1.0 / 200.0, solver_vel_iters=4)
    tb = nks.cook(path, dt=1.0 / 200.0, vel_iters=4, kp=0.0, kd=0.0, scene_filters=True, ground_height=None, max_contacts=35)
    b = nuka.World.create_from_template(device, tb.blob(), E)
    assert a.info.contact_slots_per_env == 35 and a.info.links_per_env == 13 and a.info.bodies_per_env == b.info.bodies_per_env
    st = T.quadruped_state(E, 0)
    for w in (a, b):
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
        w.step_n(40)
    for f in (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.RIGID_BODY_TRANSFORM, F.CONTACT_COUNT):
        assert np.array_equal(a.download(f), b.download(f)), f
    assert a.download(F.CONTACT_COUNT).sum() > 0
    a.destroy(); b.destroy()


def test_observation_record_matches_the_reference_contract(device):
    """The pack kernel against the numpy statement of python/nuka/tasks/go2_obs.py:282-305 (the reference checks its
    own composer the same way, python/tests/test_gym_env.py:87), with a joint permutation, a reward column and a row
    stride as used for a gather-buffer slice."""
    import torch
    from nuka import shard
    E = 33
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
    st = T.quadruped_state(E, 2)
    st["base_pose"][:, 3:] += 0.3 * np.random.default_rng(1).normal(size=(E, 4)).astype(np.float32)     # tilted bases
    st["base_pose"][:, 3:] /= np.linalg.norm(st["base_pose"][:, 3:], axis=1, keepdims=True)
    w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
    w.step_n(3)
    assert w.observation_width() == shard.OBS_FLOATS
    rng = np.random.default_rng(3)
    command = torch.tensor(rng.normal(size=(E, 3)).astype(np.float32), device="cuda")
    action = torch.tensor(rng.normal(size=(E, 12)).astype(np.float32), device="cuda")
    default = torch.tensor(rng.normal(size=12).astype(np.float32), device="cuda")
    order = torch.tensor(rng.permutation(12).astype(np.int32), device="cuda")
    reward = torch.tensor(rng.normal(size=E).astype(np.float32), device="cuda")
    stride = 56
    out = torch.full((E, stride), -7.0, dtype=torch.float32, device="cuda")
    desc = w.observation_desc(command, last_action=action, default_position=default, joint_order=order, reward=reward, row_stride=stride)
    w.pack_observations(desc, out); w.synchronize()
    get = lambda f: w.download(f)
    want = shard.observation_record(get(F.JOINT_POSITION), get(F.JOINT_VELOCITY), get(F.ARTICULATION_LINK_POSE), get(F.LINK_VELOCITY),
                                    command.cpu().numpy(), action.cpu().numpy(), default.cpu().numpy(), order.cpu().numpy(),
                                    reward=reward.cpu().numpy())
    got = out.cpu().numpy()
    assert np.allclose(got[:, :49], want, rtol=1e-6, atol=1e-6)
    assert np.array_equal(got[:, 12:24], want[:, 12:24]) and np.array_equal(got[:, 36:49], want[:, 36:49])
    assert (got[:, 49:] == -7.0).all()                      # the padding of each row is untouched
    # shared command, identity order, no reward, packed rows
    shared = torch.tensor([0.5, 0.0, -0.1], device="cuda")
    tight = torch.zeros((E, 48), dtype=torch.float32, device="cuda")
    w.pack_observations(w.observation_desc(shared), tight); w.synchronize()
    want = shard.observation_record(get(F.JOINT_POSITION), get(F.JOINT_VELOCITY), get(F.ARTICULATION_LINK_POSE), get(F.LINK_VELOCITY),
                                    (0.5, 0.0, -0.1), np.zeros((E, 12), np.float32))
    assert np.allclose(tight.cpu().numpy(), want, rtol=1e-6, atol=1e-6)
    small = torch.zeros(10, dtype=torch.float32, device="cuda")
    with pytest.raises(nuka.NukaError):
        w.pack_observations(w.observation_desc(shared), small)
    w.destroy()


def test_masked_reset_matches_reset_envs(device):
    """The device-mask reset gives the bytes of nuka_world_reset_envs for the same env set, without a host round trip."""
    import torch
    E = 40
    a, b = quad_world(device, E, 4), quad_world(device, E, 4)
    a.step_n(5); b.step_n(5)
    ids = np.array([0, 7, 8, 31, 39], np.uint32)
    mask = torch.zeros(E, dtype=torch.int32, device="cuda")
    mask[torch.tensor(ids.astype(np.int64), device="cuda")] = 1
    torch.cuda.synchronize()
    a.reset_envs(ids); b.reset_envs_masked(mask)
    fields = (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.ARTICULATION_LINK_POSE, F.RIGID_BODY_TRANSFORM, F.LINK_VELOCITY, F.ENV_STATUS)
    for f in fields:
        assert a.download(f).tobytes() == b.download(f).tobytes(), f
    a.step_n(3); b.step_n(3)
    for f in fields:
        assert a.download(f).tobytes() == b.download(f).tobytes(), f
    a.destroy(); b.destroy()


def test_contact_readout_can_be_switched_off(device):
    E = 16
    a, b = quad_world(device, E, 2), quad_world(device, E, 2)
    b.set_contact_readout(False)
    a.step_n(40); b.step_n(40)
    assert a.download(F.JOINT_POSITION).tobytes() == b.download(F.JOINT_POSITION).tobytes()
    assert a.download(F.CONTACT_COUNT).sum() > 0 and b.download(F.CONTACT_COUNT).sum() == 0      # never written while off
    b.set_contact_readout(True)
    a.step(); b.step()
    assert np.array_equal(a.download(F.CONTACT_COUNT), b.download(F.CONTACT_COUNT))
    assert np.array_equal(a.download(F.PAIR_COUNT), b.download(F.PAIR_COUNT))
    a.destroy(); b.destroy()


def test_destroyed_handles_stay_dead(device):
    """Handle ids are never reused (reference src/c_abi/handle_table.hpp:18-26): a handle kept past destroy does not
    address a world created later."""
    lib = _abi.lib()
    w = quad_world(device, 4, 0)
    stale = ctypes.c_void_p(w._h.value)
    w.destroy()
    fresh = quad_world(device, 4, 0)
    assert fresh._h.value != stale.value
    assert lib.nuka_world_step(stale) == _abi.NULL_HANDLE
    fresh.step()
    fresh.destroy()


def test_outputs_reject_uploads(device):
    w = quad_world(device, 4, 0)
    lib = _abi.lib()
    buf = np.zeros((4, 13 * 7), np.float32)
    assert lib.nuka_world_upload_field(w._h, int(F.ARTICULATION_LINK_POSE), buf.ctypes.data, buf.nbytes, 0) == _abi.NOT_SUPPORTED
    assert lib.nuka_world_upload_field(w._h, int(F.SOLVER_RESIDUAL), buf.ctypes.data, 16, 0) == _abi.NOT_SUPPORTED
    assert lib.nuka_world_download_field(w._h, int(F.ARTICULATION_LINK_POSE), buf.ctypes.data, buf.nbytes, 0) == _abi.OK
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


def test_slim_and_regular_kernel_builds_give_the_same_state(device):
    """A world picks the 128-register build of its step kernel where that buys residency; the two builds are the same
    arithmetic, so the states they produce are bit-identical."""
    import os
    E = 128
    st = T.quadruped_state(E, 3)
    out = []
    for slim in ("0", "1"):
        os.environ["NUKA_B200_SLIM"] = slim            # read when the world lays out its launch
        try:
            w = nuka.World.create_from_template(device, T.quadruped(0).blob(), E)
        finally:
            del os.environ["NUKA_B200_SLIM"]
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
        w.step_n(80)
        out.append([w.download(f) for f in (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.LINK_VELOCITY, F.CONTACT_COUNT, F.SOLVER_SWEEPS)])
        w.destroy()
    for a, b in zip(*out):
        assert np.array_equal(a, b)


def test_dof_names_of_a_scene_world(device):
    """nuka_world_get_dof_name on a world created from a scene file: joint names in link order, the size query, a buffer
    that is too small, an index past the last env's links; NOT_SUPPORTED for a procedural template without names."""
    import ctypes
    import os
    from nuka import _abi, templates as T
    scene = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "scene_quadruped.nks")
    w = nuka.World.create_from_scene(device, scene, 4)
    assert w.dof_names() == ["link0"] + [f"joint{i}" for i in range(1, 13)]
    assert list(w.dof_index("joint7")) == [7] and list(w.dof_index("robot/joint1")) == [1, 10, 11, 12] and w.dof_index("nothing").size == 0
    assert w.base_link_count == 13 and w.action_dim == 12
    w.set_drive_targets(np.arange(4 * 13, dtype=np.float32))
    assert np.array_equal(w.download(F.DRIVE_TARGET).reshape(-1), np.arange(4 * 13, dtype=np.float32))
    need = ctypes.c_size_t()
    assert _abi.lib().nuka_world_get_dof_name(w._h, 13 * 3 + 2, None, 0, ctypes.byref(need)) == 0 and need.value == 6      # env 3's joint2
    small = ctypes.create_string_buffer(4)
    assert _abi.lib().nuka_world_get_dof_name(w._h, 2, small, 4, ctypes.byref(need)) == 1 and need.value == 6
    assert _abi.lib().nuka_world_get_dof_name(w._h, 13 * 4, None, 0, ctypes.byref(need)) == 1
    w.destroy()
    w = nuka.World.create_from_template(device, T.quadruped(0).blob(), 4)
    with pytest.raises(nuka.NukaError) as err:
        w.dof_names()
    assert err.value.code == 7
    w.destroy()

"""Checkpoints through the C ABI (reference nuka.h:387-404, src/c_abi/checkpoint.cpp): capture, restore, file round
trip, equality and the state hash.  The property checked at the benchmark's size is that a restored world repeats
the steps that followed the capture bit for bit."""
import numpy as np
import pytest

import nuka
from nuka import Field as F
from nuka import templates as T

pytestmark = pytest.mark.gpu


def _quadruped_world(device, E):
    st = T.quadruped_state(E, 3)
    w = nuka.World.create_from_template(device, T.quadruped().blob(), E)
    w.upload(F.JOINT_POSITION, st["q"])
    w.upload(F.BASE_POSE, st["base_pose"])
    w.forward_kinematics()
    return w


def test_restore_repeats_the_following_steps_bit_for_bit(device):
    E = 4096
    w = _quadruped_world(device, E)
    w.step_n(40)
    ck = w.checkpoint_capture()
    h0 = w.state_hash()
    w.step_n(25)
    first = {f: w.download(f).copy() for f in (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.LINK_VELOCITY, F.ARTICULATION_LINK_POSE)}
    h1 = w.state_hash()
    assert h1 != h0
    w.checkpoint_restore(ck)
    assert w.state_hash() == h0
    w.step_n(25)
    for f, v in first.items():
        assert np.array_equal(w.download(f), v), f
    assert w.state_hash() == h1
    ck.destroy()
    w.destroy()


def test_file_round_trip_equality_and_sizes(device, tmp_path):
    E = 64
    w = _quadruped_world(device, E)
    w.set_velocity_iterations(6)
    w.step_n(10)
    a = w.checkpoint_capture()
    b = w.checkpoint_capture()
    assert a == b and a.byte_size == b.byte_size and a.byte_size > E * 13 * 4
    path = tmp_path / "quad.nkc"
    a.write(path)
    assert path.stat().st_size == 32 + a.byte_size + 16
    w.step_n(3)
    c = w.checkpoint_capture()
    assert not (a == c)
    w.set_velocity_iterations(2)
    r = w.checkpoint_read(path)
    assert r == a
    w.checkpoint_restore(r)
    assert w.get_velocity_iterations() == 6
    d = w.checkpoint_capture()
    assert d == a
    for ck in (a, b, c, r, d):
        ck.destroy()
    w.destroy()


def test_free_bodies_and_contact_cache_are_part_of_the_state(device):
    E = 64
    st = T.box_pile_state(E, 2, count=6)
    w = nuka.World.create_from_template(device, T.box_pile(2, count=6).blob(), E)
    w.upload(F.RIGID_BODY_TRANSFORM, st["body_pose"])
    w.forward_kinematics()
    w.step_n(30)                                   # boxes have landed: the warm-start cache is in use
    ck = w.checkpoint_capture()
    w.step_n(10)
    pose = w.download(F.RIGID_BODY_TRANSFORM).copy()
    lin = w.download(F.BODY_LINEAR_VELOCITY).copy()
    w.checkpoint_restore(ck)
    w.step_n(10)
    assert np.array_equal(w.download(F.RIGID_BODY_TRANSFORM), pose)
    assert np.array_equal(w.download(F.BODY_LINEAR_VELOCITY), lin)
    ck.destroy()
    w.destroy()


def test_error_behaviour(device, tmp_path):
    w1 = _quadruped_world(device, 8)
    w2 = _quadruped_world(device, 8)
    w3 = _quadruped_world(device, 16)
    ck = w1.checkpoint_capture()
    with pytest.raises(nuka.NukaError) as err:     # another world's checkpoint, even of the same layout
        w2.checkpoint_restore(ck)
    assert err.value.code == 1
    path = tmp_path / "w1.nkc"
    ck.write(path)
    r2 = w2.checkpoint_read(path)                  # same layout: reading into another world is allowed
    w2.checkpoint_restore(r2)
    with pytest.raises(nuka.NukaError) as err:     # other env count: layout hash differs
        w3.checkpoint_read(path)
    assert err.value.code == 1
    short = tmp_path / "short.nkc"
    short.write_bytes(path.read_bytes()[:100])
    with pytest.raises(nuka.NukaError) as err:
        w1.checkpoint_read(short)
    assert err.value.code == 1
    with pytest.raises(nuka.NukaError) as err:
        w1.checkpoint_read(tmp_path / "absent.nkc")
    assert err.value.code == 1
    ck.destroy()
    with pytest.raises(nuka.NukaError) as err:     # destroyed handle
        w1.checkpoint_restore(ck) if ck._h else w1.checkpoint_restore(nuka.Checkpoint(None))
    assert err.value.code == 2
    r2.destroy()
    for w in (w1, w2, w3):
        w.destroy()

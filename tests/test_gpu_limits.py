"""Sizes at the edges of what the path accepts: one env, the largest articulation (32 links; 64 coordinates would need
more links than fit, so 31 scalar joints under a floating base: 37 coordinates, two per lane), a world without
collidables, and templates just past the limits."""
import numpy as np
import pytest

import nuka
from nuka import Field as F, templates as T

pytestmark = pytest.mark.gpu


def chain(links, floating=True):
    """A serial chain of revolute joints with alternating axes under a floating (or fixed) root."""
    tb = T.TemplateBuilder(dt=1.0 / 500.0, vel_iters=4, max_contacts=0)
    tb.add_link(None, T.FLOATING if floating else T.FIXED, mass=2.0, inertia_diag=(0.02, 0.02, 0.02))
    for i in range(links - 1):
        tb.add_link(i, T.REVOLUTE, axis=(0, 0, 1) if i % 2 == 0 else (0, 1, 0), offset=(0.0 if i == 0 else 0.1, 0, 0), mass=0.3,
                    inertia_diag=T.box_inertia(0.3, (0.1, 0.02, 0.02)), com=(0.05, 0, 0), kp=5.0, kd=0.2)
    return tb


def rel(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max() / max(np.abs(b).max(), 1e-12))


def test_largest_articulation_matches_the_oracle(device, oracle):
    E, L = 6, 32
    tb = chain(L)
    rng = np.random.Generator(np.random.PCG64(3))
    q = np.zeros((E, L), np.float32)
    q[:, 1:] = rng.uniform(-0.3, 0.3, size=(E, L - 1))
    blob = tb.blob()
    w = nuka.World.create_from_template(device, blob, E)
    o = oracle.World(blob, E)
    w.upload(F.JOINT_POSITION, q); o.set("q", q)
    w.forward_kinematics(); o.refresh()
    assert w.info.links_per_env == 32 and w.info.dofs_per_env == 37
    assert rel(w.download(F.ARTICULATION_LINK_POSE), o.get("link_pose", 7 * L)) < 1e-6
    w.run_stage(1); o.dynamics(False)
    assert rel(w.download(F.MASS_MATRIX), o.get("mass_matrix", 37 * 37)) < 1e-5
    w.step_n(20); o.step(20)
    assert rel(w.download(F.JOINT_POSITION), o.get("q", L)) < 1e-4
    assert not w.download(F.ENV_STATUS).any() and np.isfinite(w.download(F.JOINT_VELOCITY)).all()
    w.destroy()


def test_one_env_and_a_world_without_collidables(device):
    w = nuka.World.create_from_template(device, T.arm7(0).blob(), 1)
    assert w.info.env_count == 1 and w.info.contact_slots_per_env == 0
    w.step_n(10)
    assert np.isfinite(w.download(F.JOINT_POSITION)).all() and w.download(F.JOINT_POSITION).shape == (1, 8)
    w.reset_envs(np.array([0], np.uint32))
    assert np.array_equal(w.download(F.JOINT_POSITION), np.zeros((1, 8), np.float32))
    w.destroy()


def test_templates_past_the_limits_are_rejected(device):
    lib = nuka._abi.lib()
    too_long = chain(33).blob()                              # 33 links
    assert lib.nuka_b200_template_check(too_long, len(too_long)) == nuka._abi.NOT_SUPPORTED
    with pytest.raises(nuka.NukaError) as e:
        nuka.World.create_from_template(device, too_long, 4)
    assert e.value.code == nuka._abi.NOT_SUPPORTED and "32 links" in str(e.value)
    crowded = T.TemplateBuilder(dt=1.0 / 240.0, vel_iters=4, max_contacts=64)
    for k in range(257):                                      # 257 collidable rows
        crowded.add_free_body((T.SPHERE, 0.05), 1.0, (0.001, 0.001, 0.001), (0.2 * k, 0.0, 1.0, 1.0, 0.0, 0.0, 0.0))
    blob = crowded.blob()
    assert lib.nuka_b200_template_check(blob, len(blob)) == nuka._abi.NOT_SUPPORTED
    slots = T.box_pile(0, count=4)
    slots.cfg["max_contacts"] = 1025                          # more contact slots than the path holds
    blob = slots.blob()
    assert lib.nuka_b200_template_check(blob, len(blob)) == nuka._abi.NOT_SUPPORTED
    with pytest.raises(nuka.NukaError):
        nuka.World.create_from_template(device, T.arm7(0).blob(), 0)       # an empty batch

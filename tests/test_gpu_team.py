"""Team mode on the GPU: an env of many free bodies is advanced by several warps (the rigid blocks of one colour
descend side by side).  Blocks of a colour share no constraint row, so the state must not depend on the team size:
every comparison here is bit-exact."""
import os

import numpy as np
import pytest

import nuka
from nuka import Field as F, templates as T

pytestmark = pytest.mark.gpu


def run(device, tb, state, E, steps, team):
    old = os.environ.get("NUKA_B200_TEAM")
    os.environ["NUKA_B200_TEAM"] = str(team)            # read when the world lays out its shared memory
    try:
        w = nuka.World.create_from_template(device, tb.blob(), E)
    finally:
        if old is None:
            del os.environ["NUKA_B200_TEAM"]
        else:
            os.environ["NUKA_B200_TEAM"] = old
    names = {"q": F.JOINT_POSITION, "base_pose": F.BASE_POSE, "body_pose": F.RIGID_BODY_TRANSFORM}
    for k, v in state.items():
        if k in names:
            w.upload(names[k], v)
    w.forward_kinematics()
    w.step_n(steps)
    out = {"pose": w.download(F.RIGID_BODY_TRANSFORM), "lin": w.download(F.BODY_LINEAR_VELOCITY), "ang": w.download(F.BODY_ANGULAR_VELOCITY),
           "status": w.download(F.ENV_STATUS), "sweeps": w.download(F.SOLVER_SWEEPS), "residual": w.download(F.SOLVER_RESIDUAL),
           "counts": w.download(F.CONTACT_COUNT)}
    if w.info.links_per_env:
        out["q"] = w.download(F.JOINT_POSITION); out["qdot"] = w.download(F.JOINT_VELOCITY)
    w.destroy()
    return out


@pytest.mark.parametrize("teams", [(1, 2), (1, 4), (1, 8)])
def test_box_pile_is_independent_of_the_team_size(device, teams):
    E = 6
    tb = T.box_pile(0, count=48)
    st = T.box_pile_state(E, 0, count=48)
    a = run(device, tb, st, E, 40, teams[0])
    b = run(device, tb, st, E, 40, teams[1])
    assert not a["status"].any()
    assert a["counts"].sum() > 48 * E          # the boxes have landed on each other
    for k in a:
        assert np.array_equal(a[k], b[k]), k


def test_default_team_of_a_large_pile_matches_one_warp(device):
    E = 5
    tb = T.box_pile(0, count=48)
    st = T.box_pile_state(E, 0, count=48)
    w = nuka.World.create_from_template(device, tb.blob(), E)
    for k, v in st.items():
        w.upload(F.RIGID_BODY_TRANSFORM, v) if k == "body_pose" else None
    w.forward_kinematics(); w.step_n(25)
    pose = w.download(F.RIGID_BODY_TRANSFORM)
    w.destroy()
    assert np.array_equal(pose, run(device, tb, st, E, 25, 1)["pose"])


def test_articulation_with_boxes_in_a_team(device):
    """The quadruped with four free boxes: the articulation's block stays with the lead warp, the boxes go to the team."""
    E = 16
    tb = T.quadruped(0, boxes=4)
    st = T.quadruped_state(E, 0)
    a = run(device, tb, st, E, 60, 1)
    b = run(device, tb, st, E, 60, 4)
    assert not a["status"].any()
    for k in a:
        assert np.array_equal(a[k], b[k]), k

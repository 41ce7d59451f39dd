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


@pytest.mark.parametrize("drill", [1, 2])
def test_a_wait_that_runs_out_sets_the_status_bit_and_the_world_lives_on(device, drill):
    """The team's warps wait for one another with a cycle budget, never without bound.  Drill 1: the lead leaves without
    dismissing its helpers, which give up after their budget.  Drill 2: helpers never answer, the lead gives up on its
    first command and finishes the env alone.  Either way the launch ends, the env carries the team-timeout bit
    (1 << 21), and the device keeps working."""
    E = 2
    tb = T.box_pile(0, count=48)
    st = T.box_pile_state(E, 0, count=48)
    os.environ["NUKA_B200_TEAM_DRILL"] = str(drill)          # read when the world lays out its shared memory
    try:
        w = nuka.World.create_from_template(device, tb.blob(), E)
    finally:
        del os.environ["NUKA_B200_TEAM_DRILL"]
    w.upload(F.RIGID_BODY_TRANSFORM, st["body_pose"])
    w.forward_kinematics()
    w.step_n(2)
    status = w.download(F.ENV_STATUS)[:, 0]
    assert ((status & (1 << 21)) != 0).all()
    if drill == 2:                                            # the lead did all the work itself: the state is the one-warp state
        want = run(device, tb, st, E, 2, 1)
        assert np.array_equal(w.download(F.RIGID_BODY_TRANSFORM), want["pose"])
    w.destroy()
    healthy = run(device, tb, st, E, 3, 8)                   # the context is intact
    assert not healthy["status"].any()

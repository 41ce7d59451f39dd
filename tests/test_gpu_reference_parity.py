"""GPU parity against the reference's OWN GPU implementation: the CUDA path, through the C ABI, on the scene files and
start states the unmodified reference was stepped on (tests/golden/ref_gpu_<case>.npz; see tests/refparity.py).

Bars (fp32): link poses 1e-6, mass matrices and bias forces 1e-5, single-step post-solve velocities 1e-5, candidate pairs
and contact counts bit-exact, 100-step trajectories 1e-4 in position (the contact-free arm and the landing quadruped
alike).  Joint accelerations are held to the distance the reference itself keeps from the double-precision solve of its
own M and bias (see tests/test_reference_parity_cpu.py)."""
import numpy as np
import pytest

import nuka
from nuka import Field as F

import refparity as RP

pytestmark = pytest.mark.gpu
NAMES = {"q": F.JOINT_POSITION, "qdot": F.JOINT_VELOCITY, "base_pose": F.BASE_POSE, "body_pose": F.RIGID_BODY_TRANSFORM,
         "link_velocity": F.LINK_VELOCITY}
ARTICULATED = sorted(c for c in RP.CASES if c not in ("pile12", "cylinders"))


def make_world(device, case):
    ref = RP.load(case)
    if ref is None:
        pytest.skip(f"no reference vectors for {case}")
    tb, E, L, n, S = RP.template(case, ref)
    w = nuka.World.create_from_template(device, tb.blob(), E, control_mode=RP.CONTROL_MODE.get(case, 0),
                                        **({"osc_task_link": RP.TASK_LINK[case]} if case in RP.TASK_LINK else {}))
    st = RP.start_state(case, E)
    for k in ("q", "qdot", "base_pose", "body_pose"):
        if k in st:
            w.upload(NAMES[k], st[k])
    for k, (_, field) in RP.DRIVE_INPUTS.items():
        if k in st:
            w.upload(getattr(F, field), st[k])
    w.forward_kinematics()
    if "link_velocity" in st:
        w.upload(F.LINK_VELOCITY, st["link_velocity"])
    return ref, w, E, L, n, S


@pytest.mark.parametrize("case", ARTICULATED)
def test_dynamics_match_the_reference(device, case):
    ref, w, E, L, n, S = make_world(device, case)
    assert RP.err_env(w.download(F.ARTICULATION_LINK_POSE), ref["start_link_pose"].reshape(E, -1)) < 1e-6
    assert np.array_equal(w.download(F.DRIVE_STIFFNESS), ref["start_kp"].reshape(E, L))
    # the reference's single-op dispatch ran without the drive stage: switch every drive input off
    w.upload(F.DRIVE_STIFFNESS, np.zeros((E, L), np.float32)); w.upload(F.DRIVE_DAMPING, np.zeros((E, L), np.float32))
    w.upload(F.JOINT_FEEDFORWARD, np.zeros((E, L), np.float32))
    if RP.CONTROL_MODE.get(case) in (1, 5):       # the target field carries efforts in these modes
        w.upload(F.DRIVE_TARGET, np.zeros((E, L), np.float32))
    w.run_stage(1)
    assert RP.err_env(w.download(F.MASS_MATRIX), ref["dyn_mass"].reshape(E, -1)) < 1e-5
    ours, theirs, largest = RP.acceleration_errors(ref, w.download(F.JOINT_ACCELERATION), E, L, n)
    assert ours < max(3.0 * theirs, 2e-5), (ours, theirs)
    if largest > 1.0:
        assert RP.err_env(w.download(F.JOINT_ACCELERATION)[:, 1:], ref["dyn_qddot"].reshape(E, L)[:, 1:]) < 1e-4
    w.destroy()


@pytest.mark.parametrize("case", sorted(RP.CASES))
def test_steps_match_the_reference(device, case):
    ref, w, E, L, n, S = make_world(device, case)
    steps = [int(s) for s in ref["traj_steps"]]
    K, B = len(steps), int(ref["run"][3])
    q, qd = ref["traj_q"].reshape(K, E, L), ref["traj_qdot"].reshape(K, E, L)
    done = 0
    own_any = np.zeros(E, np.uint32)
    for i, s in enumerate(steps):
        if case in RP.SENSITIVE and s > RP.SENSITIVE[case]:
            break
        if case in RP.SENSITIVE:        # one step at a time: the free-rotation bit describes the latest step only
            for _ in range(s - done):
                w.step_n(1)
                own_any |= w.download(F.ENV_STATUS)[:, 0]
        else:
            w.step_n(s - done)
            own_any |= w.download(F.ENV_STATUS)[:, 0]
        done = s
        first = i == 0
        ref_any = ref["traj_status_any"].reshape(K, E)[i] if "traj_status_any" in ref else ref["traj_status"].reshape(K, E)[i]
        keep = RP.comparable(case, ref_any, own_any)
        if L:
            RP.assert_position_parity(w.download(F.JOINT_POSITION), q[i], first, (case, s, "q"), case, keep=keep)
            RP.assert_velocity_parity(w.download(F.JOINT_VELOCITY), qd[i], first, (case, s, "joint rates"), case, keep=keep)
            if first:
                RP.assert_ill_conditioned_first_step(case, w.download(F.JOINT_VELOCITY), qd[i])
        if ref["traj_base_pose"].size:
            RP.assert_position_parity(w.download(F.BASE_POSE), ref["traj_base_pose"].reshape(K, E, 7)[i], first,
                                      (case, s, "base"), case, keep=keep)
            twist = w.download(F.LINK_VELOCITY).reshape(E, L, 6)[:, 0]
            RP.assert_velocity_parity(twist, ref["traj_root_twist"][i], first, (case, s, "root twist"), case, keep=keep)
        if "traj_body_pose" in ref:
            RP.assert_position_parity(w.download(F.RIGID_BODY_TRANSFORM).reshape(E, 7 * B), ref["traj_body_pose"].reshape(K, E, 7 * B)[i],
                                      first, (case, s, "bodies"), case, absolute=True, keep=keep)
        assert not w.download(F.ENV_STATUS)[keep].any()
        if S:
            count = ref["traj_pair_count"].reshape(K, E)[i]
            pairs = ref["traj_candidate_pairs"].reshape(K, E, S, 2)[i]
            mine = w.download(F.CANDIDATE_PAIRS).reshape(E, S, 2)
            same = (w.download(F.PAIR_COUNT)[:, 0] == count)
            same &= np.array([same[e] and np.array_equal(mine[e, :count[e]], pairs[e, :count[e]]) for e in range(E)])
            same &= (w.download(F.CONTACT_COUNT) == ref["traj_contact_count"].reshape(K, E, S)[i]).all(axis=1)
            # bit-exact in every compared env; along a chaotic or sensitive trajectory in every env that has not left the
            # common trajectory (at least 90 % of them, see refparity.CHAOTIC and refparity.SENSITIVE)
            if first or (case not in RP.CHAOTIC and case not in RP.SENSITIVE):
                assert same[keep].all(), (case, s, int((~same[keep]).sum()))
            else:
                assert same[keep].mean() >= 0.9, (case, s, float(same[keep].mean()))
    w.destroy()


def test_tree_broadphase_matches_the_reference_at_8192_envs(device):
    """8192 envs of the 12-box pile: the reference's broadphase takes its LBVH route there (B^2 E > 2^20), and so does this
    library by the same rule.  Candidate pairs and contact counts, compared through per-env digests: bit-equal in all 8192
    envs on the first step, afterwards in every env that has not left the reference's trajectory (at least 90 %)."""
    from nuka import nks, templates as T
    ref = RP.load("pile12_tree")
    if ref is None:
        pytest.skip("no reference vectors for pile12_tree")
    E, B, S, iters = (int(ref["run"][k]) for k in (0, 3, 4, 5))
    tb = nks.cook(RP.os.path.join(RP.GOLDEN, "scene_pile12.nks"), dt=float(ref["run_dt"][0]), vel_iters=iters, kp=0.0, kd=0.0,
                  scene_filters=True, ground_height=None, max_contacts=S, max_points=RP.MAX_POINTS["pile12"])
    w = nuka.World.create_from_template(device, tb.blob(), E)
    w.upload(F.RIGID_BODY_TRANSFORM, T.box_pile_state(E, 0, count=12)["body_pose"].reshape(E, -1))
    w.forward_kinematics()
    done = 0
    for i, s in enumerate(int(v) for v in ref["traj_steps"]):
        w.step_n(s - done)
        done = s
        count = w.download(F.PAIR_COUNT)[:, 0]
        pairs, contacts = RP.pair_digests(count, w.download(F.CANDIDATE_PAIRS), w.download(F.CONTACT_COUNT))
        same = (pairs == ref["pair_digest"][i]) & (contacts == ref["contact_digest"][i]) & (count == ref["traj_pair_count"][i])
        assert same.all() if i == 0 else same.mean() >= 0.9, (s, float(same.mean()))
        d = RP.err_envs(w.download(F.RIGID_BODY_TRANSFORM).reshape(E, 7 * B)[:128], ref["traj_body_pose_head"][i], floor=1.0)
        assert np.median(d) < 1e-5 and np.percentile(d, 90) < 1e-4, (s, float(np.median(d)), float(np.percentile(d, 90)))
    assert not w.download(F.ENV_STATUS).any()
    w.destroy()

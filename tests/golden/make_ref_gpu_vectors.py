"""Golden vectors from the reference's OWN GPU implementation (oracle/_ref/ref_driver, built by oracle/ref_gpu/Makefile
from the reference checkout).  Three phases, because the driver needs a GPU and the checkout does not travel:

  python tests/golden/make_ref_gpu_vectors.py prepare   writes the scene files (.nks, from the procedural templates), the
                                                        per-env start states and run.sh into oracle/_ref/run/, and the
                                                        reference's cook of each scene (no GPU needed) into tests/golden/
  bash oracle/_ref/run/run.sh                           on a machine with a GPU: steps the scenes with the reference and
                                                        writes OUT/ref_*.nkt and OUT/ref_timing.jsonl (OUT defaults to the
                                                        repository's scratch output folder)
  python tests/golden/make_ref_gpu_vectors.py collect   copies the results into tests/golden/

Both sides of the later comparison read the same .nks scene: the reference through its loader and cooker, this
library through nuka.nks.cook."""
import json
import os
import shutil
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "nuka-physics_b200"))
sys.path.insert(0, HERE)
from nuka import nks, nkt, templates as T
import ref_cases

RUN = os.path.join(ROOT, "oracle", "_ref", "run")
DRIVER = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
ENVS = 128          # above 64, where the reference solver's blocks never wait on one another
CASES = {
    # name: (template, state maker, dt, velocity iterations, steps, sampling stride)
    "arm7": (lambda: T.arm7(0), lambda E: T.arm7_state(E, 0), 1.0 / 500.0, 4, 100, 20),
    "quadruped": (lambda: T.quadruped(0), lambda E: T.quadruped_state(E, 0), 1.0 / 200.0, 4, 100, 20),
    # the same robot started with joint rates and a base twist: meaningful joint accelerations, airborne then landing
    "quadruped_moving": (lambda: T.quadruped(0), lambda E: ref_cases.quadruped_moving_state(E, 0), 1.0 / 200.0, 4, 40, 10),
    # free rigid boxes dropping onto the plane and each other: box-box and box-plane manifolds, rigid blocks in the solver
    "pile12": (lambda: T.box_pile(0, count=12), lambda E: T.box_pile_state(E, 0, count=12), 1.0 / 240.0, 8, 60, 20),
    # configs[4]'s env: the quadruped with four free boxes around it
    "quadbox": (lambda: T.quadruped(0, boxes=4), lambda E: T.quadruped_state(E, 0), 1.0 / 200.0, 4, 60, 20),
    # configs[2]'s env: the 35-coordinate humanoid with ground and limb self-contact
    "humanoid": (lambda: T.humanoid(0), lambda E: T.humanoid_state(E, 0), 1.0 / 200.0, 8, 40, 10),
    # computed-torque control (control mode 3): the arm without contacts, the quadruped landing with saturating force limits
    "arm7_ct": (lambda: T.arm7(0), lambda E: ref_cases.arm_computed_torque_state(E, 0), 1.0 / 500.0, 4, 100, 20),
    "quadruped_ct": (lambda: T.quadruped(0), lambda E: ref_cases.quadruped_computed_torque_state(E, 0), 1.0 / 200.0, 4, 60, 20),
    # the other control modes on the landing quadruped: joint efforts with a feedforward term (1), rate targets (2),
    # efforts inside a torque-speed envelope (5)
    "quadruped_torque": (lambda: T.quadruped(0), lambda E: ref_cases.quadruped_mode_state(1, E), 1.0 / 200.0, 4, 40, 10),
    "quadruped_velocity": (lambda: T.quadruped(0), lambda E: ref_cases.quadruped_mode_state(2, E), 1.0 / 200.0, 4, 40, 10),
    "quadruped_actuator": (lambda: T.quadruped(0), lambda E: ref_cases.quadruped_mode_state(5, E), 1.0 / 200.0, 4, 40, 10),
    # operational-space control (control mode 4): the arm's tip and one foot of the landing quadruped as task frames
    "arm7_osc": (lambda: T.arm7(0), lambda E: ref_cases.arm_osc_state(E, 0), 1.0 / 500.0, 4, 40, 10),
    "quadruped_osc": (lambda: T.quadruped(0), lambda E: ref_cases.quadruped_osc_state(E, 0), 1.0 / 200.0, 4, 20, 5),
    # free cylinders and spheres over a plane: the cylinder-plane (cap, rim, side) and cylinder-sphere manifolds
    "cylinders": (lambda: ref_cases.cylinder_field(), lambda E: ref_cases.cylinder_field_state(E), 1.0 / 250.0, 8, 80, 20),
    # seeded random articulations (random trees, revolute / prismatic / fixed joints, limits, dry friction, armature,
    # spheres with boxes or capsules, free bodies): parity beyond the benchmark robots
    **{f"random{k}": (lambda k=k: ref_cases.random_robot(k), lambda E, k=k: ref_cases.random_robot_state(k, E), 1.0 / 250.0, 6, 60, 20)
       for k in (0, 1, 3, 7)},
}
# Runs large enough for the reference to take its tree broadphase (B^2 E > 2^20, ops/broadphase.cu:581): kept as per-env
# digests of the candidate pairs and contact counts (tests/refparity.py:pair_digests) plus the poses of the first 128 envs
# (name: scene case, envs, dt, iterations, steps, sampling stride, start state)
LARGE = {"pile12_tree": ("pile12", 8192, 1.0 / 240.0, 8, 30, 10, lambda E: {"body_pose": T.box_pile_state(E, 0, count=12)["body_pose"]})}
SCENE_OF = {"quadruped_moving": "quadruped", "arm7_ct": "arm7", "quadruped_ct": "quadruped", "quadruped_torque": "quadruped",
            "quadruped_velocity": "quadruped", "quadruped_actuator": "quadruped", "arm7_osc": "arm7", "quadruped_osc": "quadruped"}
CONTROL_MODE = {"arm7_ct": 3, "quadruped_ct": 3, "quadruped_torque": 1, "quadruped_velocity": 2, "quadruped_actuator": 5,
                "arm7_osc": 4, "quadruped_osc": 4}
TASK_LINK = {"arm7_osc": 7, "quadruped_osc": 3}
STATE_FIELDS = ("q", "qdot", "base_pose", "link_velocity", "body_pose", "drive_target", "vel_target", "acc_target", "kp", "kd", "force_limit",
                "noload_speed", "feedforward", "task_target", "task_rotation", "task_frame", "null_kp", "null_kd")
# throughput of the reference on the other configurations, on the protocol of bench.py --workload: the same seeded
# per-env start states, the same untimed settle steps, then the timed steps
# (scene case, envs, dt, iterations, settle steps, timed steps, start state)
TIMINGS = [("humanoid", 8192, 1.0 / 200.0, 8, 300, 30, lambda E: T.humanoid_state(E, 0)),
           ("quadbox", 8192, 1.0 / 200.0, 4, 300, 30, lambda E: T.quadruped_state(E, 0)),
           ("pile48", 16384, 1.0 / 240.0, 8, 240, 20, lambda E: {"body_pose": T.box_pile_state(E, 0)["body_pose"]})]


def prepare():
    os.makedirs(RUN, exist_ok=True)
    lines = ["#!/bin/bash", "# written by tests/golden/make_ref_gpu_vectors.py", 'cd "$(dirname "$0")"',
             'OUT="${OUT:-../../../gpurun_out}"', 'mkdir -p "$OUT"', ': > "$OUT/ref_timing.jsonl"']
    for name, (make, state, dt, iters, steps, every) in CASES.items():
        tb = make()
        with open(os.path.join(RUN, f"{name}.nks"), "w") as f:
            json.dump(nks.scene_from_builder(tb), f)
        scene = SCENE_OF.get(name, name)
        shutil.copy(os.path.join(RUN, f"{name}.nks"), os.path.join(HERE, f"scene_{scene}.nks"))
        st = {k: np.ascontiguousarray(v, np.float32).reshape(ENVS, -1) for k, v in state(ENVS).items() if k in STATE_FIELDS}
        with open(os.path.join(RUN, f"{name}_state.nkt"), "wb") as f:
            f.write(nkt.pack(st))
        subprocess.run([DRIVER, "--scene", os.path.join(RUN, f"{name}.nks"), "--envs", "1", "--cook-only", "--dump",
                        os.path.join(HERE, f"ref_cook_{scene}.nkt")], check=True, stdout=subprocess.DEVNULL)
        mode = f" --control-mode {CONTROL_MODE[name]}" if name in CONTROL_MODE else ""
        if name in TASK_LINK:
            mode += f" --task-link {TASK_LINK[name]}"
        lines.append(f"../ref_driver --scene {name}.nks --envs {ENVS} --dt {dt!r} --vel-iters {iters}{mode} --state {name}_state.nkt "
                     f"--steps {steps} --every {every} --dump \"$OUT/ref_{name}.nkt\"")
    for name, (scene, envs, dt, iters, steps, every, state) in LARGE.items():
        st = {k: np.ascontiguousarray(v, np.float32).reshape(envs, -1) for k, v in state(envs).items()}
        with open(os.path.join(RUN, f"{name}_state.nkt"), "wb") as f:
            f.write(nkt.pack(st))
        lines.append(f"../ref_driver --scene {scene}.nks --envs {envs} --dt {dt!r} --vel-iters {iters} --state {name}_state.nkt "
                     f"--steps {steps} --every {every} --dump \"$OUT/ref_{name}.nkt\"")
    # the number to beat: the reference's own step on the bench workload, eager and graph mode, 100 warm-up + 1000 timed steps
    with open(os.path.join(RUN, "quadruped_state4096.nkt"), "wb") as f:
        st = T.quadruped_state(4096, 0)
        f.write(nkt.pack({k: np.ascontiguousarray(st[k], np.float32) for k in ("q", "base_pose")}))
    lines.append('../ref_driver --scene quadruped.nks --envs 4096 --dt 0.005 --vel-iters 4 --state quadruped_state4096.nkt '
                 '--time 100,1000,3 >> "$OUT/ref_timing.jsonl"')
    # the same after 1000 settle steps (the prepared state bench.py measures on): 1000 untimed, then 200 timed
    lines.append('../ref_driver --scene quadruped.nks --envs 4096 --dt 0.005 --vel-iters 4 --state quadruped_state4096.nkt '
                 '--time 1000,200,1 --active 0.15 >> "$OUT/ref_timing.jsonl"')
    with open(os.path.join(RUN, "pile48.nks"), "w") as f:
        json.dump(nks.scene_from_builder(T.box_pile(0, count=48)), f)
    split = len(lines)
    for scene, envs, dt, iters, warm, timed, state in TIMINGS:
        st = {k: np.ascontiguousarray(v, np.float32).reshape(envs, -1) for k, v in state(envs).items() if k in ("q", "qdot", "base_pose", "body_pose")}
        with open(os.path.join(RUN, f"{scene}_state{envs}.nkt"), "wb") as f:
            f.write(nkt.pack(st))
        lines.append(f'timeout 600 ../ref_driver --scene {scene}.nks --envs {envs} --dt {dt!r} --vel-iters {iters} --state {scene}_state{envs}.nkt '
                     f'--time {warm},{timed},1 >> "$OUT/ref_timing.jsonl" || echo "{{\\"scene\\": \\"{scene}.nks\\", \\"envs\\": {envs}, \\"failed\\": $?}}" >> "$OUT/ref_timing.jsonl"')
    # run.sh does everything; timings.sh only the throughput lines of the other configurations (appending)
    with open(os.path.join(RUN, "timings.sh"), "w") as f:
        f.write("\n".join(lines[:5] + lines[split:]) + "\n")
    with open(os.path.join(RUN, "run.sh"), "w") as f:
        f.write("\n".join(lines) + "\n")
    print("prepared", RUN)


KEEP = ("run", "run_dt", "dyn_qddot", "dyn_mass", "dyn_bias", "start_link_pose", "start_kp", "start_kd", "start_force_limit",
        "start_drive_target", "traj_steps", "traj_q", "traj_qdot", "traj_base_pose", "traj_status", "traj_status_any",
        "traj_solver_sweeps", "traj_solver_residual", "traj_pair_count", "traj_candidate_pairs", "traj_contact_count")
FREE_BODY_CASES = ("pile12", "quadbox", "cylinders", "random0", "random1", "random3", "random7")     # body poses are kept where free bodies carry state of their own


def collect(src):
    """Keeps what the tests compare (the root twist of the link velocities; body poses only where free bodies exist) as
    compressed .npz files."""
    for name in CASES:
        if not os.path.exists(os.path.join(src, f"ref_{name}.nkt")):     # a partial run: keep the vectors already collected
            continue
        with open(os.path.join(src, f"ref_{name}.nkt"), "rb") as f:
            arrays = nkt.unpack(f.read())
        E, L = int(arrays["run"][0]), int(arrays["run"][1])
        out = {k: arrays[k] for k in KEEP if k in arrays}
        samples = len(arrays["traj_steps"])
        if name in FREE_BODY_CASES:
            out["traj_body_pose"] = arrays["traj_body_pose"]
        if L:
            out["traj_root_twist"] = arrays["traj_link_velocity"].reshape(samples, E, L, 6)[:, :, 0].copy()
        np.savez_compressed(os.path.join(HERE, f"ref_gpu_{name}.npz"), **out)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import refparity
    for name in LARGE:
        path = os.path.join(src, f"ref_{name}.nkt")
        if not os.path.exists(path):
            continue
        with open(path, "rb") as f:
            arrays = nkt.unpack(f.read())
        E, B, S = int(arrays["run"][0]), int(arrays["run"][3]), int(arrays["run"][4])
        K = len(arrays["traj_steps"])
        digests = [refparity.pair_digests(arrays["traj_pair_count"].reshape(K, E)[i], arrays["traj_candidate_pairs"].reshape(K, E, S, 2)[i],
                                          arrays["traj_contact_count"].reshape(K, E, S)[i]) for i in range(K)]
        np.savez_compressed(os.path.join(HERE, f"ref_gpu_{name}.npz"), run=arrays["run"], run_dt=arrays["run_dt"], traj_steps=arrays["traj_steps"],
                            traj_pair_count=arrays["traj_pair_count"].reshape(K, E), traj_status=arrays["traj_status"].reshape(K, E),
                            pair_digest=np.stack([d[0] for d in digests]), contact_digest=np.stack([d[1] for d in digests]),
                            traj_body_pose_head=arrays["traj_body_pose"].reshape(K, E, B * 7)[:, :128].copy())
    if not os.path.exists(os.path.join(src, "ref_timing.jsonl")):
        print("collected into", HERE, "(no timing file in", src + ")")
        return
    with open(os.path.join(src, "ref_timing.jsonl")) as f:
        lines = [line for line in f if line.startswith("{")]
    with open(os.path.join(HERE, "ref_gpu_timing.jsonl"), "w") as f:
        f.writelines(lines)
    print("collected into", HERE)


if __name__ == "__main__":
    if len(sys.argv) >= 2 and sys.argv[1] == "prepare":
        prepare()
    elif len(sys.argv) >= 2 and sys.argv[1] == "collect":
        collect(sys.argv[2] if len(sys.argv) > 2 else os.path.join(ROOT, "gpurun_out"))
    else:
        raise SystemExit(__doc__)

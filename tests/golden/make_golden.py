"""Regenerates the golden fixtures from the CPU oracle:  python tests/golden/make_golden.py

The fixtures hold seeded inputs and the oracle's outputs for small cases of the benchmark configurations, so
the CUDA path can be checked on a machine where only the committed files exist.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "nuka-physics_b200"))
sys.path.insert(0, os.path.join(ROOT, "oracle"))

import orc  # noqa: E402
from nuka import templates as T  # noqa: E402


def arm7():
    E = 4
    tb = T.arm7(0)
    st = T.arm7_state(E, 0)
    w = orc.World(tb.blob(), E)
    w.set("q", st["q"]); w.set("qdot", st["qdot"]); w.refresh()
    w.dynamics(False)
    out = {"q_in": st["q"], "qdot_in": st["qdot"], "mass": w.get("mass_matrix", 49), "qdd": w.get("qddot", 8),
           "link_pose": w.get("link_pose", 56)}
    w.step(100)
    out.update(q_100=w.get("q", 8), qdot_100=w.get("qdot", 8))
    np.savez(os.path.join(HERE, "arm7_seed0.npz"), **out)


def quadruped():
    E = 4
    tb = T.quadruped(0)
    st = T.quadruped_state(E, 0)
    rng = np.random.Generator(np.random.PCG64(7))
    qdot = np.zeros((E, 13), np.float32)
    qdot[:, 1:] = rng.normal(0, 0.5, size=(E, 12))
    lv = np.zeros((E, 13, 6), np.float32)
    lv[:, 0, :] = rng.normal(0, 0.3, size=(E, 6))
    w = orc.World(tb.blob(), E)
    w.set("q", st["q"]); w.set("qdot", qdot); w.set("base_pose", st["base_pose"]); w.set("link_velocity", lv.reshape(E, -1)); w.refresh()
    w.dynamics(False)
    out = {"q_in": st["q"], "qdot_in": qdot, "base_in": st["base_pose"], "link_vel_in": lv.reshape(E, -1),
           "mass": w.get("mass_matrix", 324), "qdd": w.get("qddot", 13)}
    w2 = orc.World(tb.blob(), E)
    w2.set("q", st["q"]); w2.set("qdot", qdot); w2.set("base_pose", st["base_pose"]); w2.set("link_velocity", lv.reshape(E, -1)); w2.refresh()
    w2.collide()
    out.update(pair_count=w2.get("pair_count", 1), pairs=w2.get("candidate_pairs", 16), contact_count=w2.get("contact_count", 8),
               contact_depth=w2.get("contact_depth", 32))
    w3 = orc.World(tb.blob(), E)
    w3.set("q", st["q"]); w3.set("qdot", qdot); w3.set("base_pose", st["base_pose"]); w3.set("link_velocity", lv.reshape(E, -1)); w3.refresh()
    w3.step(1)
    out.update(qdot_1=w3.get("qdot", 13), link_vel_1=w3.get("link_velocity", 78), q_1=w3.get("q", 13), base_1=w3.get("base_pose", 7))
    np.savez(os.path.join(HERE, "quadruped_seed0.npz"), **out)


if __name__ == "__main__":
    orc.build()
    arm7()
    quadruped()
    print("golden fixtures written to", HERE)

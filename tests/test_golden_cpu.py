"""The committed golden fixtures are what the oracle produces today (guards against silent oracle drift)."""
import os

import numpy as np

from nuka import templates as T

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_arm7_fixture(oracle):
    g = np.load(os.path.join(GOLDEN, "arm7_seed0.npz"))
    w = oracle.World(T.arm7(0).blob(), 4)
    w.set("q", g["q_in"]); w.set("qdot", g["qdot_in"]); w.refresh()
    w.dynamics(False)
    assert np.array_equal(w.get("mass_matrix", 49), g["mass"]) and np.array_equal(w.get("qddot", 8), g["qdd"])
    w.step(100)
    assert np.array_equal(w.get("q", 8), g["q_100"])


def test_quadruped_fixture(oracle):
    g = np.load(os.path.join(GOLDEN, "quadruped_seed0.npz"))
    w = oracle.World(T.quadruped(0).blob(), 4)
    w.set("q", g["q_in"]); w.set("qdot", g["qdot_in"]); w.set("base_pose", g["base_in"]); w.set("link_velocity", g["link_vel_in"]); w.refresh()
    w.step(1)
    assert np.array_equal(w.get("qdot", 13), g["qdot_1"]) and np.array_equal(w.get("base_pose", 7), g["base_1"])

"""The .nks cooker on a scene document written here in the reference's schema (no reference files needed)."""
import json

import numpy as np

from nuka import nks, templates as T


def _scene():
    shape = lambda kind, **kw: dict(type=kind, local=kw.pop("local", {"pos": [0, 0, 0], "quat": [1, 0, 0, 0]}), contype=1, conaffinity=1,  # noqa: E731
                                    friction_mu=kw.pop("mu", 0.7), half_extents=kw.pop("he", [0.5] * 3), radius=kw.pop("r", 0.5),
                                    half_height=kw.pop("hh", 0.5))
    leg = dict(name="leg", transform={"pos": [0.2, 0.0, -0.1], "quat": [1, 0, 0, 0]},
               rigid_body={"mass": 1.5, "inertia": [0.01, 0.02, 0.03], "is_static": False,
                           "inertial": {"pos": [0.0, 0.0, -0.1], "quat": [0.7071068, 0.0, 0.7071068, 0.0]}},
               joint={"type": "revolute", "axis": [0, 1, 0], "lower_limit": -1.0, "upper_limit": 2.0, "damping": 0.5, "armature": 0.01,
                      "initial_position": 0.3, "parent_frame": {"pos": [0.0, 0.05, 0.0], "quat": [1, 0, 0, 0]},
                      "child_frame": {"pos": [0, 0, 0], "quat": [1, 0, 0, 0]}},
               children=[dict(name="g0", collision_shape=shape("capsule", r=0.03, hh=0.1, local={"pos": [0, 0, -0.1], "quat": [1, 0, 0, 0]})),
                         dict(name="g1", collision_shape=shape("sphere", r=0.04, local={"pos": [0, 0, -0.2], "quat": [1, 0, 0, 0]}, mu=0.9))])
    base = dict(name="base", transform={"pos": [0, 0, 0.5], "quat": [1, 0, 0, 0]},
                rigid_body={"mass": 4.0, "inertia": [0.1, 0.2, 0.3], "is_static": False, "inertial": {"pos": [0.01, 0, 0], "quat": [1, 0, 0, 0]}},
                children=[dict(name="g", collision_shape=shape("box", he=[0.2, 0.1, 0.05])), dict(name="mesh", visual_mesh={}), leg])
    return {"nks_version": 1, "tree": [base]}


def test_cook_builds_links_shapes_and_exclusions(tmp_path):
    path = tmp_path / "robot.nks"
    path.write_text(json.dumps(_scene()))
    tb = nks.cook(str(path), dt=0.005, kp=30.0, kd=1.0)
    a = tb.arrays()
    assert list(a["jtype"]) == [T.FLOATING, T.REVOLUTE] and T.dof_count(a) == 7
    assert list(a["shape_kind"]) == [T.BOX, T.CAPSULE, T.SPHERE, T.PLANE] and list(a["body_to_link"][:3]) == [0, 1, 1]
    assert np.allclose(a["base_pose0"], [0, 0, 0.5, 1, 0, 0, 0])
    assert np.allclose(a["local_pos"][3:], [0.2, 0.0, -0.1]) and np.allclose(a["parent_offset"][3:], [0.0, 0.05, 0.0])
    assert np.allclose(a["q0"], [0, 0.3]) and np.allclose(a["kp0"], [0, 30.0]) and np.allclose(a["limit_lower"][1], -1.0)
    assert a["limit_flags"][1] == 3 and np.isclose(a["damping"][1], 0.5) and np.isclose(a["armature"][1], 0.01)
    # the inertial frame is rotated 90 degrees about y: principal x and z swap in link axes
    I = a["inertia"].reshape(2, 6, 6)[1]
    com = np.array([0.0, 0.0, -0.1])
    want = np.diag([0.03, 0.02, 0.01]) + 1.5 * (com.dot(com) * np.eye(3) - np.outer(com, com))
    assert np.allclose(I[:3, :3], want, atol=1e-6) and np.allclose(I[3:, 3:], 1.5 * np.eye(3))
    # per-row shape frames and exclusions: nothing pairs inside the leg or between leg and base
    assert np.allclose(a["body_geom_pos"].reshape(4, 3)[2], [0, 0, -0.2]) and np.isclose(a["mu"][2], 0.9)
    keys = {(int(k) >> 32, int(k) & 0xffffffff) for k in a["excluded"]}
    assert keys == {(0, 1), (0, 2), (1, 2)}
    assert a["cfg_u"][2] == 3 and nks.link_names(str(path)) == ["base", "leg"]


def test_cooked_scene_runs_in_the_oracle(oracle, tmp_path):
    tb = nks.cook(_scene(), dt=0.005)
    E = 3
    o = oracle.World(tb.blob(), E)
    o.step(200)
    assert o.get("env_status", 1).max() == 0
    assert np.isfinite(o.get("base_pose", 7)).all() and o.get("pair_count", 1).max() >= 1


def test_contact_point_capacity_travels_in_the_template(tmp_path):
    """The cooker's max_points option becomes the template's optional max_points record (absent by default); the Go2
    fixture carries 32."""
    import os
    from nuka import nkt
    assert "max_points" not in nks.cook(_scene()).arrays()
    arrays = nkt.unpack(nks.cook(_scene(), max_points=12).blob())
    assert arrays["max_points"].tolist() == [12]
    out = tmp_path / "robot.nkt"
    path = tmp_path / "robot.nks"
    path.write_text(json.dumps(_scene()))
    nks.main([str(path), str(out), "--max-points", "20"])
    assert nkt.unpack(out.read_bytes())["max_points"].tolist() == [20]
    fixture = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "go2.nkt")
    with open(fixture, "rb") as f:
        assert nkt.unpack(f.read())["max_points"].tolist() == [32]


def test_link_names_travel_in_the_template():
    """The cooked template names every link after the joint whose child it is (the root after its body), NUL-terminated in
    one word record; templates built without names carry no such record."""
    import os
    from nuka import templates as T
    scene = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "scene_quadruped.nks")
    a = nks.cook(scene).arrays()
    names = a["link_names"].tobytes().split(b"\0")[:13]
    assert [n.decode() for n in names] == ["link0"] + [f"joint{i}" for i in range(1, 13)]
    assert "link_names" not in T.quadruped(0).arrays()

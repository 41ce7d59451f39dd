"""The library's own scene cooker (csrc/nkb_scene.cpp, what nuka_world_create_from_scene runs on a `.nks` path) against
the Python cooker of the same rules (nuka/nks.py), array by array, on every scene file the reference itself was run on;
plus the cooker's error behaviour.  No device is needed: cooking is host work."""
import json
import os

import numpy as np
import pytest

import nuka
from nuka import nks, nkt

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
SCENES = ["arm7", "quadruped", "humanoid", "pile12", "quadbox", "cylinders", "random0", "random1", "random3", "random7"]


def compare(native_bytes, tb):
    mine, want = nkt.unpack(native_bytes), tb.arrays()
    assert set(mine) == set(want)
    for name, w in want.items():
        m = mine[name]
        assert m.dtype == w.dtype and m.shape == w.shape, name
        if w.dtype == np.float32:
            # both cookers compute in double and round once; a product order may differ in the last bit
            assert np.allclose(m, w, rtol=2e-7, atol=1e-12), name
        else:
            assert np.array_equal(m, w), name


@pytest.mark.parametrize("scene", SCENES)
def test_reference_semantics_match_the_python_cooker(scene):
    """The defaults of the in-library cooker: drives from the scene's actuators only, the scene's own ground and filter bits."""
    path = os.path.join(GOLDEN, f"scene_{scene}.nks")
    text = open(path).read()
    slots = 7
    native = nks.cook_native(text, dt=1.0 / 240.0, velocity_iterations=6, max_contacts=slots, max_points=33)
    tb = nks.cook(path, dt=1.0 / 240.0, vel_iters=6, kp=0.0, kd=0.0, scene_filters=True, ground_height=None, max_contacts=slots, max_points=33)
    compare(native, tb)


@pytest.mark.parametrize("scene", ["quadruped", "humanoid"])
def test_robot_versus_ground_options_match_the_python_cooker(scene):
    """The offline cooker's defaults: hold drives on every scalar joint, robot rows that meet the ground only, one slot per
    shape row."""
    path = os.path.join(GOLDEN, f"scene_{scene}.nks")
    native = nks.cook_native(open(path).read(), default_kp=60.0, default_kd=2.0, scene_filters=0, self_collision=0, max_contacts=0)
    compare(native, nks.cook(path))


def test_every_admissible_pair_gets_a_slot():
    """The reference sizes its candidate slots as the number of pairs its filters admit (cook_to_model.cpp:1541-1546); the
    reference's own cook of these scenes reported 5, 78, 35 and 54 slots per env."""
    for scene, slots in (("quadruped", 5), ("pile12", 78), ("quadbox", 35), ("humanoid", 54)):
        arrays = nkt.unpack(nks.cook_native(open(os.path.join(GOLDEN, f"scene_{scene}.nks")).read()))
        assert int(arrays["cfg_u"][2]) == slots, scene


def test_a_scene_with_more_pairs_than_slots_is_refused_by_the_template_check():
    """48 boxes and a plane admit 1176 pairs; the path holds 1024 candidate slots per env, so the reference's budget of one
    slot per admissible pair does not fit and the cooked template says so at the check (a caller can cook with its own
    max_contacts instead)."""
    from nuka import templates as T
    text = json.dumps(nks.scene_from_builder(T.box_pile(0, count=48)))
    lib = nuka._abi.lib()
    blob = nks.cook_native(text)
    assert int(nkt.unpack(blob)["cfg_u"][2]) == 1176
    assert lib.nuka_b200_template_check(blob, len(blob)) == nuka._abi.NOT_SUPPORTED
    blob = nks.cook_native(text, max_contacts=288, max_points=288)
    assert lib.nuka_b200_template_check(blob, len(blob)) == 0


def test_cooked_scene_passes_the_template_check():
    lib = nuka._abi.lib()
    for scene in SCENES:
        blob = nks.cook_native(open(os.path.join(GOLDEN, f"scene_{scene}.nks")).read())
        assert lib.nuka_b200_template_check(blob, len(blob)) == 0, scene


def test_scene_errors_are_reported_not_thrown():
    scene = json.load(open(os.path.join(GOLDEN, "scene_quadruped.nks")))
    with pytest.raises(nuka.NukaError) as e:
        nks.cook_native("{ \"nks_version\": 1, \"tree\": [")
    assert e.value.code == 5                                   # NUKA_RESULT_PARSE_ERROR
    bad = json.loads(json.dumps(scene))
    bad["nks_version"] = 2
    with pytest.raises(nuka.NukaError) as e:
        nks.cook_native(json.dumps(bad))
    assert e.value.code == 7                                   # NUKA_RESULT_NOT_SUPPORTED
    bad = json.loads(json.dumps(scene))
    shape = next(c for c in bad["tree"][0]["children"] if "collision_shape" in c)
    shape["collision_shape"]["type"] = "convex_hull"
    with pytest.raises(nuka.NukaError) as e:
        nks.cook_native(json.dumps(bad))
    assert e.value.code == 7 and "convex_hull" in str(e.value)
    with pytest.raises(nuka.NukaError) as e:
        nks.cook_native(json.dumps(scene), dt=0.0)
    assert e.value.code == 1                                   # NUKA_RESULT_INVALID_ARG

"""Cooks the reference's Go2 scene (examples/scenes/go2.nks) into tests/golden/go2.nkt.

Run with NUKA_REFERENCE_ROOT pointing at a checkout of the reference; tests only need the cooked template.  The scene's joint
positions are all zero, which violates the calf limits, so the template starts from the robot's usual standing
pose (hip 0, thigh 0.9, calf -1.8 rad, base 0.30 m above the ground) and its drives hold that pose.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "nuka-physics_b200"))

from nuka import nks  # noqa: E402

SCENE = os.path.join(os.environ.get("NUKA_REFERENCE_ROOT", ""), "examples", "scenes", "go2.nks")
STANCE = {"hip": 0.0, "thigh": 0.9, "calf": -1.8}


def main():
    # 32 contact points per env: four feet plus every other segment lying on the ground needs 24
    tb = nks.cook(SCENE, dt=1.0 / 200.0, vel_iters=4, kp=60.0, kd=2.0, max_points=32)
    names = nks.link_names(SCENE)
    for link, name in zip(tb.links, names):
        for key, angle in STANCE.items():
            if name.endswith(key):
                link["q0"] = angle
    tb.base_pose[2] = 0.30
    out = os.path.join(HERE, "go2.nkt")
    with open(out, "wb") as f:
        f.write(tb.blob())
    print(out, os.path.getsize(out), "bytes;", len(tb.links), "links,", len(tb.bodies), "collidable rows")


if __name__ == "__main__":
    main()

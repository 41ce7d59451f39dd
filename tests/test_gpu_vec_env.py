"""The RL step loop over a world: action write, decimated stepping, GPU observations, autoreset."""
import numpy as np
import pytest

import nuka
from nuka import Field as F, shard, templates as T
from nuka.vec_env import NukaVecEnv

pytestmark = pytest.mark.gpu


def test_step_loop_shapes_reset_and_autoreset(device):
    torch = pytest.importorskip("torch")
    E = 64
    env = NukaVecEnv(device, T.quadruped(0).blob(), E, decimation=4, episode_length_s=0.4)      # 20 control steps per episode
    obs0 = env.reset()
    assert obs0.shape == (E, shard.OBS_FLOATS) and env.num_joints == 12
    gen = torch.Generator(device="cuda").manual_seed(0)
    resets = 0
    for k in range(45):
        actions = 0.2 * torch.randn((E, 12), generator=gen, device="cuda")
        obs, reward, terminated, truncated, info = env.step(actions)
        assert obs.shape == (E, shard.OBS_FLOATS) and reward.shape == (E,)
        assert torch.isfinite(obs).all() and torch.isfinite(reward).all()
        resets += int(info["done"].sum())
        if k == 19:                                  # every env hits the episode limit together
            assert bool(truncated.all()) and not bool(terminated.any())
            assert torch.equal(obs[:, 12:24], obs0[:, 12:24])      # fresh-episode joint positions (q - default)
            assert bool((obs[:, 36:48] == 0).all())                # and a cleared last action
    assert resets >= 2 * E
    # the last targets written are default + scale * action (the last step reset no env: 45 is not a multiple of 20)
    env.world.synchronize()
    targets = env.world.download(F.DRIVE_TARGET)
    want = env.default_targets.cpu().numpy()[:, 1:] + env.action_scale * actions.cpu().numpy()
    assert np.allclose(targets[:, 1:], want, atol=1e-6)
    assert torch.equal(obs[:, 36:48], actions)                      # the record carries the action just applied
    env.close()


def test_joint_order_permutes_observations_and_actions(device):
    """Caller joint i is library slot joint_order[i] on the way out, and actions go back through the inverse map
    (python/nuka/tasks/go2_obs.py:252-262, 307-325)."""
    torch = pytest.importorskip("torch")
    E = 8
    order = [3, 4, 5, 0, 1, 2, 9, 10, 11, 6, 7, 8]
    env = NukaVecEnv(device, T.quadruped(0).blob(), E, joint_order=order)
    plain = NukaVecEnv(device, T.quadruped(0).blob(), E)
    o1, o0 = env.reset(), plain.reset()
    assert torch.equal(o1[:, :12], o0[:, :12])
    a = 0.3 * torch.randn((E, 12), generator=torch.Generator(device="cuda").manual_seed(1), device="cuda")
    inverse = torch.empty(12, dtype=torch.long); inverse[torch.tensor(order)] = torch.arange(12)
    o1 = env.step(a)[0]
    o0 = plain.step(a[:, inverse.cuda()])[0]                # the same physical targets in the library's own order
    env.world.synchronize(); plain.world.synchronize()
    assert torch.equal(o1[:, 12:24], o0[:, 12:24][:, order]) and torch.equal(o1[:, 24:36], o0[:, 24:36][:, order])
    env.close(); plain.close()


def test_fallen_envs_terminate_and_restart(device):
    torch = pytest.importorskip("torch")
    E = 16
    env = NukaVecEnv(device, T.quadruped(0).blob(), E, termination_height=0.5)       # standing height is below 0.5: all fall
    env.reset()
    obs, reward, terminated, truncated, info = env.step(torch.zeros((E, 12), device="cuda"))
    assert bool(terminated.all()) and int(info["done"].sum()) == E
    assert int(env.episode_steps.max()) == 0
    env.close()

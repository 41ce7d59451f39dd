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
    assert obs0.shape == (E, shard.RECORD_FLOATS) and env.num_joints == 12
    gen = torch.Generator(device="cuda").manual_seed(0)
    resets = 0
    for k in range(45):
        actions = 0.2 * torch.randn((E, 12), generator=gen, device="cuda")
        obs, reward, terminated, truncated, info = env.step(actions)
        assert obs.shape == (E, shard.RECORD_FLOATS) and reward.shape == (E,)
        assert torch.isfinite(obs).all() and torch.isfinite(reward).all()
        resets += int(info["reset_ids"].numel())
        if k == 19:                                  # every env hits the episode limit together
            assert bool(truncated.all()) and not bool(terminated.any())
            assert torch.equal(obs[:, :12], obs0[:, :12])          # fresh-episode joint positions
    assert resets >= 2 * E
    # the last targets written are default + scale * action
    targets = env.world.download(F.DRIVE_TARGET)
    want = env.default_targets.cpu().numpy()[:, 1:] + env.action_scale * actions.cpu().numpy()
    assert np.allclose(targets[:, 1:], want, atol=1e-6)
    env.close()


def test_fallen_envs_terminate_and_restart(device):
    torch = pytest.importorskip("torch")
    E = 16
    env = NukaVecEnv(device, T.quadruped(0).blob(), E, termination_height=0.5)       # standing height is below 0.5: all fall
    env.reset()
    obs, reward, terminated, truncated, info = env.step(torch.zeros((E, 12), device="cuda"))
    assert bool(terminated.all()) and info["reset_ids"].numel() == E
    assert int(env.episode_steps.max()) == 0
    env.close()

"""Vectorised RL env over one world, after the reference's NukaGymEnv step loop (python/nuka/gym/env.py:1-60):

    actions -> DRIVE_TARGET (default pose + scale * action) -> step_n(decimation) -> observations composed on the
    GPU -> reward, termination / truncation -> autoreset of the finished envs through reset_envs, whose fresh
    observations are what the caller gets back for them.

Observations are the library's packed record (nuka_b200_world_pack_observations: joint positions and velocities,
base pose, root twist, previous targets, base height).  The reward is a plain standing/forward-velocity term;
tasks replace ``compute_reward``.  Needs torch with CUDA; no gymnasium dependency.
"""
import math

import numpy as np

from . import Field, World


class NukaVecEnv:
    def __init__(self, device, template_blob, num_envs, decimation=4, action_scale=0.25, command=(0.5, 0.0, 0.0),
                 termination_height=0.18, termination_tilt_deg=75.0, episode_length_s=20.0):
        import torch
        self._torch = torch
        self.num_envs = int(num_envs)
        self.decimation = int(decimation)
        self.action_scale = float(action_scale)
        self.world = World.create_from_template(device, template_blob, self.num_envs)
        info = self.world.info
        self.num_joints = info.links_per_env - 1
        self.dt = float(self.world.dt) if hasattr(self.world, "dt") else None
        self.obs_width = self.world.observation_width()
        self.command = torch.tensor(command, dtype=torch.float32, device="cuda")
        self.termination_height = float(termination_height)
        self.min_up = math.cos(math.radians(termination_tilt_deg))
        self._targets = self.world.view(Field.DRIVE_TARGET).torch()
        self._base = self.world.view(Field.BASE_POSE).torch()
        self._link_velocity = self.world.view(Field.LINK_VELOCITY).torch()
        self._status = self.world.view(Field.ENV_STATUS).torch()
        self.default_targets = self._targets.clone()
        self.obs = torch.zeros((self.num_envs, self.obs_width), dtype=torch.float32, device="cuda")
        self.episode_steps = torch.zeros(self.num_envs, dtype=torch.int32, device="cuda")
        self._episode_length_s = float(episode_length_s)
        self.max_episode_length = None

    # ---- helpers -------------------------------------------------------------------------------------------
    def _stream(self):
        torch = self._torch
        import ctypes
        from . import _abi, _check
        ptr = ctypes.c_void_p()
        _check(_abi.lib().nuka_world_get_stream(self.world._h, ctypes.byref(ptr)))
        return torch.cuda.ExternalStream(ptr.value)

    def _compose(self):
        self.world.pack_observations(self.obs)
        return self.obs

    def compute_reward(self):
        """Forward-velocity tracking minus a height penalty; root twist is (angular, linear) in the base frame."""
        torch = self._torch
        forward = self._link_velocity[:, 3]
        track = torch.exp(-4.0 * (forward - self.command[0]) ** 2)
        return track - 2.0 * torch.clamp(0.25 - self._base[:, 2], min=0.0)

    def _up_axis_z(self):
        # z component of the base frame's up axis from the base quaternion (w, x, y, z)
        q = self._base[:, 3:7]
        return 1.0 - 2.0 * (q[:, 1] ** 2 + q[:, 2] ** 2)

    # ---- gym-style surface ---------------------------------------------------------------------------------
    def reset(self):
        torch = self._torch
        with torch.cuda.stream(self._stream()):
            self.world.reset()
            self._targets.copy_(self.default_targets)
            self.episode_steps.zero_()
            obs = self._compose().clone()
        self.world.synchronize()
        return obs

    def step(self, actions, control_dt=None):
        """``actions``: E x num_joints CUDA float tensor.  Returns (obs, reward, terminated, truncated, info)."""
        torch = self._torch
        if self.max_episode_length is None:
            control_dt = control_dt if control_dt is not None else 0.005 * self.decimation
            self.max_episode_length = max(1, int(round(self._episode_length_s / control_dt)))
        with torch.cuda.stream(self._stream()):
            self._targets[:, 1:] = self.default_targets[:, 1:] + self.action_scale * actions
            self.world.step_n(self.decimation)
            self.episode_steps += 1
            reward = self.compute_reward()
            fallen = (self._base[:, 2] < self.termination_height) | (self._up_axis_z() < self.min_up) | (self._status != 0).reshape(-1)
            truncated = self.episode_steps >= self.max_episode_length
            done = fallen | truncated
            obs = self._compose()
            ids = torch.nonzero(done).reshape(-1)
        self.world.synchronize()
        if ids.numel() > 0:
            host_ids = ids.to("cpu").numpy().astype(np.uint32)
            self.world.reset_envs(host_ids)
            with torch.cuda.stream(self._stream()):
                self._targets[ids] = self.default_targets[ids]
                self.episode_steps[ids] = 0
                obs = self._compose()              # finished envs report their fresh-episode observation
            self.world.synchronize()
        return obs.clone(), reward, fallen, truncated & ~fallen, {"reset_ids": ids}

    def close(self):
        self.world.destroy()

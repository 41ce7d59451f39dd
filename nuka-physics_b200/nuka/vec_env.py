"""Vectorised RL env over one world, after the reference's NukaGymEnv step loop (python/nuka/gym/env.py:1-21):

    actions -> DRIVE_TARGET (default pose + 0.25 x action, caller joint order through the permutation table)
    -> step_n(decimation) -> reward, termination / truncation on the GPU -> autoreset of the finished envs
    -> the 48-float observation record of python/nuka/tasks/go2_obs.py:11-20, composed by one kernel
       (nuka_b200_world_pack_observations); finished envs report their fresh-episode observation.

Everything between two calls of step() stays on the world's stream: the finished envs are reset through a device
mask (nuka_b200_world_reset_envs_masked), so no id list travels to the host and nothing synchronises.  The reward
is a plain forward-velocity / height term; tasks replace ``compute_reward``.  Needs torch with CUDA; no gymnasium
dependency.
"""
import math

from . import Field, World

ACTION_SCALE = 0.25         # python/nuka/tasks/go2_obs.py:64
ACTION_CLIP = 100.0         # python/nuka/tasks/go2_obs.py:66


class NukaVecEnv:
    def __init__(self, device, template_blob, num_envs, decimation=4, action_scale=ACTION_SCALE, command=(0.5, 0.0, 0.0),
                 termination_height=0.18, termination_tilt_deg=75.0, episode_length_s=20.0, joint_order=None):
        import torch
        self._torch = torch
        self.num_envs = int(num_envs)
        self.decimation = int(decimation)
        self.action_scale = float(action_scale)
        self.world = World.create_from_template(device, template_blob, self.num_envs)
        info = self.world.info
        self.num_joints = info.links_per_env - 1
        self.dt = float(info.fixed_dt)
        self.control_dt = self.dt * self.decimation
        self.max_episode_length = max(1, int(round(float(episode_length_s) / self.control_dt)))
        self.obs_width = self.world.observation_width()
        cuda = torch.device("cuda", device.gpu_index)
        self._stream_obj = self._stream()
        self.command = torch.tensor(command, dtype=torch.float32, device=cuda)
        self.termination_height = float(termination_height)
        self.min_up = math.cos(math.radians(termination_tilt_deg))
        self._targets = self.world.view(Field.DRIVE_TARGET).torch()
        self._base = self.world.view(Field.BASE_POSE).torch()
        self._link_velocity = self.world.view(Field.LINK_VELOCITY).torch()
        self._status = self.world.view(Field.ENV_STATUS).torch()
        # joint_order[i] = library joint slot of the caller's joint i (the reference's urdf_from_nuka_slot table,
        # python/nuka/tasks/go2_obs.py:252-262); identity when the template already uses the caller's order
        order = list(range(self.num_joints)) if joint_order is None else [int(j) for j in joint_order]
        if sorted(order) != list(range(self.num_joints)):
            raise ValueError("joint_order must be a permutation of the actuated joints")
        self.joint_order = torch.tensor(order, dtype=torch.int32, device=cuda)
        self._order_long = self.joint_order.long()
        self._slot_for_joint = torch.empty_like(self._order_long)
        self._slot_for_joint[self._order_long] = torch.arange(self.num_joints, device=cuda)
        self.default_targets = self._targets.clone()
        self.default_position = self.default_targets[0, 1:].index_select(0, self._order_long).contiguous()
        self.last_action = torch.zeros((self.num_envs, self.num_joints), dtype=torch.float32, device=cuda)
        self.obs = torch.zeros((self.num_envs, self.obs_width), dtype=torch.float32, device=cuda)
        self.episode_steps = torch.zeros(self.num_envs, dtype=torch.int32, device=cuda)
        self._done_mask = torch.zeros(self.num_envs, dtype=torch.int32, device=cuda)
        self._obs_desc = self.world.observation_desc(self.command, last_action=self.last_action, default_position=self.default_position,
                                                     joint_order=self.joint_order)

    # ---- helpers -------------------------------------------------------------------------------------------
    def _stream(self):
        torch = self._torch
        import ctypes
        from . import _abi, _check
        ptr = ctypes.c_void_p()
        _check(_abi.lib().nuka_world_get_stream(self.world._h, ctypes.byref(ptr)))
        return torch.cuda.ExternalStream(ptr.value)

    def _compose(self):
        self.world.pack_observations(self._obs_desc, self.obs)
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
        with torch.cuda.stream(self._stream_obj):
            self.world.reset()
            self._targets.copy_(self.default_targets)
            self.episode_steps.zero_()
            self.last_action.zero_()
            obs = self._compose().clone()
        self.world.synchronize()
        obs.record_stream(torch.cuda.current_stream())
        return obs

    def step(self, actions):
        """``actions``: E x num_joints CUDA float tensor in the caller's joint order.  Returns (obs, reward, terminated,
        truncated, info).  The work runs on the world's stream; the caller's current stream is ordered behind it on the
        device (stream waits, no host synchronisation), so the returned tensors can be used there directly."""
        torch = self._torch
        caller = torch.cuda.current_stream()
        self._stream_obj.wait_stream(caller)           # the actions were produced on the caller's stream
        with torch.cuda.stream(self._stream_obj):
            action = actions.clamp(-ACTION_CLIP, ACTION_CLIP)
            target = self.default_position + self.action_scale * action            # caller joint order
            self._targets[:, 1:] = target.index_select(1, self._slot_for_joint)    # -> library slots (go2_obs.py:307-325)
            self.last_action.copy_(action)
            self.world.step_n(self.decimation)
            self.episode_steps += 1
            reward = self.compute_reward()
            fallen = (self._base[:, 2] < self.termination_height) | (self._up_axis_z() < self.min_up) | (self._status != 0).reshape(-1)
            truncated = self.episode_steps >= self.max_episode_length
            done = fallen | truncated
            # autoreset on the device: mask -> reset kernel -> refreshed poses, then the per-episode bookkeeping
            self._done_mask.copy_(done)
            self.world.reset_envs_masked(self._done_mask)
            keep = (~done).unsqueeze(1)
            self._targets.copy_(torch.where(keep, self._targets, self.default_targets))
            self.last_action.mul_(keep)
            self.episode_steps.mul_(~done)
            obs = self._compose().clone()              # finished envs report their fresh-episode observation
            terminated, truncated = fallen, truncated & ~fallen
        caller.wait_stream(self._stream_obj)
        for tensor in (obs, reward, terminated, truncated, done):
            tensor.record_stream(caller)
        return obs, reward, terminated, truncated, {"done": done}

    def close(self):
        self.world.destroy()

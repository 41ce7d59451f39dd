"""Env sharding across GPUs: one process per GPU, one world per process, no collective inside the step.

Envs never interact (the reference drops cross-env pairs, src/phi/op_schema.hpp:236-252, and builds trees, slots,
rows and solver tiles per env), so rank g of G owns a contiguous env range and steps it alone.  The only exchange
is the caller's: packed observations + reward per env, gathered after a step (python/nuka/gym/env.py composes the
same 48 floats on the GPU, python/nuka/tasks/go2_obs.py:47-48).
"""
import torch

OBS_FLOATS = 48       # joint positions 12, joint velocities 12, base pose 7, base twist 6, last targets 11
RECORD_FLOATS = OBS_FLOATS + 1      # + reward


def env_range(rank, world_size, total_envs):
    """Contiguous env range [begin, end) of `rank`; the first `total_envs % world_size` ranks hold one more env."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank outside the process group")
    if total_envs < 0:
        raise ValueError("negative env count")
    base, extra = divmod(total_envs, world_size)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sizes(world_size, total_envs):
    return [env_range(r, world_size, total_envs)[1] - env_range(r, world_size, total_envs)[0] for r in range(world_size)]


def pack_observations(out, q, qdot, base_pose, link_velocity, drive_target):
    """Writes one record per env into `out` (E x 49): quadruped observation + height reward.

    q, qdot, drive_target are E x 13 (slot 0 = root), base_pose E x 7, link_velocity E x 78 (root twist first)."""
    out[:, 0:12] = q[:, 1:]
    out[:, 12:24] = qdot[:, 1:]
    out[:, 24:31] = base_pose
    out[:, 31:37] = link_velocity[:, 0:6]
    out[:, 37:48] = drive_target[:, 1:12]
    out[:, 48] = base_pose[:, 2]
    return out


def gather_observations(local, gathered=None, group=None):
    """All-gathers equally sized per-rank records (E_local x 49) into (world_size * E_local) x 49, rank-major."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = torch.empty((world * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if gathered.shape[0] != world * local.shape[0]:
        raise ValueError("gather buffer does not hold world_size shards")
    dist.all_gather_into_tensor(gathered, local.contiguous(), group=group)
    return gathered

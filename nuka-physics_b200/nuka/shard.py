"""Env sharding across GPUs: one process per GPU, one world per process, no collective inside the step.

Envs never interact (the reference drops cross-env pairs, src/phi/op_schema.hpp:236-252, and builds trees, slots,
rows and solver tiles per env), so rank g of G owns a contiguous env range and steps it alone.  The only exchange
is the caller's: the observation record + reward per env, gathered after a step.  The pack kernel writes each rank's
records straight into that rank's slice of the gather buffer, so the all-gather runs in place without a staging copy;
ObservationExchange double-buffers that buffer and runs the all-gather on a side stream, under the next step.
"""
import numpy as np

OBS_FLOATS = 48                     # python/nuka/tasks/go2_obs.py:11-20, 12 actuated joints
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


def observation_record(q, qdot, link_pose, link_velocity, command, last_action, default_position=None, joint_order=None,
                       reward=None, scales=(2.0, 0.25, 1.0, 0.05), command_scale=(2.0, 2.0, 0.25), clip=100.0):
    """numpy statement of the observation record (python/nuka/tasks/go2_obs.py:282-305): the checker of the pack kernel
    and the host-side form for CPU tests.  q, qdot: E x L (slot 0 = root); link_pose E x L x 7; link_velocity E x L x 6
    (angular first); command E x 3 or 3; last_action E x nj.  Returns E x (12 + 3 nj [+ 1])."""
    q, qdot = np.asarray(q, np.float32), np.asarray(qdot, np.float32)
    E, L = q.shape
    nj = L - 1
    pose = np.asarray(link_pose, np.float32).reshape(E, L, 7)
    twist = np.asarray(link_velocity, np.float32).reshape(E, L, 6)[:, 0]
    order = np.arange(nj) if joint_order is None else np.asarray(joint_order, np.int64)
    default = np.zeros(nj, np.float32) if default_position is None else np.asarray(default_position, np.float32)
    w, u = pose[:, 0, 3:4], pose[:, 0, 4:7]
    g = np.broadcast_to(np.array([0.0, 0.0, -1.0], np.float32), (E, 3))
    gravity = (w * w - (u * u).sum(-1, keepdims=True)) * g - 2.0 * w * np.cross(u, g) + 2.0 * u * (u * g).sum(-1, keepdims=True)
    cmd = np.broadcast_to(np.asarray(command, np.float32).reshape(-1, 3), (E, 3)) * np.asarray(command_scale, np.float32)
    parts = [twist[:, 3:6] * np.float32(scales[0]), twist[:, 0:3] * np.float32(scales[1]), gravity.astype(np.float32), cmd,
             (q[:, 1:][:, order] - default) * np.float32(scales[2]), qdot[:, 1:][:, order] * np.float32(scales[3]),
             np.asarray(last_action, np.float32).reshape(E, nj)]
    out = np.clip(np.concatenate(parts, axis=1), -clip, clip).astype(np.float32)
    if reward is not None:
        out = np.concatenate([out, np.asarray(reward, np.float32).reshape(E, 1)], axis=1)
    return out


def gather_buffer(local_envs, world_size, width=RECORD_FLOATS, device=None):
    """Rank-major gather buffer (world_size * local_envs) x width; rank r's records live in rows [r E, (r + 1) E)."""
    import torch
    return torch.empty((world_size * local_envs, width), dtype=torch.float32, device=device)


def local_slice(gathered, rank, world_size):
    """This rank's rows of the gather buffer: the pack kernel's output and the in-place all-gather's input."""
    rows = gathered.shape[0] // world_size
    return gathered[rank * rows:(rank + 1) * rows]


def gather_observations(gathered, rank=None, group=None):
    """In-place all-gather: every rank has filled its own slice (local_slice) of `gathered`; afterwards all slices are valid."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group) if rank is None else rank
    if gathered.shape[0] % world:
        raise ValueError("gather buffer does not hold world_size equal shards")
    dist.all_gather_into_tensor(gathered, local_slice(gathered, rank, world), group=group)
    return gathered


class ObservationExchange:
    """Double-buffered observation exchange of one rank.

    Step k's records are packed (on the world's stream, a few microseconds) into this rank's slice of buffer k % 2;
    the all-gather of that buffer is issued on a side stream and runs under step k + 1, which writes nothing the gather
    reads.  The consumer of the gathered records (a learner, a logger) therefore sees them one step late, the usual
    pipelined arrangement; `wait` orders a consumer stream behind the latest gather.  A buffer is packed again two steps
    later, after its previous gather in side-stream order.  On CPU tensors (gloo, tests) everything is synchronous."""

    def __init__(self, local_envs, world_size, rank, width=RECORD_FLOATS, device=None, group=None):
        import torch
        self.world_size, self.rank, self.group = world_size, rank, group
        self.buffers = [gather_buffer(local_envs, world_size, width, device=device) for _ in range(2)]
        self.cuda = self.buffers[0].is_cuda
        self.side = torch.cuda.Stream(device=device) if self.cuda else None
        self.packed = [torch.cuda.Event() for _ in range(2)] if self.cuda else None
        self.gathered = [torch.cuda.Event() for _ in range(2)] if self.cuda else None
        self.issued = [False, False]
        self.parity = 0            # buffer the next pack goes into
        self.pending = None        # buffer packed but not yet gathered
        self.latest = None         # buffer of the last gather issued

    def pack_target(self, stream=None):
        """This rank's slice of the buffer the coming pack writes into.  `stream` (the packing stream) first waits for that
        buffer's previous gather, issued two steps ago."""
        k = self.parity
        if self.cuda and self.issued[k] and stream is not None:
            stream.wait_event(self.gathered[k])
        return local_slice(self.buffers[k], self.rank, self.world_size)

    def packed_on(self, stream=None):
        """Call after the pack kernel was enqueued on `stream`: the buffer becomes the pending one."""
        k = self.parity
        if self.cuda:
            self.packed[k].record(stream)
        self.pending = k
        self.parity ^= 1

    def gather(self, after=None):
        """Issues the all-gather of the pending buffer on the side stream, behind its pack and, if given, behind the event
        `after` (a caller that wants the gather to start with its next step passes that step's start event)."""
        import torch
        import torch.distributed as dist
        k = self.pending
        if k is None:
            return None
        self.pending = None
        buf = self.buffers[k]
        if not self.cuda:
            dist.all_gather_into_tensor(buf, local_slice(buf, self.rank, self.world_size), group=self.group)
        else:
            self.side.wait_event(self.packed[k])
            if after is not None:
                self.side.wait_event(after)
            with torch.cuda.stream(self.side):
                dist.all_gather_into_tensor(buf, local_slice(buf, self.rank, self.world_size), group=self.group)
                self.gathered[k].record(self.side)
            self.issued[k] = True
        self.latest = k
        return buf

    def wait(self, stream=None):
        """Orders `stream` behind the latest gather and returns its buffer (all slices valid once the stream gets there)."""
        if self.latest is None:
            return None
        if self.cuda and stream is not None:
            stream.wait_event(self.gathered[self.latest])
        return self.buffers[self.latest]

"""Host-side multi-GPU logic on CPU: env ranges and the observation gather with two gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from nuka import shard


def test_env_ranges_tile_the_env_set():
    for total in (0, 1, 7, 4096, 65536, 65537):
        for world in (1, 2, 3, 8):
            spans = [shard.env_range(r, world, total) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[k][1] == spans[k + 1][0] for k in range(world - 1))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == shard.shard_sizes(world, total)
    with pytest.raises(ValueError):
        shard.env_range(2, 2, 10)


def test_observation_record_follows_the_reference_contract():
    """python/nuka/tasks/go2_obs.py:11-20: scales 2.0 / 0.25 / 1.0 / 0.05, command scale (2, 2, 0.25), gravity in the base
    frame, caller joint order through the permutation table, clip to +-100."""
    E, L = 5, 13
    rng = np.random.default_rng(0)
    q, qd = rng.normal(size=(E, L)).astype(np.float32), rng.normal(size=(E, L)).astype(np.float32)
    pose = rng.normal(size=(E, L, 7)).astype(np.float32)
    pose[:, :, 3:] /= np.linalg.norm(pose[:, :, 3:], axis=-1, keepdims=True)
    pose[0, 0, 3:] = (1, 0, 0, 0)                                   # upright base: gravity is (0, 0, -1)
    c, s_ = np.cos(0.25), np.sin(0.25)
    pose[1, 0, 3:] = (c, s_, 0, 0)                                  # rolled by 0.5 rad about x
    twist = rng.normal(size=(E, L, 6)).astype(np.float32)
    twist[2, 0, 3] = 80.0                                           # 80 x 2.0 is clipped to 100
    action = rng.normal(size=(E, 12)).astype(np.float32)
    default = rng.normal(size=12).astype(np.float32)
    order = rng.permutation(12)
    out = shard.observation_record(q, qd, pose, twist, (0.5, -0.2, 1.0), action, default, order)
    assert out.shape == (E, shard.OBS_FLOATS)
    assert np.allclose(out[0, 0:3], twist[0, 0, 3:6] * 2.0) and np.allclose(out[0, 3:6], twist[0, 0, 0:3] * 0.25)
    assert np.allclose(out[0, 6:9], (0, 0, -1), atol=1e-6)
    assert np.allclose(out[1, 6:9], (0, -np.sin(0.5), -np.cos(0.5)), atol=1e-6)
    assert np.allclose(out[:, 9:12], (1.0, -0.4, 0.25))
    assert np.allclose(out[:, 12:24], q[:, 1:][:, order] - default) and np.allclose(out[:, 24:36], qd[:, 1:][:, order] * 0.05)
    assert np.array_equal(out[:, 36:48], action) and out[2, 0] == 100.0
    with_reward = shard.observation_record(q, qd, pose, twist, (0.5, -0.2, 1.0), action, default, order, reward=np.arange(E))
    assert with_reward.shape == (E, shard.RECORD_FLOATS) and np.array_equal(with_reward[:, 48], np.arange(E, dtype=np.float32))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, total_envs, result_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    begin, end = shard.env_range(rank, world, total_envs)
    # each rank's record carries its global env id, so the gathered order can be checked
    gathered = shard.gather_buffer(end - begin, world)
    gathered.fill_(-1.0)
    local = shard.local_slice(gathered, rank, world)         # what the pack kernel writes into
    local[:, 0] = torch.arange(begin, end, dtype=torch.float32)
    local[:, 48] = float(rank)
    shard.gather_observations(gathered)
    dist.barrier()
    torch.save(gathered, os.path.join(result_dir, f"rank{rank}.pt"))
    dist.destroy_process_group()


def test_two_rank_gather_is_rank_major(tmp_path):
    world, total = 2, 64
    mp.spawn(_rank_main, args=(world, _free_port(), total, str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    assert torch.equal(outs[0], outs[1])
    assert torch.equal(outs[0][:, 0], torch.arange(total, dtype=torch.float32))
    assert torch.equal(outs[0][:, 48], torch.repeat_interleave(torch.arange(world, dtype=torch.float32), total // world))


def _exchange_main(rank, world, port, total_envs, result_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    begin, end = shard.env_range(rank, world, total_envs)
    ex = shard.ObservationExchange(end - begin, world, rank)
    seen = []
    for step in range(5):
        local = ex.pack_target()                              # the pack kernel's output on a GPU
        local.fill_(-1.0)
        local[:, 0] = torch.arange(begin, end, dtype=torch.float32)
        local[:, 48] = float(100 * step + rank)
        ex.packed_on()
        assert ex.pending == step % 2
        out = ex.gather()
        assert out is ex.buffers[step % 2] and ex.wait() is out and ex.gather() is None      # nothing pending twice
        seen.append(out.clone())
    dist.barrier()
    torch.save(torch.stack(seen), os.path.join(result_dir, f"exchange{rank}.pt"))
    dist.destroy_process_group()


def test_double_buffered_exchange_alternates_buffers(tmp_path):
    """Two gloo ranks, five steps: buffers alternate, every gather holds the step's records of both ranks in rank-major
    order, and a buffer's earlier contents never leak into a later step."""
    world, total = 2, 48
    mp.spawn(_exchange_main, args=(world, _free_port(), total, str(tmp_path)), nprocs=world, join=True)
    outs = [torch.load(os.path.join(tmp_path, f"exchange{r}.pt")) for r in range(world)]
    assert torch.equal(outs[0], outs[1])
    for step in range(5):
        assert torch.equal(outs[0][step][:, 0], torch.arange(total, dtype=torch.float32))
        want = torch.repeat_interleave(torch.tensor([100.0 * step, 100.0 * step + 1.0]), total // world)
        assert torch.equal(outs[0][step][:, 48], want)

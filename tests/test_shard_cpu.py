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


def test_pack_observations_layout():
    E = 5
    rng = np.random.default_rng(0)
    q, qd, tg = (torch.from_numpy(rng.normal(size=(E, 13)).astype(np.float32)) for _ in range(3))
    base = torch.from_numpy(rng.normal(size=(E, 7)).astype(np.float32))
    lv = torch.from_numpy(rng.normal(size=(E, 78)).astype(np.float32))
    out = shard.pack_observations(torch.zeros(E, shard.RECORD_FLOATS), q, qd, base, lv, tg)
    assert torch.equal(out[:, :12], q[:, 1:]) and torch.equal(out[:, 24:31], base)
    assert torch.equal(out[:, 31:37], lv[:, :6]) and torch.equal(out[:, 48], base[:, 2])


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
    local = torch.zeros((end - begin, shard.RECORD_FLOATS))
    local[:, 0] = torch.arange(begin, end, dtype=torch.float32)
    local[:, 48] = float(rank)
    gathered = shard.gather_observations(local)
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

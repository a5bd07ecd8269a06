"""Host-side multi-GPU logic on CPU: shard planning, and a world-size-2 gloo run in which each rank computes its
head shard (with the CPU oracle standing in for the device kernel) and the shards are all-gathered."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import sharding

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,batch,hq,hkv", [(8, 1, 64, 8), (8, 2, 32, 8), (8, 4, 32, 32), (2, 4, 32, 32),
                                                 (4, 64, 32, 32), (8, 3, 8, 2), (3, 2, 12, 4), (8, 5, 6, 6)])
def test_plan_covers_every_batch_head_pair_once(world, batch, hq, hkv):
    shards = sharding.plan(world, batch, hq, hkv)
    assert len(shards) == world
    seen = np.zeros((batch, hq), np.int32)
    group = hq // hkv
    for s in shards:
        assert s.head_begin % group == 0 and s.head_count % group == 0     # whole KV groups
        seen[s.batch_begin:s.batch_begin + s.batch_count, s.head_begin:s.head_begin + s.head_count] += 1
    assert np.all(seen == 1)


def test_baseline_configs_shard_as_documented():
    c5 = sharding.plan(8, 1, 64, 8)
    assert [(s.head_begin, s.head_count) for s in c5] == [(8 * g, 8) for g in range(8)] and sharding.gatherable(c5)
    c3 = sharding.plan(8, 2, 32, 8)
    assert all(s.head_count == 4 for s in c3) and sharding.gatherable(c3)
    c2 = sharding.plan(8, 4, 32, 32)
    assert all(s.head_count == 4 for s in c2)
    assert not sharding.gatherable(sharding.plan(8, 3, 8, 2))
    with pytest.raises(ValueError):
        sharding.plan(2, 1, 6, 4)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q, k, v, out_path):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from oracle import sdpa_oracle as O
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    B, Hq = q.shape[0], q.shape[1]
    Hkv = k.shape[1]
    group = Hq // Hkv
    s = sharding.plan(world, B, Hq, Hkv)[rank]
    kv0, kvn = s.head_begin // group, s.head_count // group
    mine = O.sdpa(q[:, s.head_begin:s.head_begin + s.head_count], k[:, kv0:kv0 + kvn], v[:, kv0:kv0 + kvn],
                  causal=True, threads=1)
    # in-place all-gather layout of the library for batch 1: rank r owns heads [r*n, (r+1)*n)
    full = torch.zeros((Hq,) + mine.shape[2:], dtype=torch.float32)
    parts = list(full.chunk(world, dim=0))
    dist.all_gather(parts, torch.from_numpy(mine[0]).contiguous())
    if rank == 0:
        np.save(out_path, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_head_shards_gathered_equal_full(tmp_path):
    import torch.multiprocessing as mp
    from oracle import sdpa_oracle as O
    rng = np.random.default_rng(9)
    q = rng.standard_normal((1, 8, 40, 16)).astype(np.float32)
    k = rng.standard_normal((1, 4, 40, 16)).astype(np.float32)
    v = rng.standard_normal((1, 4, 40, 16)).astype(np.float32)
    out_path = str(tmp_path / "gathered.npy")
    mp.spawn(_worker, args=(2, _free_port(), q, k, v, out_path), nprocs=2, join=True)
    full = O.sdpa(q, k, v, causal=True)
    assert np.array_equal(np.load(out_path), full[0])

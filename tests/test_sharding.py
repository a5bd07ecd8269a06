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


def _peer_worker(rank, world, port, scenario, out_dir):
    """The host side of the fused gather (peer.exchange_mappings) with the three library calls replaced by fakes."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    from aidotnet.tensors_b200.peer import exchange_mappings
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    closed = []

    def export(ptr):
        if scenario == "export_fails_on_1" and rank == 1:
            raise RuntimeError("no handle for this allocation")
        return bytes([rank]) * 64, 16 * rank

    def open_mapping(handle):
        if scenario == "open_fails_on_0" and rank == 0:
            raise RuntimeError("cannot map")
        return 0x100000 * (1 + handle[0])

    result = None
    try:
        pointers, bases = exchange_mappings(dist, 0xABC000 + rank, export, open_mapping, closed.append)
        result = ("ok", pointers, bases)
    except RuntimeError as exc:
        result = ("error", str(exc), list(closed))
    np.save(os.path.join(out_dir, f"peer{rank}.npy"), np.array([repr(result)]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("scenario", ["fine", "export_fails_on_1", "open_fails_on_0"])
def test_peer_mapping_exchange_agrees_on_success_and_failure(tmp_path, scenario):
    """Two gloo ranks: on success every rank holds the other's tensor at base + offset; a failure on ONE rank makes
    BOTH raise the same error (nobody is left waiting in a collective) and unmaps what had been mapped."""
    import torch.multiprocessing as mp
    mp.spawn(_peer_worker, args=(2, _free_port(), scenario, str(tmp_path)), nprocs=2, join=True)
    res = [eval(str(np.load(tmp_path / f"peer{r}.npy")[0])) for r in range(2)]
    if scenario == "fine":
        assert res[0] == ("ok", [0xABC000, 0x200000 + 16], [0x200000])
        assert res[1] == ("ok", [0x100000 + 0, 0xABC001], [0x100000])
    elif scenario == "export_fails_on_1":
        assert res[0][0] == res[1][0] == "error"
        assert "rank 1: no handle" in res[0][1] and "rank 1: no handle" in res[1][1]
    else:
        assert res[0][0] == res[1][0] == "error" and "rank 0: cannot map" in res[1][1]
        assert res[1][2] == [0x100000]      # rank 1 had mapped rank 0's tensor and let go of it again


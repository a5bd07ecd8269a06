"""Two-GPU test of the head-sharded path: each rank computes its head shard of a GQA prefill through the C ABI and
the library's in-stream ncclAllGather (desc.nccl_comm + args.gather_output) leaves the full output on every rank.
Skipped on a single-GPU machine.  NVLS is switched off: the test needs nothing from it."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from aidotnet.tensors_b200 import native as N, nccl_util, sharding
    from tests._harness import gen
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    B, Hq, Hkv, S, D = 1, 8, 4, 512, 128
    q, _ = gen((B, Hq, S, D), "bf16", 101)   # every rank holds the full tensors; it computes only its shard
    k, _ = gen((B, Hkv, S, D), "bf16", 102)
    v, _ = gen((B, Hkv, S, D), "bf16", 103)
    q, k, v = q.to(f"cuda:{rank}"), k.to(f"cuda:{rank}"), v.to(f"cuda:{rank}")
    shard = sharding.plan(world, B, Hq, Hkv)[rank]
    comm = nccl_util.create_comm(rank, world)
    out = torch.zeros((B, Hq, S, D), device=f"cuda:{rank}")
    h = N.Handle(device=rank, qkv_dtype=N.BF16, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=True,
                 head_begin=shard.head_begin, head_count=shard.head_count, nccl_comm=comm)
    stream = torch.cuda.current_stream().cuda_stream
    h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=S, seq_kv=S,
             stream=stream, gather_output=True)
    h.poll(stream)
    assert h.last_launch_count == 2          # the attention kernel and the collective
    full = torch.zeros_like(out)
    hf = N.Handle(device=rank, qkv_dtype=N.BF16, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=True)
    hf.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=full.data_ptr(), batch=B, seq_q=S, seq_kv=S,
              stream=stream)
    hf.poll(stream)
    ok = bool(torch.equal(out, full))
    np.save(os.path.join(out_dir, f"ok{rank}.npy"), np.array([ok]))
    h.close()
    hf.close()
    nccl_util.destroy_comm(comm)
    dist.barrier()
    dist.destroy_process_group()


def _peer_worker(rank, world, port, out_dir):
    """Fused gather: every rank's kernel stores its head shard into its own output tensor and, through peer mappings,
    into the other rank's - no collective launch.  Plain peer stores (TMA stores to a peer address), NVLS untouched."""
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from aidotnet.tensors_b200 import native as N, sharding
    from aidotnet.tensors_b200.peer import PeerTensor
    from tests._harness import gen
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    ok = True
    for (B, Hq, Hkv, S, D, odt) in ((1, 8, 4, 512, 128, torch.float32), (2, 8, 2, 700, 64, torch.bfloat16)):
        q, _ = gen((B, Hq, S, D), "bf16", 111)   # every rank holds the full tensors; it computes only its shard
        k, _ = gen((B, Hkv, S, D), "bf16", 112)
        v, _ = gen((B, Hkv, S, D), "bf16", 113)
        q, k, v = q.to(f"cuda:{rank}"), k.to(f"cuda:{rank}"), v.to(f"cuda:{rank}")
        shard = sharding.plan(world, B, Hq, Hkv)[rank]
        out = torch.zeros((B, Hq, S, D), dtype=odt, device=f"cuda:{rank}")
        torch.cuda.synchronize()
        peers = PeerTensor(out, dist)
        adt = N.F32 if odt == torch.float32 else N.BF16
        h = N.Handle(device=rank, qkv_dtype=N.BF16, out_dtype=adt, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=True,
                     head_begin=shard.head_begin, head_count=shard.head_count)
        stream = torch.cuda.current_stream().cuda_stream
        dist.barrier()                           # every rank's output tensor is zeroed and mapped before anyone writes
        h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=S, seq_kv=S,
                 stream=stream, peer_out=peers.others)
        h.poll(stream)
        assert h.last_launch_count == 1          # one kernel, no collective
        torch.cuda.synchronize()
        dist.barrier()                           # ... and every rank's stores have landed before anyone reads
        full = torch.zeros_like(out)
        hf = N.Handle(device=rank, qkv_dtype=N.BF16, out_dtype=adt, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=True)
        hf.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=full.data_ptr(), batch=B, seq_q=S, seq_kv=S,
                  stream=stream)
        hf.poll(stream)
        ok = ok and bool(torch.equal(out, full))
        dist.barrier()
        peers.close()
        h.close()
        hf.close()
    np.save(os.path.join(out_dir, f"peer_ok{rank}.npy"), np.array([ok]))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_head_shards_with_peer_stores(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_peer_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(bool(np.load(tmp_path / f"peer_ok{r}.npy")[0]) for r in range(2))


def test_two_gpu_head_shards_with_nccl_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(bool(np.load(tmp_path / f"ok{r}.npy")[0]) for r in range(2))

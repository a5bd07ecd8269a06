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


def test_two_gpu_head_shards_with_nccl_gather(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert all(bool(np.load(tmp_path / f"ok{r}.npy")[0]) for r in range(2))

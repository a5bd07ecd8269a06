"""What a direct caller of the C ABI may leave in memory, and what a launch may touch.

* Key / value rows that no query can see (rows past kv_len[b], the unused tail of a pool block) may hold NaN or Inf:
  their probability is 0, but 0 * NaN is NaN, so every forward kernel has to keep them out of the P.V product.  The
  reference's callers never see this (CudaBackend.AllocateBuffer zero-fills), a caller with uninitialised padding does.
* A launch allocates nothing, neither through torch nor through the CUDA runtime (the reference asserts the same of
  its hand-written kernels: tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/DirectPtxWmmaTests.cs:561-566).
* Guard words around output, log-sum-exp and workspace stay intact (checked by the harness after every launch).
"""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O
from tests._harness import compare, gen, run_gpu

pytestmark = pytest.mark.gpu


def _poison(t, kv_len, value):
    """Fills rows >= kv_len[b] of a [B, H, S, D] tensor with `value`."""
    t = t.clone()
    for b, n in enumerate(kv_len):
        t[b, :, n:] = value
    return t


@pytest.mark.parametrize("path,dtype,D", [(N.PATH_GENERIC, "f32", 64), (N.PATH_GENERIC, "bf16", 128),
                                          (N.PATH_PREFILL_SM100, "bf16", 128), (N.PATH_PREFILL_SM100, "f16", 64)])
@pytest.mark.parametrize("poison", [float("nan"), float("inf")])
def test_prefill_ignores_non_finite_padding_rows(path, dtype, D, poison):
    B, Hq, Hkv, Sq, Sk = 3, 4, 2, 200, 333
    q, qf = gen((B, Hq, Sq, D), dtype, 601, 1.0 if dtype == "f32" else 0.5)
    k, kf = gen((B, Hkv, Sk, D), dtype, 602, 1.0 if dtype == "f32" else 0.5)
    v, vf = gen((B, Hkv, Sk, D), dtype, 603, 1.0 if dtype == "f32" else 0.5)
    kv = np.array([333, 130, 65], np.int32)        # the last tile of every sequence is partly padding
    kp, vp = _poison(k, kv, poison), _poison(v, kv, poison)
    for causal in (False, True):
        out, lse, info = run_gpu(q, kp, vp, dtype=dtype, causal=causal, kv_len=torch.from_numpy(kv).cuda(), want_lse=True, path=path)
        assert info["path"] == path
        ref = O.sdpa(qf, kf, vf, causal=causal, kv_len=kv)
        compare(out, ref, dtype, f"poisoned padding, path {path}, causal {causal}")
        assert not torch.isnan(lse).any()


@pytest.mark.parametrize("dtype,D,group", [("bf16", 128, 1), ("bf16", 64, 4), ("f32", 64, 2)])
def test_decode_ignores_non_finite_padding_rows(dtype, D, group):
    B, Hkv, Sk = 4, 4, 1100
    q, qf = gen((B, Hkv * group, 1, D), dtype, 611, 1.0 if dtype == "f32" else 0.5)
    k, kf = gen((B, Hkv, Sk, D), dtype, 612, 1.0 if dtype == "f32" else 0.5)
    v, vf = gen((B, Hkv, Sk, D), dtype, 613, 1.0 if dtype == "f32" else 0.5)
    kv = np.array([1100, 1, 513, 777], np.int32)
    kp, vp = _poison(k, kv, float("nan")), _poison(v, kv, float("nan"))
    out, _, info = run_gpu(q, kp, vp, dtype=dtype, kv_len=torch.from_numpy(kv).cuda(), decode_chunk=128)
    assert info["path"] == N.PATH_DECODE
    compare(out, O.sdpa(qf, kf, vf, kv_len=kv), dtype, "decode with poisoned padding")


def _pool_from(k, v, lens, block_size, fill, seed):
    """Scatters contiguous K / V [B, Hkv, S, D] into a pool [blocks, block_size, Hkv, D] whose unused rows hold `fill`."""
    B, Hkv, _, D = k.shape
    per_seq = [(int(n) + block_size - 1) // block_size for n in lens]
    nblocks = sum(per_seq) + 3
    perm = np.random.Generator(np.random.Philox(seed)).permutation(nblocks)
    kpool = torch.full((nblocks, block_size, Hkv, D), fill, dtype=k.dtype, device="cuda")
    vpool = torch.full((nblocks, block_size, Hkv, D), fill, dtype=v.dtype, device="cuda")
    table = np.full((B, max(per_seq)), 0x3fffffff, np.int32)
    at = 0
    for b in range(B):
        for j in range(per_seq[b]):
            blk = int(perm[at])
            at += 1
            table[b, j] = blk
            n = min(block_size, int(lens[b]) - j * block_size)
            kpool[blk, :n] = k[b, :, j * block_size:j * block_size + n].permute(1, 0, 2)
            vpool[blk, :n] = v[b, :, j * block_size:j * block_size + n].permute(1, 0, 2)
    return kpool, vpool, torch.from_numpy(table).cuda(), nblocks


@pytest.mark.parametrize("block_size", [16, 64, 128])
def test_paged_prefill_ignores_the_unused_tail_of_the_last_block(block_size):
    """PagedAttentionPrefill on the tcgen05 kernel: the last block of each sequence is partly unused and holds NaN."""
    B, Hq, Hkv, D = 2, 4, 2, 128
    lens = np.array([300, 170], np.int32)
    Sk = int(lens.max())
    q, qf = gen((B, Hq, 96, D), "bf16", 621)
    k, kf = gen((B, Hkv, Sk, D), "bf16", 622)
    v, vf = gen((B, Hkv, Sk, D), "bf16", 623)
    kpool, vpool, table, nblocks = _pool_from(k, v, lens, block_size, fill=float("nan"), seed=5)
    out = torch.full((B, Hq, 96, D), float("nan"), device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=True,
                 causal_bottom_right=False, causal_offset=int(lens.min()) - 96, path=N.PATH_PREFILL_SM100)
    stream = torch.cuda.current_stream().cuda_stream
    kvt = torch.from_numpy(lens).cuda()
    h.launch(q=q.data_ptr(), k=kpool.data_ptr(), v=vpool.data_ptr(), out=out.data_ptr(), batch=B, seq_q=96, seq_kv=Sk,
             stream=stream, kv_len=kvt.data_ptr(), block_table=table.data_ptr(), block_table_stride=table.shape[1],
             block_size=block_size, num_blocks=nblocks)
    h.poll(stream)
    assert h.last_path == N.PATH_PREFILL_SM100
    h.close()
    ref = O.sdpa(qf, kf, vf, causal=True, causal_offset=int(lens.min()) - 96, kv_len=lens)
    compare(out, ref, "bf16", f"paged prefill, block {block_size}, NaN in unused block tails")


def _mem_get_info():
    return torch.cuda.mem_get_info()   # cudaMemGetInfo


@pytest.mark.parametrize("kind", ["prefill", "decode", "generic"])
def test_a_launch_allocates_nothing(kind):
    """100 launches: device memory (cudaMemGetInfo) and torch's allocator are where they were after the first one."""
    if kind == "prefill":
        q, _ = gen((2, 8, 512, 128), "bf16", 631)
        k, _ = gen((2, 4, 512, 128), "bf16", 632)
        kw = dict(dtype=N.BF16, causal=True)
    elif kind == "decode":
        q, _ = gen((8, 8, 1, 128), "bf16", 633)
        k, _ = gen((8, 8, 2048, 128), "bf16", 634)
        kw = dict(dtype=N.BF16, causal=False)
    else:
        q, _ = gen((1, 4, 200, 64), "f32", 635, 1.0)
        k, _ = gen((1, 4, 200, 64), "f32", 636, 1.0)
        kw = dict(dtype=N.F32, causal=False)
    v = k.clone()
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    out = torch.empty((B, Hq, Sq, D), device="cuda")
    h = N.Handle(device=0, qkv_dtype=kw["dtype"], head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=kw["causal"],
                 max_batch=B, max_seq_q=Sq, max_seq_kv=Sk)
    stream = torch.cuda.current_stream().cuda_stream
    launch = lambda: h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=Sq,
                              seq_kv=Sk, stream=stream)
    launch()
    h.poll(stream)
    torch.cuda.synchronize()
    free0, _ = _mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    for _ in range(100):
        launch()
    h.poll(stream)
    torch.cuda.synchronize()
    free1, _ = _mem_get_info()
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    assert free1 == free0, f"device memory changed across 100 launches: {free0} -> {free1}"
    h.close()


def test_launch_check_switch_reports_a_failure_at_the_call_that_caused_it():
    """AIDOTNET_KERNEL_LAUNCH_CHECK=1 (the reference's switch, CudaBackend.cs:5381-5421): the launch itself returns the
    expired bounded wait that normally only aidn_sdpa_poll reports.  The failure is provoked with the test hook that
    withholds the producer's loads (20 ms budget, no fault); the variable is read once per process, hence the child."""
    import os
    import subprocess
    import sys
    code = r'''
import torch
from aidotnet.tensors_b200 import native as N
from tests._harness import gen
q, _ = gen((1, 4, 256, 128), "bf16", 1); k, _ = gen((1, 2, 256, 128), "bf16", 2); v = k.clone()
out = torch.zeros((1, 4, 256, 128), device="cuda")
h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=4, num_kv_heads=2, causal=True)
st = torch.cuda.current_stream().cuda_stream
go = lambda: h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=1, seq_q=256, seq_kv=256, stream=st)
go()                                  # a healthy launch passes the check
h.debug_set(None, 3)
try:
    go()
    raise SystemExit("the launch did not report the expired wait")
except N.AidnError as e:
    assert e.status == N.ETIMEOUT and "LAUNCH-FAULT" in e.message, (e.status, e.message)
h.debug_set(None, 0)
try:
    h.poll(st)                        # clears the status word
except N.AidnError:
    pass
go(); h.poll(st)
print("launch check ok")
'''
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, AIDOTNET_KERNEL_LAUNCH_CHECK="1", PYTHONPATH=root)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, env=env, cwd=root)
    assert r.returncode == 0 and "launch check ok" in r.stdout, f"stdout:\n{r.stdout}\nstderr:\n{r.stderr[-2000:]}"

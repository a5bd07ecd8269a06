"""The decode entry point that allocates nothing (aidn_sdpa_decode_noalloc).

It exists for hosts that may not allocate device memory at the point where they decode (a serving loop or a
graph-replaying runtime that fixed its memory up front, a managed runtime whose GPU buffers all come from one
pre-sized pool): the split-KV partials live in a 16 MiB array inside the library instead of a workspace.  The
test calls it through the C ABI twice in a row, with different shapes so that the second call finds the first
call's partials still in the shared array, and checks both results against the regular entry point
(aidn_sdpa_launch with a caller workspace) within the parity tolerance of the 16-bit contract.

Collected last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from tests._harness import TOL_16_MAX, TOL_16_MEAN, gen, run_gpu

pytestmark = pytest.mark.gpu


def _noalloc(q, k, v, kv_len, *, causal=False, decode_chunk=0, want_lse=True):
    B, Hq, _, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    d = N.SdpaDesc()
    d.device, d.qkv_dtype, d.out_dtype, d.head_dim = 0, N.BF16, N.F32, D
    d.num_q_heads, d.num_kv_heads = Hq, Hkv
    d.causal, d.causal_bottom_right, d.emit_lse, d.decode_chunk = int(causal), 1, int(want_lse), decode_chunk
    out = torch.full((B, Hq, 1, D), float("nan"), device="cuda")
    lse = torch.full((B, Hq, 1), float("nan"), device="cuda")
    a = N.SdpaArgs()
    a.q, a.k, a.v, a.out, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.kv_len = kv_len.data_ptr() if kv_len is not None else None
    a.batch, a.seq_q, a.seq_kv = B, 1, Sk
    stream = torch.cuda.current_stream().cuda_stream
    N.decode_noalloc(d, a, stream)
    torch.cuda.synchronize()
    return out, lse


def _close(a, b):
    diff = (a.float() - b.float()).abs()
    assert torch.isfinite(a).all()
    assert float(diff.max()) <= TOL_16_MAX and float(diff.mean()) <= TOL_16_MEAN, (float(diff.max()), float(diff.mean()))


def test_decode_noalloc_matches_regular_entry_point_twice():
    torch.cuda.set_device(0)
    # call 1: 16 splits per (batch, head), ragged lengths, GQA 4
    q1, _ = gen((4, 16, 1, 128), "bf16", 901)
    k1, _ = gen((4, 4, 2048, 128), "bf16", 902)
    v1, _ = gen((4, 4, 2048, 128), "bf16", 903)
    kv1 = torch.tensor([2048, 1, 777, 1300], dtype=torch.int32, device="cuda")
    ref1, rlse1, info = run_gpu(q1, k1, v1, dtype="bf16", kv_len=kv1, want_lse=True, decode_chunk=128)
    assert info["path"] == N.PATH_DECODE and info["launches"] == 2
    out1, lse1 = _noalloc(q1, k1, v1, kv1, decode_chunk=128)
    _close(out1, ref1)
    assert torch.allclose(lse1, rlse1, atol=2e-2)

    # call 2, straight after: smaller shape, other split size, MHA; the array still holds call 1's partials
    q2, _ = gen((2, 8, 1, 64), "bf16", 911)
    k2, _ = gen((2, 8, 900, 64), "bf16", 912)
    v2, _ = gen((2, 8, 900, 64), "bf16", 913)
    kv2 = torch.tensor([900, 65], dtype=torch.int32, device="cuda")
    out2, lse2 = _noalloc(q2, k2, v2, kv2, decode_chunk=64)
    ref2, rlse2, _ = run_gpu(q2, k2, v2, dtype="bf16", kv_len=kv2, want_lse=True, decode_chunk=64)
    _close(out2, ref2)
    assert torch.allclose(lse2, rlse2, atol=2e-2)

    # and call 1 again gives what it gave before
    out3, _ = _noalloc(q1, k1, v1, kv1, decode_chunk=128)
    assert torch.equal(out3, out1)


def test_decode_noalloc_rejects_oversized_requests_clearly():
    torch.cuda.set_device(0)
    # 64 * 64 * ceil(4096/64) * 130 * 4 bytes = 136 MB of partials: far beyond the 16 MiB array
    q = torch.zeros((64, 64, 1, 128), dtype=torch.bfloat16, device="cuda")
    k = torch.zeros((64, 1, 4096, 128), dtype=torch.bfloat16, device="cuda")
    d = N.SdpaDesc()
    d.device, d.qkv_dtype, d.out_dtype, d.head_dim, d.num_q_heads, d.num_kv_heads, d.decode_chunk = 0, N.BF16, N.F32, 128, 64, 1, 64
    out = torch.zeros((64, 64, 1, 128), device="cuda")
    a = N.SdpaArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), k.data_ptr(), out.data_ptr()
    a.batch, a.seq_q, a.seq_kv = 64, 1, 4096
    with pytest.raises(N.AidnError) as e:
        N.decode_noalloc(d, a, torch.cuda.current_stream().cuda_stream)
    assert e.value.status == N.EWORKSPACE and "static array" in e.value.message
    a.seq_q = 2
    with pytest.raises(N.AidnError) as e:
        N.decode_noalloc(d, a, torch.cuda.current_stream().cuda_stream)
    assert e.value.status == N.EUNSUPPORTED

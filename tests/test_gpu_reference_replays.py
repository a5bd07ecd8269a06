"""Replays of the reference's own attention tests that were not yet replayed elsewhere, through the C ABI on the GPU.

Inputs the reference draws from System.Random are re-seeded here (its assertions compare implementation against
reference, not against fixed numbers); shapes, layouts, scales and tolerances are the reference's.  Paths are relative
to tests/AiDotNet.Tensors.Tests/Engines/ of the reference.

* IntoKernelParityTests.cs:40-74      ScaledDotProductAttentionInto: contiguous operands, and [B,S,H,D] storage viewed
                                      as [B,H,S,D] (permuted, unit stride on D) for Q, K, V - and here also for the
                                      destination, on every kernel family
* SdpaDoubleFastPathTests.cs:99-131   the double fast path against a scalar reference: shape list, uniform(-1,1) inputs
* Autodiff/FusedAttentionFp32PrecisionTests.cs:40-55   fp32 arithmetic against an fp64 reference: < 2e-3 absolute
* DirectGpu/DirectPtxWmmaTests.cs:498-583 with the release matrix of
  src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Ptx/DirectPtxOnlineAttentionReleaseMatrix.cs:39-47 and the oracle
  ValidateOnlineFamily (:3053-3134): fp16 inputs in +-0.25, D = 64, scale 0.125, rectangular GQA / MQA / MHA, causal
  with a query offset (last visible key = min(row + offset, Skv - 1)), log-sum-exp; output <= 0.012, LSE <= 0.02
"""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O
from tests._harness import AIDN_DT, TORCH_DT, check_guards, guarded

pytestmark = pytest.mark.gpu


def _uniform(shape, seed, lo=-1.0, hi=1.0):
    g = np.random.Generator(np.random.Philox(seed))
    return (g.random(shape, dtype=np.float32) * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def _launch(q, k, v, out, *, dtype, B, Hq, Hkv, Sq, Sk, D, scale, q_stride=None, k_stride=None, v_stride=None, o_stride=None,
            causal=False, bottom_right=True, causal_offset=0, lse=None, path=N.PATH_AUTO, out_dtype="f32"):
    h = N.Handle(device=0, qkv_dtype=AIDN_DT[dtype], out_dtype=AIDN_DT[out_dtype], head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv,
                 causal=causal, causal_bottom_right=bottom_right, causal_offset=causal_offset, emit_lse=lse is not None, path=path)
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = h.workspace_bytes(B, Sq, Sk)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=Sq, seq_kv=Sk, stream=stream,
             lse=lse.data_ptr() if lse is not None else None, q_stride=q_stride, k_stride=k_stride, v_stride=v_stride,
             o_stride=o_stride, scale=scale, workspace=ws.data_ptr() if nbytes else None, workspace_bytes=nbytes)
    h.poll(stream)
    p = h.last_path
    h.close()
    return p


# ------------------------------------------------------------------------------------------------ *Into
@pytest.mark.parametrize("dtype,shape,path,tol", [
    ("f32", (2, 4, 6, 8), N.PATH_GENERIC, 1e-5),       # IntoKernelParityTests.cs:40-52 (contiguous), its own shape
    ("f32", (2, 3, 5, 8), N.PATH_GENERIC, 1e-5),       # :54-74 (permuted), its own shape
    ("bf16", (2, 4, 300, 128), N.PATH_PREFILL_SM100, 2e-2),   # the same two layouts through the tcgen05 kernel
    ("f16", (1, 6, 129, 64), N.PATH_PREFILL_SM100, 2e-2),
    ("bf16", (3, 8, 1, 128), N.PATH_DECODE, 2e-2),            # ... and the decode kernel (one query token)
])
@pytest.mark.parametrize("permuted", [False, True])
def test_into_matches_allocating_for_contiguous_and_permuted_views(dtype, shape, path, tol, permuted):
    """The destination and every operand either dense [B,H,S,D] or a [B,S,H,D] allocation viewed as [B,H,S,D]
    (TensorPermute([0,2,1,3]) in the reference); both must give what the dense call gives."""
    B, H, S, D = shape
    Sk = S if path != N.PATH_DECODE else 700
    scale = 0.1875 if not permuted else 0.125
    tdt = TORCH_DT[dtype]
    amp = 1.0 if dtype == "f32" else 0.5
    qd = torch.from_numpy(_uniform((B, H, S, D), 11) * amp).to(tdt).cuda()
    kd = torch.from_numpy(_uniform((B, H, Sk, D), 12) * amp).to(tdt).cuda()
    vd = torch.from_numpy(_uniform((B, H, Sk, D), 13) * amp).to(tdt).cuda()
    ref = O.sdpa(qd.float().cpu().numpy(), kd.float().cpu().numpy(), vd.float().cpu().numpy(), scale=scale)
    if not permuted:
        flat, out = guarded((B, H, S, D), torch.float32, "cuda")
        used = _launch(qd, kd, vd, out, dtype=dtype, B=B, Hq=H, Hkv=H, Sq=S, Sk=Sk, D=D, scale=scale, path=path)
        got = out
    else:
        # storage [B, S, H, D]; strides of the [B, H, S, D] view in elements: (S*H*D, D, H*D)
        qp, kp, vp = (t.permute(0, 2, 1, 3).contiguous() for t in (qd, kd, vd))
        flat, outp = guarded((B, S, H, D), torch.float32, "cuda")
        sq = (S * H * D, D, H * D)
        sk = (Sk * H * D, D, H * D)
        used = _launch(qp, kp, vp, outp, dtype=dtype, B=B, Hq=H, Hkv=H, Sq=S, Sk=Sk, D=D, scale=scale, path=path,
                       q_stride=sq, k_stride=sk, v_stride=sk, o_stride=sq)
        got = outp.permute(0, 2, 1, 3)
    check_guards(flat, "Into destination")
    assert used == path
    err = np.abs(got.float().cpu().numpy() - ref)
    bound = tol * max(np.abs(ref).max(), 1e-30) if dtype == "f32" else tol
    assert err.max() <= bound, f"{dtype} {shape} permuted={permuted}: {err.max():.3e}"


# ------------------------------------------------------------------------------------------------ double fast path
@pytest.mark.parametrize("batch,heads,seq_q,seq_k,d", [(1, 1, 4, 4, 8), (1, 2, 8, 8, 16), (2, 4, 16, 16, 32), (1, 16, 64, 64, 128)])
def test_fp32_path_on_the_double_fast_path_shapes(batch, heads, seq_q, seq_k, d):
    """SdpaDoubleFastPathTests.cs:99-131: uniform(-1,1) inputs, scale 1/sqrt(d), against a scalar float64 reference.
    The library has no fp64 kernel (the GPU backend's buffers are fp32); its fp32 path must agree to fp32 accuracy."""
    q = _uniform((batch, heads, seq_q, d), 42)
    k = _uniform((batch, heads, seq_k, d), 43)
    v = _uniform((batch, heads, seq_k, d), 44)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(d)
    p = np.exp(s - s.max(-1, keepdims=True))
    ref = np.einsum("bhqk,bhkd->bhqd", p / p.sum(-1, keepdims=True), v.astype(np.float64))
    out = torch.empty((batch, heads, seq_q, d), device="cuda")
    _launch(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), out, dtype="f32", B=batch,
            Hq=heads, Hkv=heads, Sq=seq_q, Sk=seq_k, D=d, scale=0.0)
    assert np.abs(out.cpu().numpy() - ref).max() <= 1e-5 * max(np.abs(ref).max(), 1.0)


# ------------------------------------------------------------------------------------------------ fp32 precision
@pytest.mark.parametrize("b,h,sq,sk,d", [(1, 1, 8, 8, 16), (2, 2, 16, 16, 8), (1, 4, 32, 32, 24), (2, 4, 70, 70, 16),
                                        (1, 8, 128, 128, 16), (1, 2, 100, 100, 24), (2, 1, 33, 65, 8)])
def test_fp32_arithmetic_stays_within_the_fp32_floor_of_an_fp64_reference(b, h, sq, sk, d):
    """FusedAttentionFp32PrecisionTests.cs:40-55: max |fp32 - fp64| < 2e-3 and not bit-identical.  Head sizes are the
    reference's rounded up to the multiple of 8 this library's fp32 kernel takes (20 -> 24, 12 -> 16)."""
    q = _uniform((b, h, sq, d), 1000 + sq)
    k = _uniform((b, h, sk, d), 2000 + sk)
    v = _uniform((b, h, sk, d), 3000 + d)
    s = np.einsum("bhqd,bhkd->bhqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(d)
    p = np.exp(s - s.max(-1, keepdims=True))
    ref = np.einsum("bhqk,bhkd->bhqd", p / p.sum(-1, keepdims=True), v.astype(np.float64))
    out = torch.empty((b, h, sq, d), device="cuda")
    _launch(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), out, dtype="f32", B=b, Hq=h,
            Hkv=h, Sq=sq, Sk=sk, D=d, scale=0.0)
    diff = np.abs(out.cpu().numpy().astype(np.float64) - ref).max()
    assert diff < 2e-3
    assert diff > 0.0


# ------------------------------------------------------------------------------------------------ online attention family
def _validate_online_family(q, k, v, B, Hq, Hkv, Sq, Sk, causal, offset, scale):
    """ValidateOnlineFamily (DirectPtxWmmaTests.cs:3053-3134), vectorised: float32 scores over the keys 0..lastKey,
    lastKey = min(row + offset, Sk - 1) when causal; a row with lastKey < 0 gives zeros and LSE -inf."""
    g = Hq // Hkv
    out = np.zeros((B, Hq, Sq, q.shape[-1]), np.float32)
    lse = np.full((B, Hq, Sq), -np.inf, np.float32)
    for b in range(B):
        for h in range(Hq):
            s = (q[b, h].astype(np.float32) @ k[b, h // g].astype(np.float32).T) * np.float32(scale)
            if causal:
                last = np.minimum(np.arange(Sq) + offset, Sk - 1)
                s = np.where(np.arange(Sk)[None, :] <= last[:, None], s, -np.inf)
            m = s.max(-1)
            ok = np.isfinite(m)
            p = np.exp(s[ok] - m[ok, None])
            den = p.sum(-1)
            out[b, h, ok] = (p / den[:, None]) @ v[b, h // g].astype(np.float32)
            lse[b, h, ok] = m[ok] + np.log(den)
    return out, lse


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,causal,offset", [
    (2, 4, 2, 32, 64, False, 0), (2, 8, 1, 32, 64, True, 0), (2, 8, 2, 32, 64, True, 32), (1, 4, 4, 128, 32, True, 0),
    (1, 4, 2, 128, 64, True, -64)])
@pytest.mark.parametrize("path", [N.PATH_PREFILL_SM100, N.PATH_GENERIC])
def test_online_attention_family_release_matrix(B, Hq, Hkv, Sq, Sk, causal, offset, path):
    D, scale = 64, 0.125
    q = _uniform((B, Hq, Sq, D), 20260800 + B * 1000 + Hq * 100 + Hkv * 10 + Sq + Sk + int(causal), -0.25, 0.25).astype(np.float16)
    k = _uniform((B, Hkv, Sk, D), 20260801 + Sq, -0.25, 0.25).astype(np.float16)
    v = _uniform((B, Hkv, Sk, D), 20260802 + Sk, -0.25, 0.25).astype(np.float16)
    want, want_lse = _validate_online_family(q, k, v, B, Hq, Hkv, Sq, Sk, causal, offset, scale)
    flat_o, out = guarded((B, Hq, Sq, D), torch.float32, "cuda")
    flat_l, lse = guarded((B, Hq, Sq), torch.float32, "cuda")
    used = _launch(torch.from_numpy(q).cuda(), torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(), out, dtype="f16", B=B,
                   Hq=Hq, Hkv=Hkv, Sq=Sq, Sk=Sk, D=D, scale=scale, causal=causal, bottom_right=False, causal_offset=offset,
                   lse=lse, path=path)
    assert used == path
    check_guards(flat_o, "output")
    check_guards(flat_l, "log-sum-exp")
    got, got_lse = out.cpu().numpy(), lse.cpu().numpy()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 0.012
    dead = np.isneginf(want_lse)
    assert np.array_equal(np.isneginf(got_lse), dead)
    assert np.abs(got_lse[~dead] - want_lse[~dead]).max(initial=0.0) <= 0.02
    assert np.abs(got[dead]).max(initial=0.0) == 0.0     # rows that see no key are exactly zero

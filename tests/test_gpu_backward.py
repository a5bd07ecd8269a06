"""GPU parity of aidn_sdpa_backward (FlashAttentionBackward) against the float64 oracle, which tests/test_oracle_pins.py
pins on finite differences of the forward oracle.  The forward output and log-sum-exp fed to the backward come from
this library's own forward launch, as they do in training."""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O

from tests._harness import AIDN_DT, TORCH_DT, gen

pytestmark = pytest.mark.gpu


def _fwd_bwd(q, k, v, dout, *, dtype, causal=False, causal_offset=0, bottom_right=False, mask=None, mask_kind=N.MASK_NONE,
             kv_len=None, scale=0.0, head_begin=0, head_count=0, path=N.PATH_AUTO, info=None):
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    hc = head_count or Hq
    out = torch.full((B, Hq, Sq, D), float("nan"), device="cuda")
    lse = torch.full((B, Hq, Sq), float("nan"), device="cuda")
    h = N.Handle(device=0, qkv_dtype=AIDN_DT[dtype], head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=causal,
                 causal_bottom_right=bottom_right, causal_offset=causal_offset, mask_kind=mask_kind, emit_lse=True,
                 head_begin=head_begin, head_count=head_count, path=path)
    stream = torch.cuda.current_stream().cuda_stream
    ms = (0, 0, 0, 0)
    if mask is not None:
        full = (B, Hq, Sq, Sk)
        st = mask.stride()
        ms = tuple(0 if (mask.shape[a] == 1 and full[a] != 1) else st[a] for a in range(4))
    kl = torch.from_numpy(np.asarray(kv_len, np.int32)).cuda() if kv_len is not None else None
    common = dict(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), lse=lse.data_ptr(), batch=B,
                  seq_q=Sq, seq_kv=Sk, stream=stream, mask=mask.data_ptr() if mask is not None else None, mask_stride=ms,
                  kv_len=kl.data_ptr() if kl is not None else None, scale=scale)
    nb = h.workspace_bytes(B, Sq, Sk)
    ws = torch.empty(max(nb, 16), dtype=torch.uint8, device="cuda")
    h.launch(workspace=ws.data_ptr() if nb else None, workspace_bytes=nb, **common)
    group = Hq // Hkv
    dq = torch.full((B, hc, Sq, D), float("nan"), device="cuda")
    dk = torch.full((B, hc // group, Sk, D), float("nan"), device="cuda")
    dv = torch.full((B, hc // group, Sk, D), float("nan"), device="cuda")
    nbw = h.backward_workspace_bytes(B, Sq)
    wsb = torch.empty(nbw, dtype=torch.uint8, device="cuda")
    h.backward(dout=dout.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(), dv=dv.data_ptr(), workspace=wsb.data_ptr(),
               workspace_bytes=nbw, **common)
    h.poll(stream)
    if info is not None:
        info["path"] = h.last_path
    h.close()
    return dq, dk, dv


def _check(got, want, dtype, what):
    g = got.cpu().numpy()
    assert np.isfinite(g).all(), what
    scale_ = max(np.abs(want).max(), 1e-6)
    rel = np.abs(g - want).max() / scale_
    # fp32: the kernels' fp32 sums against float64; 16-bit inputs: the forward O / lse came from the 16-bit kernels
    tol = 2e-5 if dtype == "f32" else 2e-2
    assert rel <= tol, f"{what}: relative error {rel:.3e}"


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 4, 4, 37, 37, 64), (1, 8, 2, 50, 83, 128), (2, 3, 1, 17, 40, 32), (1, 2, 2, 33, 65, 256),
                                   (1, 4, 4, 130, 130, 96)])
@pytest.mark.parametrize("causal", [False, True])
def test_backward_shapes(dtype, shape, causal):
    """Odd lengths, Sq != Sk, MHA / GQA / MQA, every head_dim bucket, top-left causal (FlashAttentionBackward) and a
    padded batch entry."""
    B, Hq, Hkv, Sq, Sk, D = shape
    q, qf = gen((B, Hq, Sq, D), dtype, 901)
    k, kf = gen((B, Hkv, Sk, D), dtype, 902)
    v, vf = gen((B, Hkv, Sk, D), dtype, 903)
    dout, dof = gen((B, Hq, Sq, D), "f32", 904, scale=1.0)
    kv_len = np.array([Sk, max(1, Sk // 2)][:B], np.int32)
    dq, dk, dv = _fwd_bwd(q, k, v, dout, dtype=dtype, causal=causal, causal_offset=0, kv_len=kv_len)
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, causal=causal, causal_offset=0, kv_len=kv_len)
    _check(dq, rq, dtype, f"dQ {shape}")
    _check(dk, rk, dtype, f"dK {shape}")
    _check(dv, rv, dtype, f"dV {shape}")


def test_backward_with_bias_and_keep_mask():
    """FlashAttentionBackward with an additive bias (3-D, batch-broadcast, as FlashAttentionBiasTests uses) and, on the
    same entry point, a boolean keep-mask with a fully masked row (its gradients are zero)."""
    B, H, S, D = 2, 3, 29, 64
    q, qf = gen((B, H, S, D), "f32", 911)
    k, kf = gen((B, H, S, D), "f32", 912)
    v, vf = gen((B, H, S, D), "f32", 913)
    dout, dof = gen((B, H, S, D), "f32", 914, scale=1.0)
    bias, bf = gen((1, H, S, S), "f32", 915, scale=0.5)
    dq, dk, dv = _fwd_bwd(q, k, v, dout, dtype="f32", causal=True, mask=bias, mask_kind=N.MASK_ADD_F32, scale=0.25)
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, scale=0.25, causal=True, causal_offset=0, bias=bf)
    for g, r, n in ((dq, rq, "dQ"), (dk, rk, "dK"), (dv, rv, "dV")):
        _check(g, r, "f32", n + " bias")
    keep = (np.random.default_rng(3).random((B, 1, S, S)) > 0.3).astype(np.uint8)
    keep[0, 0, 5, :] = 0
    kd = torch.from_numpy(keep).cuda()
    dq, dk, dv = _fwd_bwd(q, k, v, dout, dtype="f32", mask=kd, mask_kind=N.MASK_KEEP_U8)
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, keep=keep, causal_offset=0)
    for g, r, n in ((dq, rq, "dQ"), (dk, rk, "dK"), (dv, rv, "dV")):
        _check(g, r, "f32", n + " keep")
    assert torch.count_nonzero(dq[0, :, 5]).item() == 0


def test_backward_is_deterministic_and_shards_by_head():
    B, Hq, Hkv, S, D = 1, 8, 4, 70, 64
    q, _ = gen((B, Hq, S, D), "bf16", 921)
    k, _ = gen((B, Hkv, S, D), "bf16", 922)
    v, _ = gen((B, Hkv, S, D), "bf16", 923)
    dout, _ = gen((B, Hq, S, D), "f32", 924, scale=1.0)
    a = _fwd_bwd(q, k, v, dout, dtype="bf16", causal=True)
    b = _fwd_bwd(q, k, v, dout, dtype="bf16", causal=True)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    # heads 4..7 (kv heads 2..3) computed alone equal the same slices of the full call
    s = _fwd_bwd(q, k, v, dout, dtype="bf16", causal=True, head_begin=4, head_count=4)
    assert torch.equal(s[0], a[0][:, 4:8]) and torch.equal(s[1], a[1][:, 2:4]) and torch.equal(s[2], a[2][:, 2:4])


def test_backward_argument_errors():
    q, _ = gen((1, 2, 8, 64), "f32", 931)
    out = torch.zeros_like(q)
    lse = torch.zeros((1, 2, 8), device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.F32, head_dim=64, num_q_heads=2, emit_lse=True)
    kw = dict(q=q.data_ptr(), k=q.data_ptr(), v=q.data_ptr(), out=out.data_ptr(), lse=lse.data_ptr(), dout=q.data_ptr(),
              dq=out.data_ptr(), dk=out.data_ptr(), dv=out.data_ptr(), batch=1, seq_q=8, seq_kv=8, stream=0)
    with pytest.raises(N.AidnError) as e:
        h.backward(workspace=q.data_ptr(), workspace_bytes=8, **kw)
    assert e.value.status == N.EWORKSPACE
    with pytest.raises(N.AidnError) as e:
        h.backward(workspace=q.data_ptr(), workspace_bytes=4096, **{**kw, "dq": None})
    assert e.value.status == N.EINVAL
    h.close()
    h = N.Handle(device=0, qkv_dtype=N.F32, head_dim=64, num_q_heads=2, softcap=30.0)
    with pytest.raises(N.AidnError) as e:
        h.backward(workspace=q.data_ptr(), workspace_bytes=4096, **kw)
    assert e.value.status == N.EUNSUPPORTED
    h.close()


def test_backend_flash_attention_backward():
    """The mirror of CudaBackend.FlashAttentionBackward (CudaBackend.cs:8580-8604): fp32 buffers, statistics from
    FlashAttentionV2, gradients written into caller buffers."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    B, H, S, D = 2, 3, 21, 16
    rng = np.random.default_rng(41)
    qf, kf, vf, dof = (rng.uniform(-1, 1, (B, H, S, D)).astype(np.float32) for _ in range(4))
    be = CudaBackend(0)
    buf = lambda a: GpuBuffer(torch.from_numpy(a).reshape(-1).cuda())
    zeros = lambda n: GpuBuffer(torch.zeros(n, device="cuda"))
    qb, kb, vb, gb = buf(qf), buf(kf), buf(vf), buf(dof)
    out, stats = zeros(B * H * S * D), zeros(B * H * S)
    be.FlashAttentionV2(qb, kb, vb, out, stats, B, H, S, S, D, 0.25, True)
    gq, gk, gv = zeros(B * H * S * D), zeros(B * H * S * D), zeros(B * H * S * D)
    be.FlashAttentionBackward(gb, qb, kb, vb, out, stats, gq, gk, gv, B, H, S, S, D, 0.25, True)
    be.Synchronize()
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, scale=0.25, causal=True, causal_offset=0)
    for g, r in ((gq, rq), (gk, rk), (gv, rv)):
        assert np.abs(g.tensor.cpu().numpy().reshape(r.shape) - r).max() <= 2e-5 * max(1.0, np.abs(r).max())
    with pytest.raises(ValueError):
        be.FlashAttentionBackward(gb, qb, kb, vb, out, stats, gq, gk, zeros(4), B, H, S, S, D, 0.25, True)
    be.Dispose()


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(1, 4, 4, 256, 256, 128), (2, 4, 2, 200, 333, 64), (1, 8, 1, 130, 517, 128), (2, 2, 2, 384, 128, 64),
                                   (1, 2, 2, 1, 300, 128)])
@pytest.mark.parametrize("causal", [False, True])
def test_backward_tensor_core_families(dtype, shape, causal):
    """16-bit inputs with head_dim 64 / 128 run the tcgen05 kernels (several 128-row tiles per sequence, ragged ends,
    grouped-query heads, bottom-right causal offsets, a padded batch entry); with desc.path = generic the same call stays
    on the mma.sync kernels.  Both meet the oracle and each is bit-reproducible."""
    B, Hq, Hkv, Sq, Sk, D = shape
    q, qf = gen((B, Hq, Sq, D), dtype, 951)
    k, kf = gen((B, Hkv, Sk, D), dtype, 952)
    v, vf = gen((B, Hkv, Sk, D), dtype, 953)
    dout, dof = gen((B, Hq, Sq, D), "f32", 954, scale=1.0)
    kv_len = np.array([Sk, max(1, Sk - 77)][:B], np.int32)
    off = Sk - Sq
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, causal=causal, causal_offset=off, kv_len=kv_len)
    for path, want_path in ((N.PATH_AUTO, N.PATH_PREFILL_SM100), (N.PATH_GENERIC, N.PATH_GENERIC)):
        info = {}
        dq, dk, dv = _fwd_bwd(q, k, v, dout, dtype=dtype, causal=causal, bottom_right=True, kv_len=kv_len, path=path, info=info)
        assert info["path"] == want_path
        _check(dq, rq, dtype, f"dQ {shape} path {path}")
        _check(dk, rk, dtype, f"dK {shape} path {path}")
        _check(dv, rv, dtype, f"dV {shape} path {path}")
        dq2, dk2, dv2 = _fwd_bwd(q, k, v, dout, dtype=dtype, causal=causal, bottom_right=True, kv_len=kv_len, path=path)
        assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


@pytest.mark.parametrize("path", [N.PATH_AUTO, N.PATH_GENERIC])
def test_backward_single_visible_key_has_no_score_gradient(path):
    """With one visible key the probabilities are exactly 1, so dS = dP - delta must cancel: dQ = dK = 0 and dV = the
    column sum of dO.  The tensor-core kernels multiply with dO rounded to the input dtype; delta is summed from the
    same rounded values, otherwise the difference of the two roundings accumulates over the queries into dK."""
    B, H, Sq, Sk, D = 2, 2, 265, 239, 64
    q, qf = gen((B, H, Sq, D), "bf16", 971)
    k, kf = gen((B, H, Sk, D), "bf16", 972)
    v, vf = gen((B, H, Sk, D), "bf16", 973)
    dout, dof = gen((B, H, Sq, D), "f32", 974, scale=1.0)
    kv_len = np.array([1, 1], np.int32)
    dq, dk, dv = _fwd_bwd(q, k, v, dout, dtype="bf16", kv_len=kv_len, path=path)
    assert float(dq.abs().max()) <= 1e-4 and float(dk.abs().max()) <= 1e-4
    want = torch.from_numpy(dof).to(torch.bfloat16).to(torch.float32).sum(dim=2).numpy()   # [B, H, D]
    got = dv.cpu().numpy()
    assert np.abs(got[:, :, 0, :] - want).max() <= 2e-2 * np.abs(want).max()
    assert np.abs(got[:, :, 1:, :]).max() == 0.0


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("kind", ["bias", "bias_broadcast", "keep_u8", "keep_f32"])
@pytest.mark.parametrize("path", [N.PATH_AUTO, N.PATH_GENERIC])
def test_backward_tensor_core_families_with_bias_and_masks(dtype, kind, path):
    """16-bit inputs with an additive bias (per batch entry or shared, FlashAttentionBackward's attentionBias,
    CudaBackend.cs:8580-8604) or a keep-mask: the row threads of the tcgen05 kernels read them per (query, key); the
    mma.sync kernels (desc.path = generic) serve the same calls.  Several tiles per sequence, grouped-query heads,
    a padded batch entry, causal on top of the mask."""
    B, Hq, Hkv, Sq, Sk, D = 2, 4, 2, 200, 333, 128
    q, qf = gen((B, Hq, Sq, D), dtype, 981)
    k, kf = gen((B, Hkv, Sk, D), dtype, 982)
    v, vf = gen((B, Hkv, Sk, D), dtype, 983)
    dout, dof = gen((B, Hq, Sq, D), "f32", 984, scale=1.0)
    kv_len = np.array([Sk, Sk - 50], np.int32)
    rng = np.random.default_rng(985)
    bias = keep = None
    if kind == "bias":
        m = rng.standard_normal((B, Hq, Sq, Sk)).astype(np.float32)
        bias, mk = m, N.MASK_ADD_F32
    elif kind == "bias_broadcast":
        m = rng.standard_normal((1, Hq, Sq, Sk)).astype(np.float32)
        bias, mk = m, N.MASK_ADD_F32
    elif kind == "keep_u8":
        keep = rng.random((B, 1, Sq, Sk)) < 0.7
        keep[..., 0] = True
        m, mk = keep.astype(np.uint8), N.MASK_KEEP_U8
    else:
        keep = rng.random((1, 1, Sq, Sk)) < 0.7
        keep[..., 0] = True
        m, mk = keep.astype(np.float32), N.MASK_KEEP_F32
    info = {}
    dq, dk, dv = _fwd_bwd(q, k, v, dout, dtype=dtype, causal=True, bottom_right=True, mask=torch.from_numpy(m).cuda(),
                          mask_kind=mk, kv_len=kv_len, path=path, info=info)
    assert info["path"] == (N.PATH_PREFILL_SM100 if path == N.PATH_AUTO else N.PATH_GENERIC)
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, causal=True, causal_offset=Sk - Sq, bias=bias, keep=keep, kv_len=kv_len)
    _check(dq, rq, dtype, f"dQ {kind} path {path}")
    _check(dk, rk, dtype, f"dK {kind} path {path}")
    _check(dv, rv, dtype, f"dV {kind} path {path}")


def test_backward_bounded_waits_expire_cleanly():
    """Failure detection without a fault on the tcgen05 backward: with the test hook the producers withhold the streamed
    tiles, the bounded waits (20 ms) run out in both launches, poll() reports AIDN_ETIMEOUT and the next backward on the
    same handle is correct."""
    B, H, S, D = 1, 2, 384, 128
    q, qf = gen((B, H, S, D), "bf16", 991)
    k, kf = gen((B, H, S, D), "bf16", 992)
    v, vf = gen((B, H, S, D), "bf16", 993)
    dout, dof = gen((B, H, S, D), "f32", 994, scale=1.0)
    out = torch.zeros((B, H, S, D), device="cuda")
    lse = torch.zeros((B, H, S), device="cuda")
    dq, dk, dv = (torch.zeros((B, H, S, D), device="cuda") for _ in range(3))
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=H, num_kv_heads=H, causal=True, emit_lse=True)
    stream = torch.cuda.current_stream().cuda_stream
    common = dict(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), lse=lse.data_ptr(), batch=B, seq_q=S,
                  seq_kv=S, stream=stream)
    h.launch(**common)
    nb = h.backward_workspace_bytes(B, S)
    ws = torch.empty(nb, dtype=torch.uint8, device="cuda")
    bwd = lambda: h.backward(dout=dout.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(), dv=dv.data_ptr(), workspace=ws.data_ptr(),
                             workspace_bytes=nb, **common)
    h.debug_set(None, 3)
    bwd()
    with pytest.raises(N.AidnError) as e:
        h.poll(stream)
    assert e.value.status == N.ETIMEOUT
    h.debug_set(None, 0)
    bwd()
    h.poll(stream)
    assert h.last_path == N.PATH_PREFILL_SM100
    rq, rk, rv, _, _ = O.sdpa_backward(qf, kf, vf, dof, causal=True, causal_offset=0)
    _check(dq, rq, "bf16", "dQ after a timed-out backward")
    _check(dk, rk, "bf16", "dK after a timed-out backward")
    _check(dv, rv, "bf16", "dV after a timed-out backward")
    h.close()

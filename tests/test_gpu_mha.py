"""GPU parity of aidn_mha_forward (MultiHeadAttentionForward: Q/K/V projections, attention, output projection) against
the float64 oracle on the same rounded inputs.  The reference pins its fused call on the decomposed chain at 1e-4 in
fp32 (Engines/MultiHeadAttentionForwardTests.cs:101-124); this path computes in 16 bits with fp32 accumulation, so the
bound is the 16-bit contract of the attention path: max-abs <= 2e-2 and mean-abs <= 2e-3 of the largest reference
magnitude."""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O

from tests._harness import AIDN_DT, TORCH_DT, gen

pytestmark = pytest.mark.gpu


def _align(n, a=1024):
    return (n + a - 1) // a * a


def _run(x, ws, heads, *, dtype, in_dtype=None, w_dtype=None, out_dtype="f32", mask=None, want_stages=False):
    """x [B,S,Dm] and the four weights are CUDA tensors already in in_dtype / w_dtype."""
    in_dtype, w_dtype = in_dtype or dtype, w_dtype or dtype
    B, S, Dm = x.shape
    d = Dm // heads
    out = torch.full((B, S, Dm), float("nan"), dtype=TORCH_DT[out_dtype], device="cuda")
    mk = N.MASK_KEEP_U8 if mask is not None else N.MASK_NONE
    h = N.Handle(device=0, qkv_dtype=AIDN_DT[dtype], out_dtype=AIDN_DT[dtype], head_dim=d, num_q_heads=heads,
                 num_kv_heads=heads, mask_kind=mk)
    ms = (0, 0, 0, 0)
    if mask is not None:
        full = (B, heads, S, S)
        st = mask.stride()
        ms = tuple(0 if (mask.shape[a] == 1 and full[a] != 1) else st[a] for a in range(4))
    nb = h.mha_workspace_bytes(B, S, AIDN_DT[in_dtype], AIDN_DT[w_dtype])
    wsb = torch.zeros(nb + 1024, dtype=torch.uint8, device="cuda")
    base = _align(wsb.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    h.mha_forward(input=x.data_ptr(), q_weight=ws[0].data_ptr(), k_weight=ws[1].data_ptr(), v_weight=ws[2].data_ptr(),
                  out_weight=ws[3].data_ptr(), out=out.data_ptr(), batch=B, seq=S, input_dtype=AIDN_DT[in_dtype],
                  weight_dtype=AIDN_DT[w_dtype], out_dtype=AIDN_DT[out_dtype], workspace=base, workspace_bytes=nb,
                  stream=stream, mask=mask.data_ptr() if mask is not None else None, mask_stride=ms)
    h.poll(stream)
    launches = h.last_launch_count
    h.close()
    if not want_stages:
        return out, launches
    # the workspace holds, in this order: [input in 16 bits] [4 weights in 16 bits] Q K V [B,H,S,d] O [B,S,Dm]
    act = _align(B * S * Dm * 2)
    off = (act if in_dtype == "f32" else 0) + (4 * _align(Dm * Dm * 2) if w_dtype == "f32" else 0)
    off += base - wsb.data_ptr()
    view = lambda i, shape: wsb[off + i * act: off + i * act + B * S * Dm * 2].view(TORCH_DT[dtype]).view(shape)
    return out, launches, [view(i, (B, heads, S, d)) for i in range(3)] + [view(3, (B, S, Dm))]


def _inputs(B, S, heads, d, dtype, seed, in_dtype=None, w_dtype=None):
    Dm = heads * d
    x, xf = gen((B, S, Dm), in_dtype or dtype, seed)
    ws, wfs = [], []
    for i in range(4):
        w, wf = gen((Dm, Dm), w_dtype or dtype, seed + 1 + i, scale=1.0 / np.sqrt(Dm))
        ws.append(w)
        wfs.append(wf)
    return x, xf, ws, wfs


def _round(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a)).to(TORCH_DT[dtype]).to(torch.float32).numpy()


def _check(got, want, what):
    g = got.to(torch.float32).cpu().numpy()
    assert np.isfinite(g).all(), what
    mag = max(np.abs(want).max(), 1e-6)
    err = np.abs(g - want)
    assert err.max() / mag <= 2e-2, f"{what}: max error {err.max() / mag:.3e} of the largest magnitude"
    assert err.mean() / mag <= 2e-3, f"{what}: mean error {err.mean() / mag:.3e} of the largest magnitude"


SHAPES = [(2, 128, 2, 64), (1, 256, 2, 128), (2, 100, 4, 64), (3, 37, 4, 128), (1, 1, 2, 64), (2, 640, 8, 128),
          (1, 5, 4, 64)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_mha_forward_shapes_and_stages(shape, dtype):
    """Tile-aligned and ragged sequence lengths (the reference's any-length theory, MultiHeadAttentionForwardTests.cs:
    237-266), d_model 128 to 1024, both column-tile widths of the projection kernel; also checks the projected Q / K / V
    and the attention output the call leaves in its workspace, which localises a failure to one of the three launches."""
    B, S, heads, d = shape
    x, xf, ws, wfs = _inputs(B, S, heads, d, dtype, 4100 + S)
    out, launches, (q, k, v, o) = _run(x, ws, heads, dtype=dtype, want_stages=True)
    assert launches >= 3
    split = lambda t: t.reshape(B, S, heads, d).transpose(0, 2, 1, 3)
    xd = xf.astype(np.float64)
    for name, got, w in (("Q", q, wfs[0]), ("K", k, wfs[1]), ("V", v, wfs[2])):
        _check(got, split(xd @ w.astype(np.float64)), f"{name} projection {shape} {dtype}")
    _check(out, O.mha_forward(xf, *wfs, heads), f"output {shape} {dtype}")
    # the output projection alone, from the attention output the call itself produced
    _check(out, o.to(torch.float32).cpu().numpy().astype(np.float64) @ wfs[3].astype(np.float64),
           f"output projection {shape} {dtype}")


def test_mha_forward_many_tiles_per_cta():
    """More tiles than SMs: every persistent CTA walks several tiles and both TMEM accumulator slots."""
    B, S, heads, d = 4, 1024, 8, 128
    x, xf, ws, wfs = _inputs(B, S, heads, d, "bf16", 4300)
    out, _ = _run(x, ws, heads, dtype="bf16")
    _check(out, O.mha_forward(xf, *wfs, heads), "output 4x1024x1024")


@pytest.mark.parametrize("kind", ["causal_full", "causal_broadcast", "row_masked"])
def test_mha_forward_keep_masks(kind):
    """MultiHeadAttentionForwardTests.cs:126-162 (causal mask), :164-203 (a [1,1,S,S] mask broadcast over batch and
    heads equals the materialised one); CpuEngine.MultiHeadAttention.cs:481-485 (a fully masked row gives zeros)."""
    B, S, heads, d = 2, 150, 4, 64
    x, xf, ws, wfs = _inputs(B, S, heads, d, "bf16", 4400)
    tri = np.tril(np.ones((S, S), bool))
    if kind == "causal_full":
        m = np.broadcast_to(tri, (B, heads, S, S)).copy()
    elif kind == "causal_broadcast":
        m = tri[None, None].copy()
    else:
        m = np.ones((B, 1, S, S), bool)
        m[1, 0, 7, :] = False
    mask = torch.from_numpy(m.astype(np.uint8)).cuda()
    out, _ = _run(x, ws, heads, dtype="bf16", mask=mask)
    want = O.mha_forward(xf, *wfs, heads, mask=m)
    _check(out, want, f"masked output ({kind})")
    if kind == "row_masked":
        assert float(out[1, 7].abs().max()) == 0.0
    else:
        unmasked, _ = _run(x, ws, heads, dtype="bf16")
        assert float((out - unmasked).abs().max()) > 1e-3


@pytest.mark.parametrize("in_dtype,w_dtype,out_dtype", [("f32", "f32", "f32"), ("f32", "bf16", "f32"), ("bf16", "f32", "bf16"),
                                                         ("bf16", "bf16", "bf16")])
def test_mha_forward_fp32_operands_are_rounded_in_the_workspace(in_dtype, w_dtype, out_dtype):
    """The reference's tensors are fp32 (IEngine.cs:4201-4208); fp32 inputs and weights are rounded to the handle's
    16-bit type by the call itself and give the same result as operands rounded beforehand."""
    B, S, heads, d = 2, 200, 2, 128
    x, xf, ws, wfs = _inputs(B, S, heads, d, "bf16", 4500, in_dtype=in_dtype, w_dtype=w_dtype)
    out, launches = _run(x, ws, heads, dtype="bf16", in_dtype=in_dtype, w_dtype=w_dtype, out_dtype=out_dtype)
    assert launches == 3 + (1 if in_dtype == "f32" else 0) + (4 if w_dtype == "f32" else 0)
    want = O.mha_forward(_round(xf, "bf16"), *[_round(w, "bf16") for w in wfs], heads)
    _check(out, want, f"output {in_dtype}/{w_dtype}/{out_dtype}")
    if in_dtype == "f32" or w_dtype == "f32":
        xr = torch.from_numpy(xf).to(torch.bfloat16).cuda()
        wr = [torch.from_numpy(w).to(torch.bfloat16).cuda() for w in wfs]
        pre, _ = _run(xr, wr, heads, dtype="bf16", out_dtype=out_dtype)
        assert torch.equal(pre, out)


def test_mha_forward_is_bit_reproducible():
    B, S, heads, d = 2, 300, 4, 64
    x, _, ws, _ = _inputs(B, S, heads, d, "bf16", 4600)
    a, _ = _run(x, ws, heads, dtype="bf16")
    b, _ = _run(x, ws, heads, dtype="bf16")
    assert torch.equal(a, b)


def test_mha_forward_rejections():
    """Handles that do not describe this op (grouped-query heads, an output type other than the attention type, a
    log-sum-exp, softcap or additive-bias request) answer AIDN_EUNSUPPORTED; a short workspace, a null tensor or a
    foreign dtype are argument errors (MultiHeadAttentionForwardTests.cs:205-235 for the reference's own)."""
    stream = torch.cuda.current_stream().cuda_stream
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device="cuda")
    p = (buf.data_ptr() + 1023) // 1024 * 1024

    def call(h, **kw):
        args = dict(input=p, q_weight=p, k_weight=p, v_weight=p, out_weight=p, out=p, batch=1, seq=8,
                    input_dtype=N.BF16, weight_dtype=N.BF16, out_dtype=N.F32, workspace=p + (1 << 19), workspace_bytes=1 << 18,
                    stream=stream)
        args.update(kw)
        h.mha_forward(**args)

    for kw, status in ((dict(head_dim=64, num_q_heads=4, num_kv_heads=2), N.EUNSUPPORTED),       # grouped-query
                       (dict(head_dim=64, num_q_heads=4, num_kv_heads=4, out_dtype=N.F32), N.EUNSUPPORTED),
                       (dict(head_dim=64, num_q_heads=4, num_kv_heads=4, emit_lse=True), N.EUNSUPPORTED),
                       (dict(head_dim=64, num_q_heads=4, num_kv_heads=4, softcap=2.0), N.EUNSUPPORTED),
                       (dict(head_dim=64, num_q_heads=4, num_kv_heads=4, mask_kind=N.MASK_ADD_F32), N.EUNSUPPORTED)):
        kw.setdefault("out_dtype", N.BF16)
        with N.Handle(device=0, qkv_dtype=N.BF16, **kw) as h:
            with pytest.raises(N.AidnError) as ei:
                call(h)
            assert ei.value.status == status, kw
    with N.Handle(device=0, qkv_dtype=N.BF16, out_dtype=N.BF16, head_dim=64, num_q_heads=2, num_kv_heads=2) as h:
        for kw, status in ((dict(workspace_bytes=1024), N.EWORKSPACE), (dict(workspace=None), N.EWORKSPACE),
                           (dict(workspace=p + (1 << 19) + 16), N.EINVAL), (dict(input=None), N.EINVAL), (dict(batch=0), N.EINVAL),
                           (dict(input_dtype=N.F16), N.EINVAL)):
            with pytest.raises(N.AidnError) as ei:
                call(h, **kw)
            assert ei.value.status == status, kw
        call(h)   # the same arguments without the fault go through
        h.poll(stream)


def test_backend_mirror_fp32_tensors_and_mask():
    """The engine-level call as the reference makes it: fp32 tensors, a [1,1,S,S] boolean mask
    (MultiHeadAttentionForwardTests.cs:164-203), through the host mirror of the interface."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    B, S, heads, d = 2, 96, 2, 64
    Dm = heads * d
    x, xf, ws, wfs = _inputs(B, S, heads, d, "f32", 4700)
    m = np.tril(np.ones((S, S), bool))[None, None].copy()
    be = CudaBackend(0)
    out = be.AllocateBuffer(B * S * Dm)
    be.MultiHeadAttentionForward(GpuBuffer(x.view(-1)), *[GpuBuffer(w.view(-1)) for w in ws], out, B, S, Dm, heads,
                                 mask=GpuBuffer(torch.from_numpy(m.astype(np.uint8)).cuda().view(-1)), maskShape=m.shape)
    be.Synchronize()
    want = O.mha_forward(_round(xf, "bf16"), *[_round(w, "bf16") for w in wfs], heads, mask=m)
    _check(out.tensor.view(B, S, Dm), want, "backend mirror")
    assert be.launch_count == 8   # input cast, 4 weight casts, projections, attention, output projection
    be.Dispose()


def test_backend_mirror_rejects_bad_shapes():
    """MultiHeadAttentionForwardTests.cs:205-235 — wrong weight shape, dModel not divisible by numHeads, numHeads <= 0."""
    from aidotnet.tensors_b200.backend import CudaBackend
    be = CudaBackend(0)
    B, S, Dm = 1, 8, 128
    x, out, w = be.AllocateBuffer(B * S * Dm), be.AllocateBuffer(B * S * Dm), be.AllocateBuffer(Dm * Dm)
    bad = be.AllocateBuffer(Dm * (Dm + 1))
    with pytest.raises(ValueError):
        be.MultiHeadAttentionForward(x, bad, w, w, w, out, B, S, Dm, 2)
    with pytest.raises(ValueError):
        be.MultiHeadAttentionForward(x, w, w, w, w, out, B, S, Dm, 3)
    with pytest.raises(ValueError):
        be.MultiHeadAttentionForward(x, w, w, w, w, out, B, S, Dm, 0)
    with pytest.raises(ValueError):
        be.MultiHeadAttentionForward(x, w, w, w, None, out, B, S, Dm, 2)
    be.Dispose()


REFERENCE_SHAPES = [(3, 5, 12, 3), (2, 7, 24, 4), (1, 100, 32, 4), (4, 13, 48, 6), (5, 3, 8, 2), (2, 6, 6, 3), (3, 9, 30, 5)]


@pytest.mark.parametrize("batch,seq,d_model,heads", REFERENCE_SHAPES + [(1, s, 32, 4) for s in (1, 2, 3, 5, 31, 128)]
                         + [(2, 70, 256, 2), (1, 200, 192, 3)])
@pytest.mark.parametrize("masked", [False, True])
def test_mha_forward_exact_route_meets_the_reference_bound(batch, seq, d_model, heads, masked):
    """fp32 tensors through an fp32 handle: the shapes of MultiHeadAttentionForwardTests.cs:288-313 (head sizes 2 to 8),
    its any-length theory (:237-266) and its causal-mask theory (:315-344), at the reference's own bound of 1e-4
    absolute; also head sizes 128 and 64 with a width that is not a multiple of 128."""
    rng = np.random.default_rng(seq * 100 + d_model)
    xf = rng.standard_normal((batch, seq, d_model)).astype(np.float32)
    wfs = [(rng.standard_normal((d_model, d_model)) / np.sqrt(d_model)).astype(np.float32) for _ in range(4)]
    x, ws = torch.from_numpy(xf).cuda(), [torch.from_numpy(w).cuda() for w in wfs]
    m = np.tril(np.ones((seq, seq), bool))[None, None].copy() if masked else None
    mask = torch.from_numpy(m.astype(np.uint8)).cuda() if masked else None
    out, launches = _run(x, ws, heads, dtype="f32", mask=mask)
    assert launches == 3
    want = O.mha_forward(xf, *wfs, heads, mask=m)
    err = np.abs(out.cpu().numpy() - want).max()
    assert err <= 1e-4, f"max error {err:.3e}"


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
def test_mha_forward_16bit_odd_head_size(dtype):
    """16-bit tensors with a head size the tensor-core GEMM does not take (32): FFMA GEMM + generic attention."""
    B, S, heads, d = 2, 50, 4, 32
    x, xf, ws, wfs = _inputs(B, S, heads, d, dtype, 4800)
    out, _ = _run(x, ws, heads, dtype=dtype)
    _check(out, O.mha_forward(xf, *wfs, heads), f"output head_dim 32 {dtype}")


def test_backend_mirror_exact_switch_and_small_heads():
    """fp32 buffers: head size 64 goes to the tensor cores unless exact=True; head size 16 always runs in fp32."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    B, S = 2, 33
    be = CudaBackend(0)
    for heads, d, exact, tol in ((2, 64, True, 1e-4), (8, 16, False, 1e-4), (2, 64, False, None)):
        Dm = heads * d
        x, xf, ws, wfs = _inputs(B, S, heads, d, "f32", 4900 + d)
        out = be.AllocateBuffer(B * S * Dm)
        be.MultiHeadAttentionForward(GpuBuffer(x.view(-1)), *[GpuBuffer(w.view(-1)) for w in ws], out, B, S, Dm, heads, exact=exact)
        be.Synchronize()
        got = out.tensor.view(B, S, Dm)
        if tol is not None:
            assert np.abs(got.cpu().numpy() - O.mha_forward(xf, *wfs, heads)).max() <= tol
        else:
            _check(got, O.mha_forward(_round(xf, "bf16"), *[_round(w, "bf16") for w in wfs], heads), "tensor route")
    be.Dispose()


def test_mha_forward_bounded_waits_expire_cleanly():
    """Failure detection without a fault: a test hook makes the producers of the projection GEMMs (and of the attention
    kernel) withhold their loads, so every bounded wait (20 ms in this mode) runs out.  The kernels must unwind and free
    TMEM, poll() must report AIDN_ETIMEOUT, and the next call on the same handle must be correct."""
    B, S, heads, d = 2, 300, 2, 128
    Dm = heads * d
    x, xf, ws, wfs = _inputs(B, S, heads, d, "bf16", 5100)
    out = torch.zeros((B, S, Dm), device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, out_dtype=N.BF16, head_dim=d, num_q_heads=heads, num_kv_heads=heads)
    nb = h.mha_workspace_bytes(B, S, N.BF16, N.BF16)
    wsb = torch.zeros(nb + 1024, dtype=torch.uint8, device="cuda")
    base = _align(wsb.data_ptr())
    stream = torch.cuda.current_stream().cuda_stream
    call = lambda: h.mha_forward(input=x.data_ptr(), q_weight=ws[0].data_ptr(), k_weight=ws[1].data_ptr(),
                                 v_weight=ws[2].data_ptr(), out_weight=ws[3].data_ptr(), out=out.data_ptr(), batch=B, seq=S,
                                 input_dtype=N.BF16, weight_dtype=N.BF16, out_dtype=N.F32, workspace=base, workspace_bytes=nb,
                                 stream=stream)
    h.debug_set(None, 3)
    call()
    with pytest.raises(N.AidnError) as e:
        h.poll(stream)
    assert e.value.status == N.ETIMEOUT
    h.debug_set(None, 0)
    call()
    h.poll(stream)
    _check(out, O.mha_forward(xf, *wfs, heads), "call after a timed-out call")
    h.close()

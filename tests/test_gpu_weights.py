"""Attention probabilities on request: the `out attentionWeights` of IEngine.ScaledDotProductAttention
(IEngine.cs:4133-4140) and of IDirectGpuBackend.GroupedQueryAttention (IDirectGpuBackend.cs:1501-1503).

The reference checks them against its CPU engine to 2e-5 absolute
(tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/GpuCpuConsistencyTests.cs:951-955, :994-1001 with a softcap,
:1046-1060 under a boolean mask); the same bar is used here against the oracle's `want_weights`, together with what
holds at every size: each visible row sums to 1, masked positions and fully masked rows are exact zeros, every
element of the buffer is written, and weights @ V reproduces the output.
"""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O
from tests._harness import compare, compare_lse, gen, run_gpu

pytestmark = pytest.mark.gpu

TOL_W32 = 2e-5     # GpuCpuConsistencyTests.cs:953
TOL_W16 = 2e-3     # 16-bit inputs: same rounded inputs on both sides, fp32 arithmetic, ex2.approx exponentials


def _check_weights(w: torch.Tensor, ref_w: np.ndarray, tol: float, what: str):
    got = w.cpu().numpy()
    assert got.shape == ref_w.shape
    assert np.isfinite(got).all(), f"{what}: an element of the weights buffer was not written"
    assert (got[ref_w == 0.0] == 0.0).all(), f"{what}: a masked position holds a non-zero weight"
    assert np.abs(got - ref_w).max() <= tol, f"{what}: weights differ by {np.abs(got - ref_w).max():.3e}"
    sums = got.sum(-1)
    live = ref_w.sum(-1) > 0
    sum_tol = 1e-4 if tol == TOL_W32 else 5e-3
    assert np.abs(sums[live] - 1.0).max(initial=0.0) <= sum_tol, f"{what}: rows do not sum to 1"
    assert (sums[~live] == 0.0).all(), f"{what}: a fully masked row is not all zero"


def test_reference_cross_attention_vectors():
    """GpuCpuConsistencyTests.cs:898-911: B=2 H=2 Sq=2 Sk=3 D=3, arithmetic sequences, scale 0.75."""
    B, H, Sq, Sk, D = 2, 2, 2, 3, 3
    qf = (-0.2 + 0.03 * np.arange(B * H * Sq * D, dtype=np.float32)).reshape(B, H, Sq, D).astype(np.float32)
    kf = (0.5 - 0.025 * np.arange(B * H * Sk * D, dtype=np.float32)).reshape(B, H, Sk, D).astype(np.float32)
    vf = (-0.1 + 0.04 * np.arange(B * H * Sk * D, dtype=np.float32)).reshape(B, H, Sk, D).astype(np.float32)
    q, k, v = (torch.from_numpy(x).cuda() for x in (qf, kf, vf))
    for softcap in (0.0, 2.0):                       # :962-1003 repeats it with a logit softcap
        out, _, info = run_gpu(q, k, v, dtype="f32", scale=0.75, softcap=softcap, want_weights=True)
        assert info["path"] == N.PATH_GENERIC
        ref, _, ref_w = O.sdpa(qf, kf, vf, scale=0.75, softcap=softcap, want_weights=True)
        assert np.abs(out.cpu().numpy() - ref).max() <= 2e-5
        _check_weights(info["weights"], ref_w, TOL_W32, f"cross attention, softcap {softcap}")
    mask = np.array([1, 0, 1, 0, 1, 1, 1, 1, 0, 1, 0, 0, 0, 1, 1, 1, 1, 0, 1, 0, 0, 0, 1, 0], np.float32).reshape(B, H, Sq, Sk)
    out, _, info = run_gpu(q, k, v, dtype="f32", scale=0.75, mask=torch.from_numpy(mask).cuda(), mask_kind=N.MASK_KEEP_F32,
                           want_weights=True)                                    # :1005-1061
    ref, _, ref_w = O.sdpa(qf, kf, vf, scale=0.75, mask=mask, mask_kind=O.MASK_KEEP_F32, want_weights=True)
    assert np.abs(out.cpu().numpy() - ref).max() <= 2e-5
    _check_weights(info["weights"], ref_w, TOL_W32, "full boolean mask")


@pytest.mark.parametrize("dtype,D", [("f32", 64), ("f32", 40), ("f32", 128), ("bf16", 128), ("f16", 64), ("f32", 256)])
@pytest.mark.parametrize("causal", [False, True])
def test_weights_match_oracle_ragged_gqa(dtype, D, causal):
    B, Hq, Hkv, Sq, Sk = 2, 6, 2, 70, 133     # nothing a multiple of a tile
    s = 1.0 if dtype == "f32" else 0.5
    q, qf = gen((B, Hq, Sq, D), dtype, 701, s)
    k, kf = gen((B, Hkv, Sk, D), dtype, 702, s)
    v, vf = gen((B, Hkv, Sk, D), dtype, 703, s)
    kv = np.array([133, 41], np.int32)
    out, lse, info = run_gpu(q, k, v, dtype=dtype, causal=causal, kv_len=torch.from_numpy(kv).cuda(), want_lse=True,
                             want_weights=True)
    assert info["path"] == N.PATH_GENERIC          # AUTO falls to the fp32 kernel whenever weights are asked for
    ref, ref_lse, ref_w = O.sdpa(qf, kf, vf, causal=causal, kv_len=kv, want_lse=True, want_weights=True)
    compare(out, ref, dtype, "output beside weights")
    compare_lse(lse, ref_lse, dtype, "lse beside weights")
    _check_weights(info["weights"], ref_w, TOL_W32 if dtype == "f32" else TOL_W16, f"{dtype} D{D} causal {causal}")
    # weights @ V is the output
    g = Hq // Hkv
    wv = torch.einsum("bhqk,bhkd->bhqd", info["weights"], v.float().repeat_interleave(g, dim=1))
    assert (wv - out).abs().max().item() <= (2e-5 if dtype == "f32" else 2e-3)


def test_weights_with_masks_bias_and_fully_masked_rows():
    B, H, Sq, Sk, D = 2, 3, 45, 97, 64
    q, qf = gen((B, H, Sq, D), "f32", 711, 1.0)
    k, kf = gen((B, H, Sk, D), "f32", 712, 1.0)
    v, vf = gen((B, H, Sk, D), "f32", 713, 1.0)
    rng = np.random.default_rng(7)
    keep = (rng.random((1, 1, Sq, Sk)) > 0.4)
    keep[0, 0, 5] = False                       # rows with no visible key
    keep[0, 0, 44] = False
    out, lse, info = run_gpu(q, k, v, dtype="f32", mask=torch.from_numpy(keep.astype(np.uint8)).cuda(),
                             mask_kind=N.MASK_KEEP_U8, want_lse=True, want_weights=True)
    ref, ref_lse, ref_w = O.sdpa(qf, kf, vf, mask=keep, mask_kind=O.MASK_KEEP_U8, want_lse=True, want_weights=True)
    compare_lse(lse, ref_lse, "f32", "lse, shared keep mask")
    _check_weights(info["weights"], ref_w, TOL_W32, "shared keep mask")
    assert (info["weights"][:, :, 5] == 0).all() and (info["weights"][:, :, 44] == 0).all()

    bias = rng.standard_normal((B, H, Sq, Sk)).astype(np.float32)
    out, lse, info = run_gpu(q, k, v, dtype="f32", mask=torch.from_numpy(bias).cuda(), mask_kind=N.MASK_ADD_F32,
                             causal=True, bottom_right=False, causal_offset=0, want_lse=True, want_weights=True)
    ref, ref_lse, ref_w = O.sdpa(qf, kf, vf, mask=bias, mask_kind=O.MASK_ADD_F32, causal=True, causal_offset=0,
                                 want_lse=True, want_weights=True)
    compare(out, ref, "f32", "bias + top-left causal")
    _check_weights(info["weights"], ref_w, TOL_W32, "bias + top-left causal")


def test_negative_causal_offset_rows_without_keys():
    """Sq > Sk with bottom-right causal: the first Sq - Sk - ... rows see nothing and get all-zero weights."""
    B, H, Sq, Sk, D = 1, 2, 90, 40, 64
    q, qf = gen((B, H, Sq, D), "f32", 721, 1.0)
    k, kf = gen((B, H, Sk, D), "f32", 722, 1.0)
    v, vf = gen((B, H, Sk, D), "f32", 723, 1.0)
    out, _, info = run_gpu(q, k, v, dtype="f32", causal=True, want_weights=True)
    ref, _, ref_w = O.sdpa(qf, kf, vf, causal=True, want_weights=True)
    _check_weights(info["weights"], ref_w, TOL_W32, "negative causal offset")
    assert (info["weights"][:, :, :Sq - Sk - 1] == 0).all()


def test_single_query_row_with_weights_leaves_the_decode_kernel():
    B, Hq, Hkv, Sk, D = 3, 8, 2, 700, 128
    q, qf = gen((B, Hq, 1, D), "bf16", 731)
    k, kf = gen((B, Hkv, Sk, D), "bf16", 732)
    v, vf = gen((B, Hkv, Sk, D), "bf16", 733)
    out, _, info = run_gpu(q, k, v, dtype="bf16", want_weights=True)
    assert info["path"] == N.PATH_GENERIC
    ref, _, ref_w = O.sdpa(qf, kf, vf, want_weights=True)
    compare(out, ref, "bf16", "decode-shaped call with weights")
    _check_weights(info["weights"], ref_w, TOL_W16, "decode-shaped call with weights")


def test_weights_are_refused_where_they_are_not_produced():
    q, _ = gen((1, 4, 256, 128), "bf16", 741)
    k, _ = gen((1, 4, 256, 128), "bf16", 742)
    with pytest.raises(N.AidnError) as e:
        run_gpu(q, k, k, dtype="bf16", path=N.PATH_PREFILL_SM100, want_weights=True)
    assert e.value.status == N.EUNSUPPORTED
    pool = torch.zeros((4, 64, 4, 128), dtype=torch.bfloat16, device="cuda")
    table = torch.arange(4, dtype=torch.int32, device="cuda").reshape(1, 4)
    out = torch.zeros((1, 4, 256, 128), device="cuda")
    w = torch.zeros((1, 4, 256, 256), device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=4, num_kv_heads=4)
    with pytest.raises(N.AidnError) as e:
        h.launch(q=q.data_ptr(), k=pool.data_ptr(), v=pool.data_ptr(), out=out.data_ptr(), batch=1, seq_q=256, seq_kv=256,
                 stream=torch.cuda.current_stream().cuda_stream, block_table=table.data_ptr(), block_table_stride=4,
                 block_size=64, num_blocks=4, weights=w.data_ptr())
    assert e.value.status == N.EUNSUPPORTED
    h.close()


def test_backend_mirror_returns_weights():
    """CudaBackend.ScaledDotProductAttention (CudaBackend.cs:8322-8372) and GroupedQueryAttention (:8721-8745) with the
    optional buffer, bottom-right and top-left causal respectively."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    B, Hq, Hkv, Sq, Sk, D = 2, 4, 2, 33, 50, 32
    q, qf = gen((B, Hq, Sq, D), "f32", 751, 1.0)
    k, kf = gen((B, Hkv, Sk, D), "f32", 752, 1.0)
    v, vf = gen((B, Hkv, Sk, D), "f32", 753, 1.0)
    be = CudaBackend(0)
    scale = 1.0 / np.sqrt(D)
    out = be.AllocateBuffer(B * Hq * Sq * D)
    w = be.AllocateBuffer(B * Hq * Sq * Sk)
    be.ScaledDotProductAttention(GpuBuffer(q.reshape(-1)), GpuBuffer(k.reshape(-1)), GpuBuffer(v.reshape(-1)), out, w, None,
                                 B, Hq, Sq, Sk, D, scale, True, 0.0, Hkv)
    be.Synchronize()
    ref, _, ref_w = O.sdpa(qf, kf, vf, causal=True, want_weights=True)
    _check_weights(w.tensor.reshape(B, Hq, Sq, Sk), ref_w, TOL_W32, "backend SDPA weights")
    assert np.abs(out.tensor.cpu().numpy().reshape(ref.shape) - ref).max() <= 2e-5
    be.GroupedQueryAttention(GpuBuffer(q.reshape(-1)), GpuBuffer(k.reshape(-1)), GpuBuffer(v.reshape(-1)), out, w,
                             B, Hq, Hkv, Sq, Sk, D, scale, True)
    be.Synchronize()
    ref, _, ref_w = O.sdpa(qf, kf, vf, causal=True, causal_offset=0, want_weights=True)
    _check_weights(w.tensor.reshape(B, Hq, Sq, Sk), ref_w, TOL_W32, "backend GQA weights")
    small = be.AllocateBuffer(8)
    with pytest.raises(ValueError):
        be.ScaledDotProductAttention(GpuBuffer(q.reshape(-1)), GpuBuffer(k.reshape(-1)), GpuBuffer(v.reshape(-1)), out, small,
                                     None, B, Hq, Sq, Sk, D, scale, True, 0.0, Hkv)
    be.Dispose()

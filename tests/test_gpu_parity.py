"""GPU parity: every CUDA kernel, called through the C ABI, against the CPU oracle on the same seeded inputs,
the committed golden fixtures, and size-independent properties at the full benchmark sizes.

Case lists follow the reference's own attention tests (tests/AiDotNet.Tensors.Tests/Engines/...): odd sequence
lengths, Sq != Sk, GQA ratios 1/2/3/4/8, MQA, fully masked rows, broadcast masks, additive bias with LSE.
"""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O
from tests._harness import TOL_16_MAX, TOL_16_MEAN, gen_config, reference_rows, compare, compare_lse, gen, oracle_rows, run_gpu

pytestmark = pytest.mark.gpu


def _t(x, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dtype).cuda()


# ------------------------------------------------------------------------------------------------ generic / fp32
def test_config1_fp32_noncausal():
    """BASELINE config 1: fp32, B1 H8 S512 D64, no mask, scale 1/sqrt(D); <= 1e-5 relative."""
    q, qf = gen_config(1, 0, (1, 8, 512, 64), "f32", 1.0)
    k, kf = gen_config(1, 1, (1, 8, 512, 64), "f32", 1.0)
    v, vf = gen_config(1, 2, (1, 8, 512, 64), "f32", 1.0)
    out, _, info = run_gpu(q, k, v, dtype="f32")
    assert info["path"] == N.PATH_GENERIC
    compare(out, O.sdpa(qf, kf, vf), "f32", "config1")


def test_golden_cross_attention_and_masks(golden):
    """GpuCpuConsistencyTests.cs:895-1061 (2e-5 there): D=3, Sq=2, Sk=3; full bool mask; logit softcap."""
    q, k, v = (_t(golden[n]) for n in ("cross_q", "cross_k", "cross_v"))
    out, _, _ = run_gpu(q, k, v, dtype="f32", scale=0.75)
    assert np.abs(out.cpu().numpy() - golden["cross_out"]).max() <= 2e-5
    m = golden["boolmask_mask"]
    out, _, _ = run_gpu(q, k, v, dtype="f32", scale=0.75, mask=_t(m, torch.uint8), mask_kind=N.MASK_KEEP_U8)
    assert np.abs(out.cpu().numpy() - golden["boolmask_out"]).max() <= 2e-5
    out, _, _ = run_gpu(q, k, v, dtype="f32", scale=0.75, mask=_t(m.astype(np.float32)), mask_kind=N.MASK_KEEP_F32)
    assert np.abs(out.cpu().numpy() - golden["boolmask_out"]).max() <= 2e-5
    q, k, v = (_t(golden[n]) for n in ("capcross_q", "capcross_k", "capcross_v"))
    out, _, _ = run_gpu(q, k, v, dtype="f32", scale=1.5, softcap=2.0)
    assert np.abs(out.cpu().numpy() - golden["capcross_out"]).max() <= 2e-5


def test_golden_softcap_closed_form(golden):
    """BatchMatMulAndAttentionTests.cs:287-317: D=1, one query, two keys."""
    out, _, _ = run_gpu(_t(golden["softcap_q"]), _t(golden["softcap_k"]), _t(golden["softcap_v"]), dtype="f32",
                        scale=1.0, softcap=2.0)
    assert abs(float(out.cpu().ravel()[0]) - float(golden["softcap_out"][0])) <= 1e-4


@pytest.mark.parametrize("mb,mh", [(1, 1), (2, 1), (1, 3), (2, 3)])
def test_golden_broadcast_masks(golden, mb, mh):
    """SdpaMaskBroadcastTests.cs:61-114: size-1 mask axes broadcast."""
    q, k, v = (_t(golden[n]) for n in ("bcast_q", "bcast_k", "bcast_v"))
    S = q.shape[2]
    mask = np.broadcast_to(np.tril(np.ones((S, S), np.uint8)), (mb, mh, S, S)).copy()
    out, _, _ = run_gpu(q, k, v, dtype="f32", mask=_t(mask, torch.uint8), mask_kind=N.MASK_KEEP_U8)
    assert np.abs(out.cpu().numpy() - golden["bcast_out"]).max() <= 1e-5
    out2, _, _ = run_gpu(q, k, v, dtype="f32", causal=True)
    assert np.abs(out2.cpu().numpy() - golden["bcast_out"]).max() <= 1e-5


@pytest.mark.parametrize("causal", [False, True])
def test_golden_gqa(golden, causal):
    """RopeGqaOpenClTests.cs:200-279: Hq 6 / Hkv 2 (ratio 3), D=8, S=5 (1e-4 there)."""
    q, k, v = (_t(golden[n]) for n in ("gqa_q", "gqa_k", "gqa_v"))
    out, _, _ = run_gpu(q, k, v, dtype="f32", causal=causal, bottom_right=False)
    want = golden["gqa_out_causal"] if causal else golden["gqa_out_plain"]
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-5


def test_golden_bias_and_lse(golden):
    """FlashAttentionBiasTests.cs: 3-D (batch-broadcast) and 4-D bias, LSE = max + ln(sum), top-left causal."""
    q, k, v = (_t(golden[n]) for n in ("bias_q", "bias_k", "bias_v"))
    out, lse, _ = run_gpu(q, k, v, dtype="f32", mask=_t(golden["bias3"][None]), mask_kind=N.MASK_ADD_F32, want_lse=True)
    assert np.abs(out.cpu().numpy() - golden["bias3_out"]).max() <= 2e-5
    assert np.abs(lse.cpu().numpy() - golden["bias3_lse"]).max() <= 2e-5
    out, lse, _ = run_gpu(q, k, v, dtype="f32", mask=_t(golden["bias4"]), mask_kind=N.MASK_ADD_F32, want_lse=True,
                          causal=True, bottom_right=False)
    assert np.abs(out.cpu().numpy() - golden["bias4c_out"]).max() <= 2e-5
    assert np.abs(lse.cpu().numpy() - golden["bias4c_lse"]).max() <= 2e-5


@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 37, 53, 40), (1, 8, 1, 130, 130, 128), (2, 3, 3, 65, 200, 256),
                                   (1, 6, 2, 17, 300, 72)])
def test_generic_kernel_shapes(dtype, shape):
    """Odd lengths, Sq != Sk, GQA 2/8/1/3, head dims off the tensor-core path; causal + padding + LSE."""
    B, Hq, Hkv, Sq, Sk, D = shape
    q, qf = gen((B, Hq, Sq, D), dtype, 11)
    k, kf = gen((B, Hkv, Sk, D), dtype, 12)
    v, vf = gen((B, Hkv, Sk, D), dtype, 13)
    kv = np.array([Sk, max(1, Sk // 3)][:B], np.int32)
    out, lse, info = run_gpu(q, k, v, dtype=dtype, causal=True, kv_len=_t(kv, torch.int32), want_lse=True,
                             path=N.PATH_GENERIC)
    ref, rlse, _ = O.sdpa(qf, kf, vf, causal=True, kv_len=kv, want_lse=True)
    compare(out, ref, dtype, f"generic {shape}")
    compare_lse(lse, rlse, dtype)


def test_fully_masked_rows_and_negative_offset():
    """A fully masked row gives zeros and LSE -inf (CpuEngine.cs:27822-27827, 29244-29250)."""
    q, qf = gen((1, 2, 40, 64), "f32", 21)
    k, kf = gen((1, 2, 24, 64), "f32", 22)
    v, vf = gen((1, 2, 24, 64), "f32", 23)
    # bottom-right causal with Sq > Sk: the first Sq - Sk rows see nothing
    out, lse, _ = run_gpu(q, k, v, dtype="f32", causal=True, want_lse=True)
    ref, rlse, _ = O.sdpa(qf, kf, vf, causal=True, want_lse=True)
    assert np.all(ref[:, :, :15] == 0) and np.all(out.cpu().numpy()[:, :, :15] == 0)
    compare(out, ref, "f32")
    compare_lse(lse, rlse, "f32")
    out, _, _ = run_gpu(q, k, v, dtype="f32", kv_len=_t(np.array([0], np.int32), torch.int32))
    assert np.all(out.cpu().numpy() == 0)


def test_output_in_input_dtype():
    q, qf = gen((1, 2, 33, 64), "bf16", 31)
    k, kf = gen((1, 2, 70, 64), "bf16", 32)
    v, vf = gen((1, 2, 70, 64), "bf16", 33)
    out, _, _ = run_gpu(q, k, v, dtype="bf16", out_dtype="bf16", path=N.PATH_GENERIC)
    assert out.dtype == torch.bfloat16
    compare(out, O.sdpa(qf, kf, vf), "bf16")


# ------------------------------------------------------------------------------------------------ decode
def test_golden_flash_decode_shapes(golden):
    """FlashDecodeCudaTests.cs:43-126 through the backend mirror: cache stored [seqLen, kvHeads, D]."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    be = CudaBackend(0)
    for n, (h, hk, d, L) in enumerate(golden["decode_shapes"]):
        qb, kb, vb = (GpuBuffer(_t(golden[f"decode{n}_{x}"]).reshape(-1)) for x in "qkv")
        for splits in (0, 1, 8):
            ob = be.FlashDecode(qb, kb, vb, int(h), int(hk), int(d), int(L), 1.0 / np.sqrt(np.float32(d)), splits)
            be.Synchronize()
            got = ob.tensor.cpu().numpy().reshape(h, d)
            e = golden[f"decode{n}_out"]
            assert np.all(np.abs(got - e) <= 2e-5 + 2e-5 * np.abs(e)), (n, splits)
    be.Dispose()


@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape", [(3, 8, 8, 700, 128), (2, 8, 2, 1000, 64), (2, 16, 2, 333, 128), (1, 6, 2, 129, 64),
                                   (2, 4, 4, 513, 256), (1, 12, 1, 64, 128)])
@pytest.mark.parametrize("chunk", [0, 64])
def test_decode_kernel_shapes(dtype, shape, chunk):
    """Ragged kv_len per batch entry, GQA ratios 1/4/8/3/12 (MQA), every dtype, forced small splits."""
    B, Hq, Hkv, L, D = shape
    if dtype == "f32" and D == 256:
        pytest.skip("fp32 D=256 is served by the generic kernel")
    q, qf = gen((B, Hq, 1, D), dtype, 41)
    k, kf = gen((B, Hkv, L, D), dtype, 42)
    v, vf = gen((B, Hkv, L, D), dtype, 43)
    kv = np.array([L, L // 2 + 1, 7][:B], np.int32)
    out, lse, info = run_gpu(q, k, v, dtype=dtype, kv_len=_t(kv, torch.int32), want_lse=True, decode_chunk=chunk)
    assert info["path"] == N.PATH_DECODE
    ref, rlse, _ = O.sdpa(qf, kf, vf, kv_len=kv, want_lse=True)
    compare(out, ref, dtype, f"decode {shape}")
    compare_lse(lse, rlse, dtype)


def test_decode_with_masks_and_softcap():
    B, Hq, Hkv, L, D = 2, 8, 4, 300, 128
    q, qf = gen((B, Hq, 1, D), "bf16", 51)
    k, kf = gen((B, Hkv, L, D), "bf16", 52)
    v, vf = gen((B, Hkv, L, D), "bf16", 53)
    rng = np.random.default_rng(5)
    keep = (rng.random((B, 1, 1, L)) > 0.3).astype(np.uint8)
    keep[1] = 0  # batch entry 1 sees nothing
    out, _, _ = run_gpu(q, k, v, dtype="bf16", mask=_t(keep, torch.uint8), mask_kind=N.MASK_KEEP_U8, softcap=5.0,
                        decode_chunk=64)
    ref = O.sdpa(qf, kf, vf, mask=keep, mask_kind=O.MASK_KEEP_U8, softcap=5.0)
    compare(out, ref, "bf16")
    assert np.all(out[1].cpu().numpy() == 0)
    bias = rng.standard_normal((B, Hq, 1, L)).astype(np.float32)
    out, _, _ = run_gpu(q, k, v, dtype="bf16", mask=_t(bias), mask_kind=N.MASK_ADD_F32)
    compare(out, O.sdpa(qf, kf, vf, mask=bias, mask_kind=O.MASK_ADD_F32), "bf16")


def test_config4_batched_decode_full_size():
    """BASELINE config 4: B64 H32 D128 bf16, kv_len uniform in [512, 4096], padded cache [64,32,4096,128]."""
    from aidotnet.tensors_b200 import synth
    B, H, L, D = 64, 32, 4096, 128
    q, qf = gen_config(4, 0, (B, H, 1, D), "bf16")
    k, kf = gen_config(4, 1, (B, H, L, D), "bf16")
    v, vf = gen_config(4, 2, (B, H, L, D), "bf16")
    kv = synth.lengths(4, B, 512, L)
    out, _, info = run_gpu(q, k, v, dtype="bf16", kv_len=_t(kv, torch.int32))
    assert info["path"] == N.PATH_DECODE
    ref = O.sdpa(qf, kf, vf, kv_len=kv)
    compare(out, ref, "bf16", "config4")
    # determinism: fixed split count => fixed reduction order => identical bits
    out2, _, _ = run_gpu(q, k, v, dtype="bf16", kv_len=_t(kv, torch.int32))
    assert torch.equal(out, out2)


# ------------------------------------------------------------------------------------------------ tcgen05 prefill
PREFILL_SHAPES = [
    # B, Hq, Hkv, Sq, Sk, D, causal
    (1, 1, 1, 128, 128, 128, False),   # one tile, one KV tile
    (1, 1, 1, 256, 128, 128, False),   # both tiles of a CTA
    (1, 1, 1, 128, 384, 128, False),   # three KV tiles: accumulation, ring reuse, rescale
    (1, 2, 1, 256, 256, 128, True),    # head pair (GQA 2), causal diagonal
    (2, 4, 4, 300, 300, 128, True),    # ragged rows, row-tile pairs with an odd tile count
    (1, 8, 2, 200, 456, 128, True),    # GQA 4, Sq != Sk (bottom-right causal)
    (2, 3, 1, 129, 1025, 128, False),  # odd group (3): row-pair mode under GQA
    (1, 4, 2, 640, 640, 64, True),     # head_dim 64
    (1, 2, 2, 1024, 1024, 128, True),  # longer causal
]


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", PREFILL_SHAPES)
def test_prefill_sm100_shapes(dtype, shape):
    B, Hq, Hkv, Sq, Sk, D, causal = shape
    q, qf = gen((B, Hq, Sq, D), dtype, 61)
    k, kf = gen((B, Hkv, Sk, D), dtype, 62)
    v, vf = gen((B, Hkv, Sk, D), dtype, 63)
    out, lse, info = run_gpu(q, k, v, dtype=dtype, causal=causal, want_lse=True, path=N.PATH_PREFILL_SM100)
    assert info["path"] == N.PATH_PREFILL_SM100
    ref, rlse, _ = O.sdpa(qf, kf, vf, causal=causal, want_lse=True)
    compare(out, ref, dtype, f"prefill {shape}")
    compare_lse(lse, rlse, dtype)


def test_prefill_sm100_padding_and_dtype_out():
    B, Hq, Hkv, Sq, Sk, D = 2, 4, 2, 260, 700, 128
    q, qf = gen((B, Hq, Sq, D), "bf16", 71)
    k, kf = gen((B, Hkv, Sk, D), "bf16", 72)
    v, vf = gen((B, Hkv, Sk, D), "bf16", 73)
    kv = np.array([700, 131], np.int32)
    out, _, _ = run_gpu(q, k, v, dtype="bf16", out_dtype="bf16", causal=True, kv_len=_t(kv, torch.int32),
                        path=N.PATH_PREFILL_SM100)
    compare(out, O.sdpa(qf, kf, vf, causal=True, kv_len=kv), "bf16")
    # top-left causal with Sq < Sk and large values that force the lazy rescale to fire
    q2, q2f = gen((B, Hq, Sq, D), "bf16", 74, 2.0)
    out, _, _ = run_gpu(q2, k, v, dtype="bf16", causal=True, bottom_right=False, path=N.PATH_PREFILL_SM100)
    compare(out, O.sdpa(q2f, kf, vf, causal=True, causal_offset=0), "bf16")


ROLE_LAYOUT_CASES = [
    # B, Hq, Hkv, Sq, Sk, D, causal, out dtype, what it selects
    (4, 8, 2, 1536, 1536, 128, True, "f32"),    # head pairs: epilogue warpgroup; 192 items, several per CTA
    (4, 8, 2, 1536, 1536, 128, True, "bf16"),   # ... one staging buffer per 64 columns
    (3, 6, 6, 1100, 1100, 128, False, "f32"),   # row pairs without a causal mask: epilogue warpgroup, ragged last tile
    (3, 6, 6, 1100, 1100, 128, True, "f32"),    # row pairs under a causal mask: the softmax warps run the epilogue
    (2, 12, 4, 900, 900, 64, True, "bf16"),     # odd group (3): row pairs; head_dim 64
    (2, 8, 4, 700, 300, 128, True, "f32"),      # Sq > Sk, bottom-right: the first row tiles see no key at all
]


@pytest.mark.parametrize("case", ROLE_LAYOUT_CASES)
def test_prefill_sm100_both_role_layouts_many_items_per_cta(case):
    """The kernel has two role layouts (softmax warps or a fourth warpgroup run the epilogue) chosen by item shape.
    Shapes with more work items than SMs, so that every hand-over between consecutive items of a CTA is exercised
    (O released to the next item's first P.V product, row sums passed through shared memory, both staging buffers),
    with ragged lengths, tiles without any visible key, 16-bit and fp32 output, and LSE."""
    B, Hq, Hkv, Sq, Sk, D, causal, odt = case
    q, qf = gen((B, Hq, Sq, D), "bf16", 131)
    k, kf = gen((B, Hkv, Sk, D), "bf16", 132)
    v, vf = gen((B, Hkv, Sk, D), "bf16", 133)
    kv = np.array([Sk, max(1, Sk // 3), 0, Sk - 7][:B], np.int32)     # full, short, empty, ragged
    out, lse, info = run_gpu(q, k, v, dtype="bf16", out_dtype=odt, causal=causal, kv_len=_t(kv, torch.int32),
                             want_lse=True, path=N.PATH_PREFILL_SM100)
    assert info["path"] == N.PATH_PREFILL_SM100
    ref, rlse, _ = O.sdpa(qf, kf, vf, causal=causal, kv_len=kv, want_lse=True)
    compare(out, ref, "bf16", f"role layouts {case}")
    compare_lse(lse, rlse, "bf16")
    # twice on one handle: scheduler counters, cached tensor maps and barrier phases start over
    again, _, _ = run_gpu(q, k, v, dtype="bf16", out_dtype=odt, causal=causal, kv_len=_t(kv, torch.int32),
                          path=N.PATH_PREFILL_SM100)
    assert torch.equal(again, out)


def test_prefill_sm100_masked_instantiation_on_both_layouts():
    """Softcap + additive bias (the MASKED instantiation) with head pairs (epilogue warpgroup) and with row pairs."""
    for Hq, Hkv in ((8, 2), (3, 3)):
        B, S, D = 2, 640, 128
        q, qf = gen((B, Hq, S, D), "bf16", 141)
        k, kf = gen((B, Hkv, S, D), "bf16", 142)
        v, vf = gen((B, Hkv, S, D), "bf16", 143)
        bias = np.random.default_rng(3).standard_normal((B, Hq, S, S)).astype(np.float32)
        out, lse, info = run_gpu(q, k, v, dtype="bf16", causal=True, softcap=3.0, mask=_t(bias), mask_kind=N.MASK_ADD_F32,
                                 want_lse=True, path=N.PATH_PREFILL_SM100)
        ref, rlse, _ = O.sdpa(qf, kf, vf, causal=True, softcap=3.0, mask=bias, mask_kind=O.MASK_ADD_F32, want_lse=True)
        compare(out, ref, "bf16", f"masked, Hq {Hq} Hkv {Hkv}")
        compare_lse(lse, rlse, "bf16")


@pytest.mark.parametrize("case", [(1, 8, 4, 640, 128, "f32", True), (2, 6, 6, 500, 64, "bf16", True), (1, 4, 4, 384, 128, "f32", False)])
def test_prefill_sm100_peer_out_on_one_device(case):
    """args.peer_out (the fused gather of a head-sharded launch) with the "other ranks" played by further tensors on
    the same device: every output box has to arrive in `out` and in each of them, through both role layouts, with
    guard words around every tensor intact.  (Across two devices: tests/test_gpu_multi.py.)"""
    from tests._harness import guarded, check_guards, TORCH_DT
    B, Hq, Hkv, S, D, odt, causal = case
    q, _ = gen((B, Hq, S, D), "bf16", 151)
    k, _ = gen((B, Hkv, S, D), "bf16", 152)
    v, _ = gen((B, Hkv, S, D), "bf16", 153)
    full, _, _ = run_gpu(q, k, v, dtype="bf16", out_dtype=odt, causal=causal, path=N.PATH_PREFILL_SM100)
    flats, bodies = zip(*(guarded((B, Hq, S, D), TORCH_DT[odt], q.device, fill=0.0) for _ in range(4)))
    stream = torch.cuda.current_stream().cuda_stream
    half = Hq // 2
    for hb in (0, half):   # two "ranks", one after the other
        h = N.Handle(device=0, qkv_dtype=N.BF16, out_dtype=N.F32 if odt == "f32" else N.BF16, head_dim=D, num_q_heads=Hq,
                     num_kv_heads=Hkv, causal=causal, head_begin=hb, head_count=half, path=N.PATH_PREFILL_SM100)
        h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=bodies[0].data_ptr(), batch=B, seq_q=S, seq_kv=S,
                 stream=stream, peer_out=[t.data_ptr() for t in bodies[1:]])
        h.poll(stream)
        assert h.last_launch_count == 1
        h.close()
    for flat, body in zip(flats, bodies):
        check_guards(flat, "a gathered output tensor")
        assert torch.equal(body, full)


def test_peer_out_is_refused_where_no_kernel_serves_it():
    q, _ = gen((1, 4, 256, 128), "f32", 161, 1.0)
    out = torch.zeros((1, 4, 256, 128), device="cuda")
    other = torch.zeros_like(out)
    stream = torch.cuda.current_stream().cuda_stream
    h = N.Handle(device=0, qkv_dtype=N.F32, head_dim=128, num_q_heads=4, num_kv_heads=4)
    with pytest.raises(N.AidnError) as e:   # fp32 inputs run on the FFMA kernel
        h.launch(q=q.data_ptr(), k=q.data_ptr(), v=q.data_ptr(), out=out.data_ptr(), batch=1, seq_q=256, seq_kv=256,
                 stream=stream, peer_out=[other.data_ptr()])
    assert e.value.status == N.EUNSUPPORTED
    h.close()
    qb = q.to(torch.bfloat16)
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=4, num_kv_heads=4)
    with pytest.raises(N.AidnError) as e:   # a null entry
        h.launch(q=qb.data_ptr(), k=qb.data_ptr(), v=qb.data_ptr(), out=out.data_ptr(), batch=1, seq_q=256, seq_kv=256,
                 stream=stream, peer_out=[other.data_ptr(), 0])
    assert e.value.status == N.EINVAL
    h.close()


def test_prefill_sm100_head_shard_matches_full():
    """A head shard (multi-GPU partition) computes exactly the rows of the full call."""
    B, Hq, Hkv, S, D = 1, 8, 4, 384, 128
    q, _ = gen((B, Hq, S, D), "bf16", 81)
    k, _ = gen((B, Hkv, S, D), "bf16", 82)
    v, _ = gen((B, Hkv, S, D), "bf16", 83)
    full, _, _ = run_gpu(q, k, v, dtype="bf16", causal=True, path=N.PATH_PREFILL_SM100)
    out = torch.zeros_like(full)
    for hb in (0, 4):
        run_gpu(q, k, v, dtype="bf16", causal=True, path=N.PATH_PREFILL_SM100, head_begin=hb, head_count=4, out=out)
    assert torch.equal(out, full)


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("kind", ["keep_u8", "keep_f32", "bias", "bias_causal_lse", "softcap", "softcap_bias"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 256, 384, 128), (1, 3, 3, 200, 333, 64), (2, 2, 1, 130, 129, 128)])
def test_prefill_sm100_masks_bias_softcap(dtype, kind, shape):
    """Explicit masks on the tensor-core kernel: bool / float keep-masks with broadcast axes, additive bias
    (3-D batch-broadcast and 4-D) with top-left causal and LSE, logit softcap; aligned and ragged key counts."""
    B, Hq, Hkv, Sq, Sk, D = shape
    q, qf = gen((B, Hq, Sq, D), dtype, 91)
    k, kf = gen((B, Hkv, Sk, D), dtype, 92)
    v, vf = gen((B, Hkv, Sk, D), dtype, 93)
    rng = np.random.default_rng(17)
    kw_gpu, kw_ref = {}, {}
    if kind == "keep_u8":
        m = (rng.random((B, 1, Sq, Sk)) > 0.4).astype(np.uint8)       # broadcast over heads
        m[0, 0, 5, :] = 0                                              # a fully masked row
        kw_gpu = dict(mask=_t(m, torch.uint8), mask_kind=N.MASK_KEEP_U8)
        kw_ref = dict(mask=m, mask_kind=O.MASK_KEEP_U8)
    elif kind == "keep_f32":
        m = (rng.random((1, Hq, Sq, Sk)) > 0.5).astype(np.float32)    # broadcast over batch
        kw_gpu = dict(mask=_t(m), mask_kind=N.MASK_KEEP_F32)
        kw_ref = dict(mask=m, mask_kind=O.MASK_KEEP_F32)
    elif kind == "bias":
        m = rng.standard_normal((1, Hq, Sq, Sk)).astype(np.float32)   # [H,Sq,Sk] bias broadcast over batch
        kw_gpu = dict(mask=_t(m), mask_kind=N.MASK_ADD_F32)
        kw_ref = dict(mask=m, mask_kind=O.MASK_ADD_F32)
    elif kind == "bias_causal_lse":
        m = rng.standard_normal((B, Hq, Sq, Sk)).astype(np.float32)
        kw_gpu = dict(mask=_t(m), mask_kind=N.MASK_ADD_F32, causal=True, bottom_right=False)
        kw_ref = dict(mask=m, mask_kind=O.MASK_ADD_F32, causal=True, causal_offset=0)
    elif kind == "softcap":
        kw_gpu = dict(softcap=1.5, causal=True)
        kw_ref = dict(softcap=1.5, causal=True)
    else:
        m = rng.standard_normal((B, Hq, Sq, Sk)).astype(np.float32)
        kw_gpu = dict(softcap=2.0, mask=_t(m), mask_kind=N.MASK_ADD_F32)
        kw_ref = dict(softcap=2.0, mask=m, mask_kind=O.MASK_ADD_F32)
    out, lse, info = run_gpu(q, k, v, dtype=dtype, want_lse=True, path=N.PATH_PREFILL_SM100, **kw_gpu)
    assert info["path"] == N.PATH_PREFILL_SM100
    ref, rlse, _ = O.sdpa(qf, kf, vf, want_lse=True, **kw_ref)
    compare(out, ref, dtype, f"masked prefill {kind} {shape}")
    compare_lse(lse, rlse, dtype)


def test_prefill_sm100_bias_at_scale_matches_generic_kernel():
    """FlashAttention-style call with a full 4-D bias at B2 H8 S1024 D128: tensor-core kernel vs the fp32-arithmetic
    generic kernel (the oracle at this size is covered above on smaller shapes)."""
    B, H, S, D = 2, 8, 1024, 128
    q, _ = gen((B, H, S, D), "bf16", 95)
    k, _ = gen((B, H, S, D), "bf16", 96)
    v, _ = gen((B, H, S, D), "bf16", 97)
    bias = torch.randn((B, H, S, S), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5))
    a, la, ia = run_gpu(q, k, v, dtype="bf16", mask=bias, mask_kind=N.MASK_ADD_F32, causal=True, bottom_right=False,
                        want_lse=True)
    b_, lb, ib = run_gpu(q, k, v, dtype="bf16", mask=bias, mask_kind=N.MASK_ADD_F32, causal=True, bottom_right=False,
                         want_lse=True, path=N.PATH_GENERIC)
    assert ia["path"] == N.PATH_PREFILL_SM100 and ib["path"] == N.PATH_GENERIC
    assert float((a - b_).abs().max()) <= 2e-2 and float((a - b_).abs().mean()) <= 2e-3
    assert float((la - lb).abs().max()) <= 2e-2


def test_config2_llama_prefill_full_size():
    """BASELINE config 2: B4 H32 S2048 D128 causal bf16 -> fp32; full tensor against the oracle, on the inputs the
    benchmark times (generator streams of configuration 2)."""
    B, H, S, D = 4, 32, 2048, 128
    q, qf = gen_config(2, 0, (B, H, S, D), "bf16")
    k, kf = gen_config(2, 1, (B, H, S, D), "bf16")
    v, vf = gen_config(2, 2, (B, H, S, D), "bf16")
    out, _, info = run_gpu(q, k, v, dtype="bf16", causal=True)
    assert info["path"] == N.PATH_PREFILL_SM100
    compare(out, O.sdpa(qf, kf, vf, causal=True), "bf16", "config2")
    out2, _, _ = run_gpu(q, k, v, dtype="bf16", causal=True)
    assert torch.equal(out, out2), "prefill must be bit-reproducible"


def _sampled_rows(S, seed, every=16, extra=256):
    """First and last row of every `every`-th 128-row tile, plus `extra` seeded random rows: the rows next to every
    tile edge and inside the heavy-first schedule are the ones a scheduling or masking bug would hit."""
    tiles = np.arange(0, (S + 127) // 128, every)
    edge = np.concatenate([tiles * 128, np.minimum(tiles * 128 + 127, S - 1)])
    rnd = np.random.Generator(np.random.Philox(seed)).integers(0, S, extra)
    return np.unique(np.concatenate([edge, rnd, [S - 1]]))


def _check_sampled(out, qf, kf, vf, what, seed0):
    """Every (batch entry, KV group): the tile-edge rows for all heads of the group, the random rows for one head."""
    B, Hq, S, D = out.shape
    Hkv = kf.shape[1]
    group = Hq // Hkv
    got = out.float().cpu().numpy()
    worst = 0.0
    for b in range(B):
        for g in range(Hkv):
            rows = _sampled_rows(S, seed0 + 97 * b + g)
            edge = rows[(rows % 128 == 0) | (rows % 128 == 127)]
            for j in range(group):
                h = g * group + j
                sel = rows if j == (b + g) % group else edge
                ref = reference_rows(qf, kf, vf, b, h, sel)
                err = np.abs(got[b, h, sel] - ref)
                assert np.isfinite(got[b, h, sel]).all(), f"{what}: non-finite output at b{b} h{h}"
                assert err.max() <= TOL_16_MAX and err.mean() <= TOL_16_MEAN, f"{what} b{b} h{h}: max {err.max():.3e} mean {err.mean():.3e}"
                worst = max(worst, float(err.max()))
    return worst


def test_config3_gqa_prefill_full_size_sampled_rows_and_properties():
    """BASELINE config 3: B2 Hq32/Hkv8 S8192 D128 causal bf16.  The full tensor is 1.1 TFLOP on the CPU, so: the C++
    oracle on contiguous row blocks, a float64 reference on the first / last row of every 16th row tile and 256 random
    rows per KV group, and two size-independent properties on the whole output."""
    B, Hq, Hkv, S, D = 2, 32, 8, 8192, 128
    q, qf = gen_config(3, 0, (B, Hq, S, D), "bf16")
    k, kf = gen_config(3, 1, (B, Hkv, S, D), "bf16")
    v, vf = gen_config(3, 2, (B, Hkv, S, D), "bf16")
    out, _, info = run_gpu(q, k, v, dtype="bf16", causal=True)
    assert info["path"] == N.PATH_PREFILL_SM100
    for r0 in (0, 127, 4096 - 32, 8192 - 64):
        ref = oracle_rows(qf, kf, vf, r0, r0 + 64, causal=True, causal_offset=0)
        compare(out[:, :, r0:r0 + 64], ref, "bf16", f"config3 rows {r0}")
    _check_sampled(out, qf, kf, vf, "config3", 0x3000)
    # (a) softmax weights sum to one: with V == 1 every output element is 1
    ones = torch.ones_like(v)
    o1, _, _ = run_gpu(q, k, ones, dtype="bf16", causal=True)
    assert float((o1 - 1).abs().max()) <= 4e-3
    # (b) linearity in V: out(V) + out(V2) == out(V + V2) up to bf16 rounding of the summed V
    v2, _ = gen_config(3, 4, (B, Hkv, S, D), "bf16")
    vs = (v.float() + v2.float()).to(torch.bfloat16)
    o2, _, _ = run_gpu(q, k, v2, dtype="bf16", causal=True)
    os_, _, _ = run_gpu(q, k, vs, dtype="bf16", causal=True)
    assert float((out + o2 - os_).abs().max()) <= 2e-2


def test_config5_long_context_shard_sampled_rows():
    """BASELINE config 5, the shard one GPU owns: the 8 query heads of KV head 3 of B1 Hq64/Hkv8 S32768 D128 (only
    those heads are materialised; the generator keys them by their global head index, as the benchmark does)."""
    S, D = 32768, 128
    q, qf = gen_config(5, 0, (1, 8, S, D), "bf16", heads=list(range(24, 32)))
    k, kf = gen_config(5, 1, (1, 1, S, D), "bf16", heads=[3])
    v, vf = gen_config(5, 2, (1, 1, S, D), "bf16", heads=[3])
    out, _, info = run_gpu(q, k, v, dtype="bf16", causal=True)
    assert info["path"] == N.PATH_PREFILL_SM100
    for r0 in (0, 16384 - 16, 32768 - 32):
        ref = oracle_rows(qf, kf, vf, r0, r0 + 32, causal=True, causal_offset=0)
        compare(out[:, :, r0:r0 + 32], ref, "bf16", f"config5 rows {r0}")
    _check_sampled(out, qf, kf, vf, "config5 shard", 0x5000)


def test_prefill_bounded_wait_expires_cleanly():
    """Failure detection without a fault: a test hook makes the producer withhold the Q tiles, so the UMMA warp's
    bounded wait (20 ms in this mode) runs out.  The kernel must unwind (every role leaves its loop, TMEM is freed,
    the scheduler counters are reset), poll() must report AIDN_ETIMEOUT, and the very next launch on the same handle
    must be correct."""
    q, qf = gen((1, 4, 512, 128), "bf16", 201)
    k, kf = gen((1, 2, 512, 128), "bf16", 202)
    v, vf = gen((1, 2, 512, 128), "bf16", 203)
    out = torch.zeros((1, 4, 512, 128), device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=4, num_kv_heads=2, causal=True,
                 path=N.PATH_PREFILL_SM100)
    stream = torch.cuda.current_stream().cuda_stream
    launch = lambda: h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=1, seq_q=512,
                              seq_kv=512, stream=stream)
    h.debug_set(None, 3)
    launch()
    with pytest.raises(N.AidnError) as e:
        h.poll(stream)
    assert e.value.status == N.ETIMEOUT
    h.debug_set(None, 0)
    launch()
    h.poll(stream)
    compare(out, O.sdpa(qf, kf, vf, causal=True), "bf16", "launch after a timed-out launch")
    h.close()


# ------------------------------------------------------------------------------------------------ casts, errors
def test_cast_kernels_bit_exact(golden):
    """BFloat16.cs:65-84 bit for bit, NaN payloads included; round trip through fp32 is lossless."""
    x = torch.from_numpy(golden["bf16_in_bits"].view(np.int32).copy()).cuda()
    dst = torch.zeros(x.numel(), dtype=torch.int16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    N.cast("f32_to_bf16", x.data_ptr(), dst.data_ptr(), x.numel(), s)
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy().view(np.uint16), golden["bf16_out_bits"])
    big = torch.randn(1 << 20, device="cuda") * 3
    b16 = torch.empty(1 << 20, dtype=torch.bfloat16, device="cuda")
    N.cast("f32_to_bf16", big.data_ptr(), b16.data_ptr(), big.numel(), s)
    back = torch.empty_like(big)
    N.cast("bf16_to_f32", b16.data_ptr(), back.data_ptr(), big.numel(), s)
    torch.cuda.synchronize()
    assert np.array_equal(b16.view(torch.int16).cpu().numpy().view(np.uint16), O.f32_to_bf16_bits(big.cpu().numpy()))
    assert torch.equal(back, b16.float())
    h16 = torch.empty(1 << 20, dtype=torch.float16, device="cuda")
    N.cast("f32_to_f16", big.data_ptr(), h16.data_ptr(), big.numel(), s)
    torch.cuda.synchronize()
    assert torch.equal(h16, big.half())


def test_error_codes_no_fallback():
    """Bad requests are status codes with a message; nothing is silently rerouted to another path."""
    with pytest.raises(N.AidnError) as e:
        N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=6, num_kv_heads=4)
    assert e.value.status == N.EINVAL
    q, _ = gen((1, 2, 16, 72), "bf16", 1)
    with pytest.raises(N.AidnError) as e:
        run_gpu(q, q, q, dtype="bf16", path=N.PATH_PREFILL_SM100)      # head_dim 72 is not a tensor-core shape
    assert e.value.status == N.EUNSUPPORTED
    with pytest.raises(N.AidnError) as e:
        run_gpu(q, q, q, dtype="bf16", path=N.PATH_DECODE)             # seq_q != 1
    assert e.value.status == N.EUNSUPPORTED
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=128, num_q_heads=2)
    with pytest.raises(N.AidnError) as e:
        h.launch(q=0, k=0, v=0, out=0, batch=1, seq_q=1, seq_kv=1, stream=0)
    assert e.value.status == N.EINVAL
    qd, _ = gen((4, 2, 1, 128), "bf16", 2)
    kd, _ = gen((4, 2, 2048, 128), "bf16", 3)
    o = torch.empty((4, 2, 1, 128), device="cuda")
    with pytest.raises(N.AidnError) as e:   # decode needs scratch and none was given
        h.launch(q=qd.data_ptr(), k=kd.data_ptr(), v=kd.data_ptr(), out=o.data_ptr(), batch=4, seq_q=1, seq_kv=2048,
                 stream=torch.cuda.current_stream().cuda_stream)
    assert e.value.status == N.EWORKSPACE
    h.close()

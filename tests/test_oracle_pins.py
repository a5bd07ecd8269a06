"""Pins the CPU oracle (oracle/sdpa_ref.cpp) before anything else trusts it.

Every case replays a test of the reference project (file:line in each docstring, paths relative to
tests/AiDotNet.Tensors.Tests/) against the stored float64 fixtures and closed forms.
"""
import numpy as np
import pytest

from oracle import sdpa_oracle as O


def test_softcap_closed_form(golden):
    """Engines/BatchMatMulAndAttentionTests.cs:287-317 — Q.K^T = [10,-10], cap 2 (4 decimals there)."""
    out, _, w = O.sdpa(golden["softcap_q"], golden["softcap_k"], golden["softcap_v"], scale=1.0, softcap=2.0,
                       want_weights=True)
    assert np.allclose(w.ravel(), golden["softcap_w"], atol=1e-6)
    assert np.allclose(out.ravel(), golden["softcap_out"], atol=1e-5)
    _, _, wp = O.sdpa(golden["softcap_q"], golden["softcap_k"], golden["softcap_v"], scale=1.0, want_weights=True)
    assert wp.ravel()[1] < 1e-3 and w.ravel()[1] > 100 * wp.ravel()[1]


def test_cross_attention_sequences(golden):
    """Engines/DirectGpu/GpuCpuConsistencyTests.cs:895-960 — Sq=2, Sk=3, D=3, scale 0.75 (2e-5 there)."""
    out, _, w = O.sdpa(golden["cross_q"], golden["cross_k"], golden["cross_v"], scale=0.75, want_weights=True)
    assert np.abs(out - golden["cross_out"]).max() <= 2e-6
    assert np.abs(w - golden["cross_w"]).max() <= 2e-6


def test_logit_softcap_sequences(golden):
    """Engines/DirectGpu/GpuCpuConsistencyTests.cs:962-1003 — scale 1.5, softcap 2."""
    out, _, w = O.sdpa(golden["capcross_q"], golden["capcross_k"], golden["capcross_v"], scale=1.5, softcap=2.0,
                       want_weights=True)
    assert np.abs(out - golden["capcross_out"]).max() <= 2e-6
    assert np.abs(w - golden["capcross_w"]).max() <= 2e-6


def test_full_boolean_mask(golden):
    """Engines/DirectGpu/GpuCpuConsistencyTests.cs:1005-1061 — full [B,H,Sq,Sk] bool mask, true = attend."""
    m = golden["boolmask_mask"]
    out, _, w = O.sdpa(golden["cross_q"], golden["cross_k"], golden["cross_v"], scale=0.75, mask=m,
                       mask_kind=O.MASK_KEEP_U8, want_weights=True)
    assert np.abs(out - golden["boolmask_out"]).max() <= 2e-6
    assert np.abs(w - golden["boolmask_w"]).max() <= 2e-6
    # the float upload of the same mask (false -> 0.0f) must mean the same thing
    out2 = O.sdpa(golden["cross_q"], golden["cross_k"], golden["cross_v"], scale=0.75, mask=m.astype(np.float32),
                  mask_kind=O.MASK_KEEP_F32)
    assert np.array_equal(out, out2)


@pytest.mark.parametrize("mb,mh", [(1, 1), (2, 1), (1, 3), (2, 3)])
def test_broadcast_mask(golden, mb, mh):
    """Engines/SdpaMaskBroadcastTests.cs:61-114 — [1,1,S,S], [B,1,S,S], [1,H,S,S] masks == materialised mask."""
    q, k, v = golden["bcast_q"], golden["bcast_k"], golden["bcast_v"]
    S = q.shape[2]
    mask = np.broadcast_to(np.tril(np.ones((S, S), np.uint8)), (mb, mh, S, S)).copy()
    out = O.sdpa(q, k, v, mask=mask, mask_kind=O.MASK_KEEP_U8)
    assert np.abs(out - golden["bcast_out"]).max() <= 1e-5
    # the causal flag (bottom-right, Sq == Sk) is the same plane
    assert np.array_equal(out, O.sdpa(q, k, v, causal=True))
    # non-vacuity (SdpaMaskBroadcastTests.cs:124-143)
    assert np.abs(O.sdpa(q, k, v) - golden["bcast_out_nomask"]).max() <= 1e-5
    assert np.abs(out - golden["bcast_out_nomask"]).max() > 1e-3


@pytest.mark.parametrize("causal", [False, True])
def test_gqa_reference(golden, causal):
    """Engines/DirectGpu/RopeGqaOpenClTests.cs:200-279 — Hq 6, Hkv 2, kv = h / group (1e-4 there)."""
    out = O.sdpa(golden["gqa_q"], golden["gqa_k"], golden["gqa_v"], causal=causal)
    want = golden["gqa_out_causal"] if causal else golden["gqa_out_plain"]
    assert np.abs(out - want).max() <= 1e-5


def test_decode_shape_list(golden):
    """Engines/DirectGpu/FlashDecodeCudaTests.cs:43-126 — K/V stored [seqLen, kvHeads, D]; tol 2e-3 + 2e-3|e|."""
    for n, (h, hk, d, L) in enumerate(golden["decode_shapes"]):
        q = golden[f"decode{n}_q"][None, :, None, :]
        k = golden[f"decode{n}_k"].transpose(1, 0, 2)[None]   # strided view, unit inner stride
        v = golden[f"decode{n}_v"].transpose(1, 0, 2)[None]
        out = O.sdpa(q, k, v)[0, :, 0, :]
        assert np.abs(out - golden[f"decode{n}_out"]).max() <= 1e-5


def test_flash_attention_bias_and_lse(golden):
    """Engines/FlashAttentionBiasTests.cs:31-274 — bias added after scale, 3-D bias broadcasts over batch,
    top-left causal, stats = max + log(sum)  (CpuEngine.cs:29226-29263)."""
    q, k, v = golden["bias_q"], golden["bias_k"], golden["bias_v"]
    out, lse, _ = O.sdpa(q, k, v, mask=golden["bias3"][None], mask_kind=O.MASK_ADD_F32, want_lse=True)
    assert np.abs(out - golden["bias3_out"]).max() <= 2e-5
    assert np.abs(lse - golden["bias3_lse"]).max() <= 2e-5
    out, lse, _ = O.sdpa(q, k, v, mask=golden["bias4"], mask_kind=O.MASK_ADD_F32, causal=True, causal_offset=0,
                         want_lse=True)
    assert np.abs(out - golden["bias4c_out"]).max() <= 2e-5
    assert np.abs(lse - golden["bias4c_lse"]).max() <= 2e-5


def test_fully_masked_rows_give_zero_and_minus_inf():
    """CpuEngine.cs:27822-27827 and 29244-29250."""
    rng = np.random.default_rng(3)
    q, k, v = (rng.standard_normal((1, 2, 4, 8)).astype(np.float32) for _ in range(3))
    mask = np.ones((1, 1, 4, 4), np.uint8)
    mask[0, 0, 2, :] = 0
    out, lse, w = O.sdpa(q, k, v, mask=mask, mask_kind=O.MASK_KEEP_U8, want_lse=True, want_weights=True)
    assert np.all(out[:, :, 2, :] == 0) and np.all(w[:, :, 2, :] == 0) and np.all(np.isneginf(lse[:, :, 2]))
    assert np.all(np.isfinite(lse[:, :, [0, 1, 3]]))
    # padding mask: kv_len = 0 masks every key of that batch entry
    out = O.sdpa(q, k, v, kv_len=np.array([0], np.int32))
    assert np.all(out == 0)


def test_bottom_right_vs_top_left_causal():
    """SDPA/GQA entry points keep k <= q + (Sk - Sq) (CpuEngine.cs:27333-27340); FlashAttention keeps k <= q."""
    rng = np.random.default_rng(5)
    q = rng.standard_normal((1, 1, 3, 8)).astype(np.float32)
    k = rng.standard_normal((1, 1, 7, 8)).astype(np.float32)
    v = rng.standard_normal((1, 1, 7, 8)).astype(np.float32)
    br = np.array([[j <= i + 4 for j in range(7)] for i in range(3)], np.uint8)[None, None]
    tl = np.array([[j <= i for j in range(7)] for i in range(3)], np.uint8)[None, None]
    assert np.array_equal(O.sdpa(q, k, v, causal=True), O.sdpa(q, k, v, mask=br, mask_kind=O.MASK_KEEP_U8))
    assert np.array_equal(O.sdpa(q, k, v, causal=True, causal_offset=0), O.sdpa(q, k, v, mask=tl, mask_kind=O.MASK_KEEP_U8))


def test_f64_mode_and_faithful_mode_agree():
    rng = np.random.default_rng(11)
    q = rng.standard_normal((2, 4, 70, 32)).astype(np.float32)
    k = rng.standard_normal((2, 2, 130, 32)).astype(np.float32)
    v = rng.standard_normal((2, 2, 130, 32)).astype(np.float32)
    kv = np.array([130, 57], np.int32)
    a = O.sdpa(q, k, v, causal=True, kv_len=kv)
    b = O.sdpa(q, k, v, causal=True, kv_len=kv, faithful=True)
    c = O.sdpa(q, k, v, causal=True, kv_len=kv, f64=True)
    assert np.abs(a - b).max() <= 1e-6     # trimming masked columns does not change a row's arithmetic
    assert np.abs(a - c).max() <= 5e-6


def test_bf16_rounding_vectors(golden):
    """NumericOperations/BFloat16.cs:65-84 — RNE, NaN keeps its payload top bits and gains the quiet bit."""
    x = golden["bf16_in_bits"].view(np.float32)
    assert np.array_equal(O.f32_to_bf16_bits(x), golden["bf16_out_bits"])
    back = O.bf16_bits_to_f32(golden["bf16_out_bits"])
    assert np.array_equal(back.view(np.uint32), golden["bf16_out_bits"].astype(np.uint32) << 16)


# ---- paged K/V ----------------------------------------------------------------------------------------------
def _paged_case(rng, heads, kv_heads, head_dim, block_size, key_len, n_q):
    n_logical = (key_len + block_size - 1) // block_size
    max_blocks = n_logical + 5                      # spare blocks, as the reference's tests allocate
    kc = rng.uniform(-1, 1, (max_blocks, block_size, kv_heads, head_dim)).astype(np.float32)
    vc = rng.uniform(-1, 1, (max_blocks, block_size, kv_heads, head_dim)).astype(np.float32)
    q = rng.uniform(-1, 1, (n_q, heads, head_dim)).astype(np.float32)
    bt = rng.permutation(max_blocks)[:n_logical].astype(np.int32)   # a scattered, non-monotonic table
    return q, kc, vc, bt


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,seq_len", [
    (4, 4, 64, 16, 40), (2, 2, 128, 8, 20), (8, 8, 32, 32, 100),      # PagedAttentionCudaTests.cs:44-46
    (8, 2, 64, 16, 40), (4, 1, 128, 8, 33)])                           # grouped-query shapes
def test_paged_decode_materialised_equals_kernel_restatement(heads, kv_heads, head_dim, block_size, seq_len):
    """materialize + sdpa (the form the GPU parity tests use) against the line-by-line restatement of
    paged_attention_decode{,_gqa}, within the reference tests' own tolerance 2e-3 + 2e-3|e| (…CudaTests.cs:118)."""
    rng = np.random.default_rng(0xA77 + heads + seq_len)
    q, kc, vc, bt = _paged_case(rng, heads, kv_heads, head_dim, block_size, seq_len, 1)
    scale = 1.0 / np.sqrt(head_dim)
    want = O.paged_attention_rows(q, kc, vc, bt, heads, kv_heads, head_dim, block_size, 1, 0, scale, decode_len=seq_len)
    got = O.paged_sdpa(q.transpose(1, 0, 2)[None], kc, vc, bt[None], block_size=block_size, seq_kv=seq_len, scale=scale)
    got = got[0].transpose(1, 0, 2)
    assert np.all(np.abs(got - want) <= 1e-5 + 1e-5 * np.abs(want))


@pytest.mark.parametrize("heads,kv_heads,head_dim,block_size,num_queries,start_pos", [
    (4, 4, 64, 16, 8, 0), (2, 2, 128, 8, 12, 5), (8, 8, 32, 32, 20, 40),   # PagedAttentionCudaTests.cs:125-127
    (8, 2, 64, 16, 8, 3)])
def test_paged_prefill_materialised_equals_kernel_restatement(heads, kv_heads, head_dim, block_size, num_queries,
                                                              start_pos):
    """Query qi sees keys 0..start_pos+qi: causal with causal_offset = start_pos over start_pos+num_queries keys."""
    rng = np.random.default_rng(0xB99 + heads + num_queries + start_pos)
    q, kc, vc, bt = _paged_case(rng, heads, kv_heads, head_dim, block_size, start_pos + num_queries, num_queries)
    scale = 1.0 / np.sqrt(head_dim)
    want = O.paged_attention_rows(q, kc, vc, bt, heads, kv_heads, head_dim, block_size, num_queries, start_pos, scale)
    got = O.paged_sdpa(q.transpose(1, 0, 2)[None], kc, vc, bt[None], block_size=block_size,
                       seq_kv=start_pos + num_queries, causal=True, causal_offset=start_pos, scale=scale)
    got = got[0].transpose(1, 0, 2)
    assert np.all(np.abs(got - want) <= 1e-5 + 1e-5 * np.abs(want))


def test_materialize_respects_kv_len_and_unused_entries():
    """Entries of the table beyond a sequence's length are never read (a cache leaves them unset)."""
    rng = np.random.default_rng(3)
    kc = rng.standard_normal((6, 4, 2, 8)).astype(np.float32)
    bt = np.array([[2, 5, -7], [1, 0, 3]], np.int32)
    out = O.materialize(kc, bt, 4, 12, kv_len=np.array([7, 12], np.int32))
    assert np.array_equal(out[0, :, :4], kc[2].transpose(1, 0, 2)) and np.array_equal(out[0, :, 4:7], kc[5, :3].transpose(1, 0, 2))
    assert np.all(out[0, :, 7:] == 0)
    assert np.array_equal(out[1, :, 8:12], kc[3].transpose(1, 0, 2))


# ---- RoPE and the packed Q/K/V projection ---------------------------------------------------------------------
def _rope_cache(max_seq, head_dim, theta=10000.0):
    """BuildRopeCache of the reference's tests (DirectGpu/RopeGqaOpenClTests.cs:51-67)."""
    half = head_dim // 2
    pos = np.arange(max_seq, dtype=np.float64)[:, None]
    freq = 1.0 / np.power(theta, 2.0 * np.arange(half) / head_dim)[None, :]
    return np.cos(pos * freq).astype(np.float32), np.sin(pos * freq).astype(np.float32)


@pytest.mark.parametrize("start", [0, 5])
def test_rope_interleaved_against_the_reference_loop(start):
    """RopeInterleaved_MatchesCpuReference (DirectGpu/RopeGqaOpenClTests.cs:92-117): heads 3, seqLen 6, headDim 8,
    maxSeq 32, expected values from the scalar RopeReference loop (:69-90), restated here element by element."""
    heads, seq_len, head_dim, max_seq = 3, 6, 8, 32
    rows = heads * seq_len
    rng = np.random.default_rng(7)
    x = rng.uniform(-1, 1, (rows, head_dim)).astype(np.float32)
    cos, sin = _rope_cache(max_seq, head_dim)
    want = np.zeros_like(x)
    for row in range(rows):
        pos = start + row % seq_len
        for i in range(head_dim // 2):
            c, s = cos[pos, i], sin[pos, i]
            xe, xo = x[row, 2 * i], x[row, 2 * i + 1]
            want[row, 2 * i] = np.float32(xe * c) - np.float32(xo * s)
            want[row, 2 * i + 1] = np.float32(xe * s) + np.float32(xo * c)
    got = O.rope_interleaved(x, cos, sin, seq_len, start)
    assert np.abs(got - want).max() <= 1e-6
    assert np.abs(np.linalg.norm(got, axis=1) - np.linalg.norm(x, axis=1)).max() <= 1e-5   # a rotation keeps norms


@pytest.mark.parametrize("heads,capacity,position", [(4, 16, 0), (8, 64, 17), (16, 128, 127)])
def test_qkv_rope_cache_composition(heads, capacity, position):
    """The shapes of DriverOnlyQkvRopeCacheD64_MatchesOracle (DirectGpu/DirectPtxWmmaTests.cs:2110-2113): head_dim 64,
    cache [capacity, heads, 64].  The oracle must equal the reference's fallback composition written out step by step
    (MatMulTransposed, BiasAdd, RopeInterleaved over 2*heads rows, three copies; CudaBackend.cs:8428-8438)."""
    D, model = 64, heads * 64
    rng = np.random.default_rng(900 + heads)
    x = rng.uniform(-1, 1, (1, model)).astype(np.float32)
    w = (rng.uniform(-1, 1, (3 * model, model)) / np.sqrt(model)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 3 * model).astype(np.float32)
    cos, sin = _rope_cache(capacity, D)
    projected = (x.astype(np.float64) @ w.astype(np.float64).T).astype(np.float32)[0]
    biased = projected + b
    rotated = O.rope_interleaved(biased[:2 * model].reshape(2 * heads, D), cos, sin, 1, position).reshape(-1)
    kc = np.zeros((capacity, model), np.float32)
    vc = np.zeros((capacity, model), np.float32)
    q = O.qkv_rope_cache(x, w, b, cos, sin, heads=heads, kv_heads=heads, head_dim=D, positions=[position],
                         cache_rows=[position], key_cache=kc, value_cache=vc)
    assert np.abs(q[0] - rotated[:model]).max() <= 1e-6
    assert np.abs(kc[position] - rotated[model:]).max() <= 1e-6
    assert np.abs(vc[position] - biased[2 * model:]).max() <= 1e-6
    assert not kc[np.arange(capacity) != position].any()


# ---- backward ----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("causal,gqa", [(False, False), (True, False), (True, True)])
def test_backward_oracle_against_finite_differences_of_the_forward(causal, gqa):
    """The backward restatement is pinned on the forward oracle itself: central differences of
    L = sum(dO * sdpa(Q, K, V)) in float64 accumulation must reproduce dQ, dK, dV (top-left causal as
    FlashAttentionBackward uses, with a bias, a padded batch entry and grouped-query heads)."""
    rng = np.random.default_rng(21 + causal + 2 * gqa)
    B, Hq, Hkv, Sq, Sk, D = 2, 4, (2 if gqa else 4), 5, 7, 8
    q = rng.standard_normal((B, Hq, Sq, D)).astype(np.float32) * 0.5
    k = rng.standard_normal((B, Hkv, Sk, D)).astype(np.float32) * 0.5
    v = rng.standard_normal((B, Hkv, Sk, D)).astype(np.float32) * 0.5
    dout = rng.standard_normal((B, Hq, Sq, D)).astype(np.float32)
    bias = rng.standard_normal((1, Hq, Sq, Sk)).astype(np.float32) * 0.3
    kv_len = np.array([Sk, 4], np.int32)
    kw = dict(scale=0.3, causal=causal, causal_offset=0, kv_len=kv_len)
    dq, dk, dv, o, lse = O.sdpa_backward(q, k, v, dout, bias=bias, **kw)
    fwd = lambda q_, k_, v_: O.sdpa(q_, k_, v_, mask=bias, mask_kind=O.MASK_ADD_F32, f64=True, want_lse=True, **kw)
    o_ref, lse_ref, _ = fwd(q, k, v)
    assert np.abs(o - o_ref).max() <= 2e-6 and np.abs(lse - lse_ref)[np.isfinite(lse_ref)].max() <= 2e-6
    loss = lambda q_, k_, v_: float((dout.astype(np.float64) * fwd(q_, k_, v_)[0].astype(np.float64)).sum())
    eps = 1e-2
    for name, x, grad in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        for _ in range(6):
            idx = tuple(rng.integers(0, n) for n in x.shape)
            xp, xm = x.copy(), x.copy()
            xp[idx] += eps
            xm[idx] -= eps
            args_p = {"q": (xp, k, v), "k": (q, xp, v), "v": (q, k, xp)}[name]
            args_m = {"q": (xm, k, v), "k": (q, xm, v), "v": (q, k, xm)}[name]
            fd = (loss(*args_p) - loss(*args_m)) / (2 * eps)
            assert abs(fd - grad[idx]) <= 2e-3 + 2e-3 * abs(fd), (name, idx, fd, grad[idx])


@pytest.mark.parametrize("batch,seq,d_model,heads", [(3, 5, 12, 3), (2, 7, 24, 4), (1, 100, 32, 4), (4, 13, 48, 6),
                                                      (5, 3, 8, 2), (2, 6, 6, 3), (3, 9, 30, 5), (1, 1, 16, 4)])
@pytest.mark.parametrize("masked", ["none", "causal", "broadcast"])
def test_mha_forward_matches_the_decomposed_chain(batch, seq, d_model, heads, masked):
    """Engines/MultiHeadAttentionForwardTests.cs:101-124, 126-162, 164-203, 288-313 — the fused call equals the chain
    Q/K/V MatMul -> split heads -> ScaledDotProductAttention -> merge heads -> output MatMul (1e-4 there), with no
    mask, a causal keep-mask and a [1,1,S,S] mask broadcast over batch and heads; same shapes as the reference's
    theory.  The chain is rebuilt here on the pinned attention oracle."""
    rng = np.random.default_rng(batch * 1000 + seq * 10 + heads)
    x = rng.standard_normal((batch, seq, d_model)).astype(np.float32)
    ws = [(rng.standard_normal((d_model, d_model)) / np.sqrt(d_model)).astype(np.float32) for _ in range(4)]
    mask = None
    if masked == "causal":
        mask = np.broadcast_to(np.tril(np.ones((seq, seq), bool)), (batch, heads, seq, seq)).copy()
    elif masked == "broadcast":
        mask = np.tril(np.ones((seq, seq), bool))[None, None]
    fused = O.mha_forward(x, *ws, heads, mask=mask)
    d = d_model // heads
    split = lambda t: np.ascontiguousarray(t.reshape(batch, seq, heads, d).transpose(0, 2, 1, 3))
    q, k, v = (split(x @ w) for w in ws[:3])
    attn = O.sdpa(q, k, v, mask=mask, f64=True)
    chain = attn.transpose(0, 2, 1, 3).reshape(batch, seq, d_model) @ ws[3]
    assert fused.shape == (batch, seq, d_model)
    assert np.abs(fused - chain).max() <= 1e-4
    if masked == "causal" and seq > 1:
        assert np.abs(fused - O.mha_forward(x, *ws, heads)).max() > 1e-4   # the mask changes the result (:154-161)


def test_mha_forward_fully_masked_row_gives_zero_attention():
    """CpuEngine.MultiHeadAttention.cs:481-485 — a query row with no visible key contributes zeros."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 4, 8)).astype(np.float32)
    ws = [rng.standard_normal((8, 8)).astype(np.float32) for _ in range(4)]
    mask = np.ones((1, 1, 4, 4), bool)
    mask[0, 0, 2, :] = False
    out = O.mha_forward(x, *ws, 2, mask=mask)
    assert np.all(out[0, 2] == 0) and np.abs(out[0, 1]).max() > 0

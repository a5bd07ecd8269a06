"""GPU parity of the decode-step front end (aidn_qkv_rope_cache, aidn_rope_interleaved) against the oracle's
restatement of the reference composition (CudaBackend.cs:8389-8439; rope_interleaved, CudaAttentionKernels.cs:1023-1050),
and the chain the fusion exists for: tokens projected and written into a 16-bit paged pool, then decoded from it."""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O

from tests._harness import AIDN_DT, TORCH_DT

pytestmark = pytest.mark.gpu


def _rope_tables(max_pos, head_dim, rng):
    ang = rng.uniform(0, 2 * np.pi, (max_pos, head_dim // 2)).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def _run(x, w, b, cos, sin, *, heads, kv_heads, head_dim, capacity, position=0, positions=None, cache_rows=None,
         weight_dtype="f32", query_dtype="f32", cache_dtype="f32", kc=None, vc=None):
    dev = "cuda"
    tokens = x.shape[0]
    xd = torch.from_numpy(x).to(dev)
    wd = torch.from_numpy(w).to(dev).to(TORCH_DT[weight_dtype])
    bd = torch.from_numpy(b).to(dev) if b is not None else None
    cd, sd = torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev)
    q = torch.full((tokens, heads * head_dim), float("nan"), dtype=TORCH_DT[query_dtype], device=dev)
    kc = torch.zeros((capacity, kv_heads * head_dim), dtype=TORCH_DT[cache_dtype], device=dev) if kc is None else kc
    vc = torch.zeros((capacity, kv_heads * head_dim), dtype=TORCH_DT[cache_dtype], device=dev) if vc is None else vc
    pd = torch.from_numpy(np.asarray(positions, np.int32)).to(dev) if positions is not None else None
    rd = torch.from_numpy(np.asarray(cache_rows, np.int32)).to(dev) if cache_rows is not None else None
    N.qkv_rope_cache(input=xd.data_ptr(), weights=wd.data_ptr(), bias=bd.data_ptr() if bd is not None else None,
                     cosine=cd.data_ptr(), sine=sd.data_ptr(), query=q.data_ptr(), key_cache=kc.data_ptr(),
                     value_cache=vc.data_ptr(), tokens=tokens, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                     position=position, positions=pd.data_ptr() if pd is not None else None,
                     cache_rows=rd.data_ptr() if rd is not None else None, weight_dtype=AIDN_DT[weight_dtype],
                     query_dtype=AIDN_DT[query_dtype], cache_dtype=AIDN_DT[cache_dtype], cache_capacity=capacity,
                     max_position=cos.shape[0], stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return q, kc, vc


@pytest.mark.parametrize("heads,capacity,position", [(4, 16, 0), (8, 64, 17), (16, 128, 127), (32, 64, 63)])
def test_single_token_d64_reference_contract(heads, capacity, position):
    """The reference's contract and its test shapes (DirectGpu/DirectPtxWmmaTests.cs:2110-2113, tolerance 2e-5 at
    :2307-2309): one fp32 token, head_dim 64, cache [capacity, heads, 64], packed bias, `position` both the RoPE
    position and the cache row; the other cache rows stay untouched."""
    rng = np.random.default_rng(100 + heads)
    D, model = 64, heads * 64
    x = rng.uniform(-1, 1, (1, model)).astype(np.float32)
    w = (rng.uniform(-1, 1, (3 * model, model)) / np.sqrt(model)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 3 * model).astype(np.float32)
    cos, sin = _rope_tables(capacity, D, rng)
    kref = np.full((capacity, model), 7.0, np.float32)
    vref = np.full((capacity, model), -3.0, np.float32)
    qref = O.qkv_rope_cache(x, w, b, cos, sin, heads=heads, kv_heads=heads, head_dim=D, positions=[position],
                            cache_rows=[position], key_cache=kref, value_cache=vref)
    kc = torch.full((capacity, model), 7.0, device="cuda")
    vc = torch.full((capacity, model), -3.0, device="cuda")
    q, kc, vc = _run(x, w, b, cos, sin, heads=heads, kv_heads=heads, head_dim=D, capacity=capacity, position=position,
                     kc=kc, vc=vc)
    for got, want in ((q, qref), (kc, kref), (vc, vref)):
        assert np.abs(got.cpu().numpy() - want).max() <= 2e-5
    untouched = np.arange(capacity) != position
    assert np.array_equal(kc.cpu().numpy()[untouched], kref[untouched])


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 7, 8, 11])
@pytest.mark.parametrize("weight_dtype,cache_dtype", [("f32", "f32"), ("bf16", "bf16"), ("bf16", "f16")])
def test_batched_tokens_gqa_positions_and_rows(tokens, weight_dtype, cache_dtype):
    """A decode batch: one token per sequence, each with its own position and its own cache row (as a paged pool hands
    them out), grouped-query projection, head_dim 128, bf16 weights and a 16-bit cache."""
    rng = np.random.default_rng(200 + tokens)
    heads, kv_heads, D, capacity, max_pos = 8, 2, 128, 40, 96
    model = heads * D
    x = rng.uniform(-1, 1, (tokens, model)).astype(np.float32)
    w = (rng.uniform(-1, 1, ((heads + 2 * kv_heads) * D, model)) / np.sqrt(model)).astype(np.float32)
    if weight_dtype == "bf16":
        w = torch.from_numpy(w).to(torch.bfloat16).to(torch.float32).numpy()   # the oracle sees the rounded weights
    b = rng.uniform(-0.1, 0.1, (heads + 2 * kv_heads) * D).astype(np.float32)
    cos, sin = _rope_tables(max_pos, D, rng)
    positions = rng.integers(0, max_pos, tokens).astype(np.int32)
    rows = rng.permutation(capacity)[:tokens].astype(np.int32)
    kref = np.zeros((capacity, kv_heads * D), np.float32)
    vref = np.zeros((capacity, kv_heads * D), np.float32)
    qref = O.qkv_rope_cache(x, w, b, cos, sin, heads=heads, kv_heads=kv_heads, head_dim=D, positions=positions,
                            cache_rows=rows, key_cache=kref, value_cache=vref)
    q, kc, vc = _run(x, w, b, cos, sin, heads=heads, kv_heads=kv_heads, head_dim=D, capacity=capacity,
                     positions=positions, cache_rows=rows, weight_dtype=weight_dtype, cache_dtype=cache_dtype)
    assert np.abs(q.cpu().numpy() - qref).max() <= 3e-5
    tol = 3e-5 if cache_dtype == "f32" else 2e-2     # one 16-bit rounding of values of magnitude <= ~2
    assert np.abs(kc.float().cpu().numpy() - kref).max() <= tol
    assert np.abs(vc.float().cpu().numpy() - vref).max() <= tol


def test_row_outside_the_cache_is_not_written():
    rng = np.random.default_rng(5)
    heads, D, capacity = 2, 64, 8
    model = heads * D
    x = rng.uniform(-1, 1, (2, model)).astype(np.float32)
    w = rng.uniform(-1, 1, (3 * model, model)).astype(np.float32)
    cos, sin = _rope_tables(16, D, rng)
    q, kc, vc = _run(x, w, None, cos, sin, heads=heads, kv_heads=heads, head_dim=D, capacity=capacity,
                     positions=[3, 5], cache_rows=[2, 99])
    assert torch.count_nonzero(kc[2]) > 0 and torch.count_nonzero(kc).item() == torch.count_nonzero(kc[2]).item()
    assert torch.isfinite(q).all()


def test_argument_errors():
    z = torch.zeros(64 * 192, device="cuda")
    kw = dict(input=z.data_ptr(), weights=z.data_ptr(), bias=None, cosine=z.data_ptr(), sine=z.data_ptr(),
              query=z.data_ptr(), key_cache=z.data_ptr(), value_cache=z.data_ptr(), tokens=1, heads=1, kv_heads=1,
              head_dim=64, cache_capacity=4, max_position=4, stream=0)
    for bad in (dict(position=4), dict(position=-1), dict(heads=0), dict(kv_heads=3), dict(head_dim=63),
                dict(tokens=0), dict(weight_dtype=N.F16)):
        with pytest.raises(N.AidnError) as e:
            N.qkv_rope_cache(**{**kw, **bad})
        assert e.value.status == N.EINVAL, bad


@pytest.mark.parametrize("rows,head_dim,seq_len,start", [(6, 64, 3, 5), (32, 128, 1, 9), (10, 8, 10, 0)])
def test_rope_interleaved(rows, head_dim, seq_len, start):
    rng = np.random.default_rng(rows)
    x = rng.uniform(-1, 1, (rows, head_dim)).astype(np.float32)
    cos, sin = _rope_tables(start + seq_len, head_dim, rng)
    want = O.rope_interleaved(x, cos, sin, seq_len, start)
    xd, cd, sd = (torch.from_numpy(a).cuda() for a in (x, cos, sin))
    out = torch.empty_like(xd)
    N.rope_interleaved(xd.data_ptr(), cd.data_ptr(), sd.data_ptr(), out.data_ptr(), rows, head_dim, seq_len, start,
                       torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-6


def test_projected_tokens_feed_the_paged_decode():
    """The chain the fusion exists for: every sequence of a decode batch appends one token to a bf16 paged pool through
    aidn_qkv_rope_cache, then aidn_sdpa_launch_paged decodes over the pool; checked against the oracle end to end."""
    rng = np.random.default_rng(77)
    B, heads, kv_heads, D, bs, max_len = 3, 8, 2, 128, 16, 64
    model = heads * D
    lens = np.array([37, 64, 1], np.int32)          # sequence lengths after the append
    nblocks = 16
    bps = max_len // bs
    perm = rng.permutation(nblocks)
    bt = np.full((B, bps), 0x3fffffff, np.int32)
    at = 0
    for b in range(B):
        n = (int(lens[b]) + bs - 1) // bs
        bt[b, :n] = perm[at:at + n]
        at += n
    # pools already hold the older tokens
    kpool = (rng.standard_normal((nblocks * bs, kv_heads * D)) * 0.5).astype(np.float32)
    vpool = (rng.standard_normal((nblocks * bs, kv_heads * D)) * 0.5).astype(np.float32)
    kpool = torch.from_numpy(kpool).to(torch.bfloat16)
    vpool = torch.from_numpy(vpool).to(torch.bfloat16)
    x = rng.uniform(-1, 1, (B, model)).astype(np.float32)
    w = torch.from_numpy((rng.uniform(-1, 1, ((heads + 2 * kv_heads) * D, model)) / np.sqrt(model)).astype(np.float32))
    w = w.to(torch.bfloat16).to(torch.float32).numpy()
    cos, sin = _rope_tables(max_len, D, rng)
    positions = lens - 1
    rows = np.array([bt[b, positions[b] // bs] * bs + positions[b] % bs for b in range(B)], np.int32)
    kref, vref = kpool.float().numpy().copy(), vpool.float().numpy().copy()
    qref = O.qkv_rope_cache(x, w, None, cos, sin, heads=heads, kv_heads=kv_heads, head_dim=D, positions=positions,
                            cache_rows=rows, key_cache=kref, value_cache=vref)
    q, kc, vc = _run(x, w, None, cos, sin, heads=heads, kv_heads=kv_heads, head_dim=D, capacity=nblocks * bs,
                     positions=positions, cache_rows=rows, weight_dtype="bf16", query_dtype="bf16", cache_dtype="bf16",
                     kc=kpool.cuda(), vc=vpool.cuda())
    # decode over the pool the projection just wrote
    out = torch.full((B, heads, D), float("nan"), device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=heads, num_kv_heads=kv_heads)
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = h.workspace_bytes(B, 1, max_len)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    btd, kl = torch.from_numpy(bt).cuda(), torch.from_numpy(lens).cuda()
    qo = (heads * D, D, heads * D)
    h.launch(q=q.data_ptr(), k=kc.data_ptr(), v=vc.data_ptr(), out=out.data_ptr(), batch=B, seq_q=1, seq_kv=max_len,
             stream=stream, kv_len=kl.data_ptr(), q_stride=qo, o_stride=qo, workspace=ws.data_ptr() if nbytes else None,
             workspace_bytes=nbytes, block_table=btd.data_ptr(), block_table_stride=bps, block_size=bs, num_blocks=nblocks)
    h.poll(stream)
    h.close()
    bf = lambda a: torch.from_numpy(a).to(torch.bfloat16).to(torch.float32).numpy()
    ref = O.paged_sdpa(bf(qref).reshape(B, 1, heads, D).transpose(0, 2, 1, 3), bf(kref).reshape(nblocks, bs, kv_heads, D),
                       bf(vref).reshape(nblocks, bs, kv_heads, D), np.where(bt == 0x3fffffff, 0, bt), block_size=bs,
                       seq_kv=max_len, kv_len=lens)
    got = out.cpu().numpy().reshape(B, heads, 1, D)
    assert np.abs(got - ref).max() <= 2e-2 and np.abs(got - ref).mean() <= 2e-3


def test_backend_mirror_methods():
    """QkvProjectionRoPECacheD64 / RopeInterleaved through the backend mirror, with the reference's argument checks."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    rng = np.random.default_rng(31)
    heads, capacity, position, D = 8, 64, 17, 64
    model = heads * D
    x = rng.uniform(-1, 1, (1, model)).astype(np.float32)
    w = (rng.uniform(-1, 1, (3 * model, model)) / np.sqrt(model)).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, 3 * model).astype(np.float32)
    cos, sin = _rope_tables(capacity, D, rng)
    kref = np.zeros((capacity, model), np.float32)
    vref = np.zeros((capacity, model), np.float32)
    qref = O.qkv_rope_cache(x, w, b, cos, sin, heads=heads, kv_heads=heads, head_dim=D, positions=[position],
                            cache_rows=[position], key_cache=kref, value_cache=vref)
    be = CudaBackend(0)
    buf = lambda a: GpuBuffer(torch.from_numpy(np.ascontiguousarray(a)).reshape(-1).cuda())
    q, kc, vc = buf(np.zeros(model, np.float32)), buf(np.zeros_like(kref)), buf(np.zeros_like(vref))
    args = (buf(x), buf(w), buf(b), buf(cos), buf(sin), q, kc, vc)
    be.QkvProjectionRoPECacheD64(*args, heads, capacity, position)
    be.Synchronize()
    assert np.abs(q.tensor.cpu().numpy() - qref[0]).max() <= 2e-5
    assert np.abs(kc.tensor.cpu().numpy().reshape(capacity, model) - kref).max() <= 2e-5
    assert np.abs(vc.tensor.cpu().numpy().reshape(capacity, model) - vref).max() <= 2e-5
    with pytest.raises(ValueError):
        be.QkvProjectionRoPECacheD64(*args, heads, capacity, capacity)
    with pytest.raises(ValueError):
        be.QkvProjectionRoPECacheD64(*args, heads, capacity, -1)
    with pytest.raises(ValueError):
        be.QkvProjectionRoPECacheD64(None, *args[1:], heads, capacity, position)
    with pytest.raises(ValueError):
        be.QkvProjectionRoPECacheD64(*args, heads * 2, capacity, position)      # buffers too small for 16 heads
    xin = rng.uniform(-1, 1, (18, 8)).astype(np.float32)
    c2, s2 = _rope_tables(32, 8, rng)
    out = buf(np.zeros_like(xin))
    be.RopeInterleaved(buf(xin), buf(c2), buf(s2), out, 18, 8, 6, 5)
    be.Synchronize()
    assert np.abs(out.tensor.cpu().numpy().reshape(18, 8) - O.rope_interleaved(xin, c2, s2, 6, 5)).max() <= 1e-6
    with pytest.raises(ValueError):
        be.RopeInterleaved(buf(xin), buf(c2), buf(s2), out, 18, 8, 6, 30)
    be.Dispose()

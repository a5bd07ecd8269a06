"""GPU parity of the paged-K/V entry point (aidn_sdpa_launch_paged) and of the backend's PagedAttention* mirror.

The cases restate tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/PagedAttentionCudaTests.cs of the reference (a pool
with spare blocks, a scattered block table, expected values from standard attention over the gathered keys) and then
widen them: batched sequences of ragged length sharing one pool, bf16 / fp16 pools, serving-sized shapes."""
import numpy as np
import pytest
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O

from tests._harness import AIDN_DT, TORCH_DT, compare, gen

pytestmark = pytest.mark.gpu


def _pool(num_blocks, block_size, kv_heads, head_dim, dtype, seed):
    k, kf = gen((num_blocks, block_size, kv_heads, head_dim), dtype, seed)
    v, vf = gen((num_blocks, block_size, kv_heads, head_dim), dtype, seed + 1)
    return k, kf, v, vf


def _tables(rng, batch, blocks_per_seq, num_blocks, lens, block_size):
    """Disjoint scattered tables; entries past a sequence's length hold a poison value that must never be read."""
    perm = rng.permutation(num_blocks)
    bt = np.full((batch, blocks_per_seq), 0x3fffffff, np.int32)
    at = 0
    for b in range(batch):
        n = (int(lens[b]) + block_size - 1) // block_size
        bt[b, :n] = perm[at:at + n]
        at += n
    assert at <= num_blocks
    return bt


def _launch_paged(q, kpool, vpool, bt, *, dtype, block_size, seq_q, seq_kv, heads, kv_heads, head_dim, kv_len=None,
                  causal=False, causal_offset=0, path=N.PATH_AUTO, out_dtype="f32", token_major=True, chunk=0,
                  num_blocks=None):
    """q is [B, seq_q, heads, D] when token_major (the reference's layout) else [B, heads, seq_q, D]."""
    B = bt.shape[0]
    out = torch.full(q.shape, float("nan"), dtype=TORCH_DT[out_dtype], device="cuda")
    h = N.Handle(device=0, qkv_dtype=AIDN_DT[dtype], out_dtype=AIDN_DT[out_dtype], head_dim=head_dim, num_q_heads=heads,
                 num_kv_heads=kv_heads, causal=causal, causal_bottom_right=False, causal_offset=causal_offset,
                 path=path, decode_chunk=chunk)
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = h.workspace_bytes(B, seq_q, seq_kv)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    btd = torch.from_numpy(bt).cuda()
    kl = torch.from_numpy(np.asarray(kv_len, np.int32)).cuda() if kv_len is not None else None
    qo = (seq_q * heads * head_dim, head_dim, heads * head_dim) if token_major else None
    h.launch(q=q.data_ptr(), k=kpool.data_ptr(), v=vpool.data_ptr(), out=out.data_ptr(), batch=B, seq_q=seq_q,
             seq_kv=seq_kv, stream=stream, kv_len=kl.data_ptr() if kl is not None else None, q_stride=qo, o_stride=qo,
             workspace=ws.data_ptr() if nbytes else None, workspace_bytes=nbytes, block_table=btd.data_ptr(),
             block_table_stride=bt.shape[1], block_size=block_size,
             num_blocks=kpool.shape[0] if num_blocks is None else num_blocks)
    h.poll(stream)
    info = dict(path=h.last_path, launches=h.last_launch_count)
    h.close()
    return out, info


# ------------------------------------------------------------------------------- the reference's own test shapes
@pytest.mark.parametrize("heads,head_dim,block_size,seq_len", [(4, 64, 16, 40), (2, 128, 8, 20), (8, 32, 32, 100)])
def test_backend_paged_decode_reference_cases(heads, head_dim, block_size, seq_len):
    """PagedAttentionDecode_MatchesCpuOracle (PagedAttentionCudaTests.cs:43-121): fp32 pool, uniform(-1,1) values,
    tolerance 2e-3 + 2e-3|e| there; held to the fp32 contract (1e-5 relative) here."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    rng = np.random.default_rng(0xA77 + heads + seq_len)
    n_logical = (seq_len + block_size - 1) // block_size
    max_blocks = n_logical + 5
    kc = rng.uniform(-1, 1, (max_blocks, block_size, heads, head_dim)).astype(np.float32)
    vc = rng.uniform(-1, 1, (max_blocks, block_size, heads, head_dim)).astype(np.float32)
    q = rng.uniform(-1, 1, (heads, head_dim)).astype(np.float32)
    bt = rng.permutation(max_blocks)[:n_logical].astype(np.int32)
    scale = 1.0 / np.sqrt(np.float32(head_dim))
    want = O.paged_attention_rows(q, kc, vc, bt, heads, heads, head_dim, block_size, 1, 0, scale, decode_len=seq_len)
    be = CudaBackend(0)
    buf = lambda a: GpuBuffer(torch.from_numpy(a).reshape(-1).cuda())
    ob = be.PagedAttentionDecode(buf(q), buf(kc), buf(vc), buf(bt), heads, head_dim, block_size, seq_len, float(scale))
    be.Synchronize()
    assert ob.Size == heads * head_dim
    got = ob.tensor.cpu().numpy().reshape(1, heads, head_dim)
    assert np.all(np.abs(got - want) <= 2e-5 + 2e-5 * np.abs(want))
    be.Dispose()


@pytest.mark.parametrize("heads,head_dim,block_size,num_queries,start_pos",
                         [(4, 64, 16, 8, 0), (2, 128, 8, 12, 5), (8, 32, 32, 20, 40)])
def test_backend_paged_prefill_reference_cases(heads, head_dim, block_size, num_queries, start_pos):
    """PagedAttentionPrefill_MatchesCpuOracle (PagedAttentionCudaTests.cs:123-205)."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    rng = np.random.default_rng(0xB99 + heads + num_queries + start_pos)
    key_len = start_pos + num_queries
    n_logical = (key_len + block_size - 1) // block_size
    max_blocks = n_logical + 5
    kc = rng.uniform(-1, 1, (max_blocks, block_size, heads, head_dim)).astype(np.float32)
    vc = rng.uniform(-1, 1, (max_blocks, block_size, heads, head_dim)).astype(np.float32)
    q = rng.uniform(-1, 1, (num_queries, heads, head_dim)).astype(np.float32)
    bt = rng.permutation(max_blocks)[:n_logical].astype(np.int32)
    scale = 1.0 / np.sqrt(np.float32(head_dim))
    want = O.paged_attention_rows(q, kc, vc, bt, heads, heads, head_dim, block_size, num_queries, start_pos, scale)
    be = CudaBackend(0)
    buf = lambda a: GpuBuffer(torch.from_numpy(a).reshape(-1).cuda())
    ob = be.PagedAttentionPrefill(buf(q), buf(kc), buf(vc), buf(bt), heads, head_dim, block_size, num_queries,
                                  start_pos, float(scale))
    be.Synchronize()
    got = ob.tensor.cpu().numpy().reshape(num_queries, heads, head_dim)
    assert np.all(np.abs(got - want) <= 2e-5 + 2e-5 * np.abs(want))
    be.Dispose()


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_backend_paged_gqa_cases(dtype):
    """The Gqa variants (pool [MaxBlocks, blockSize, kvHeads, D], kv head = h / (heads / kvHeads))."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    heads, kv_heads, head_dim, block_size = 8, 2, 64, 16
    rng = np.random.default_rng(77)
    be = CudaBackend(0)
    buf = lambda t: GpuBuffer(t.reshape(-1))
    for num_queries, start_pos in ((1, 52), (9, 30)):
        key_len = start_pos + num_queries
        n_logical = (key_len + block_size - 1) // block_size
        k, kf, v, vf = _pool(n_logical + 3, block_size, kv_heads, head_dim, dtype, 300 + num_queries)
        q, qf = gen((num_queries, heads, head_dim), dtype, 310 + num_queries)
        bt = rng.permutation(n_logical + 3)[:n_logical].astype(np.int32)
        btb = GpuBuffer(torch.from_numpy(bt).cuda())
        if num_queries == 1:
            ob = be.PagedAttentionDecodeGqa(buf(q), buf(k), buf(v), btb, heads, kv_heads, head_dim, block_size, key_len, 0.125)
            want = O.paged_attention_rows(qf, kf, vf, bt, heads, kv_heads, head_dim, block_size, 1, 0, 0.125, decode_len=key_len)
        else:
            ob = be.PagedAttentionPrefillGqa(buf(q), buf(k), buf(v), btb, heads, kv_heads, head_dim, block_size,
                                             num_queries, start_pos, 0.125)
            want = O.paged_attention_rows(qf, kf, vf, bt, heads, kv_heads, head_dim, block_size, num_queries, start_pos, 0.125)
        be.Synchronize()
        compare(ob.tensor.reshape(num_queries, heads, head_dim), want, dtype, f"gqa paged nq={num_queries}")
    be.Dispose()


def test_backend_paged_guards():
    """GpuKernelGuards.Attention / Gqa / PagedAttentionBuffers (GpuKernelGuards.cs:15-35, 83-99)."""
    from aidotnet.tensors_b200.backend import CudaBackend, GpuBuffer
    be = CudaBackend(0)
    z = lambda n, dt=torch.float32: GpuBuffer(torch.zeros(n, dtype=dt, device="cuda"))
    q, pool, bt = z(4 * 64), z(3 * 16 * 4 * 64), z(3, torch.int32)
    with pytest.raises(ValueError):
        be.PagedAttentionDecode(q, pool, pool, bt, 0, 64, 16, 40, 0.125)
    with pytest.raises(ValueError):
        be.PagedAttentionDecode(q, pool, pool, bt, 4, 300, 16, 40, 0.125)
    with pytest.raises(ValueError):
        be.PagedAttentionDecode(q, pool, pool, bt, 4, 64, 0, 40, 0.125)
    with pytest.raises(ValueError):
        be.PagedAttentionDecode(q, pool, pool, bt, 4, 64, 16, 64, 0.125)        # table too short for 64 keys
    with pytest.raises(ValueError):
        be.PagedAttentionDecode(q, pool, z(5), bt, 4, 64, 16, 40, 0.125)        # pools differ in size
    with pytest.raises(ValueError):
        be.PagedAttentionDecode(q, z(1000), z(1000), bt, 4, 64, 16, 40, 0.125)  # not a whole number of blocks
    with pytest.raises(ValueError):
        be.PagedAttentionDecodeGqa(q, pool, pool, bt, 4, 3, 64, 16, 40, 0.125)
    with pytest.raises(ValueError):
        be.PagedAttentionPrefill(q, pool, pool, bt, 4, 64, 16, 1, -1, 0.125)
    be.Dispose()


# ------------------------------------------------------------------------------- batched, ragged, 16-bit pools
@pytest.mark.parametrize("dtype", ["bf16", "f16", "f32"])
@pytest.mark.parametrize("shape", [(5, 8, 8, 128, 16, 700), (3, 16, 2, 128, 32, 1000), (4, 8, 2, 64, 8, 333),
                                   (2, 12, 1, 128, 64, 260), (3, 4, 4, 256, 16, 200), (2, 6, 2, 64, 24, 130)])
@pytest.mark.parametrize("chunk", [0, 64])
def test_paged_decode_batched_ragged(dtype, shape, chunk):
    """Sequences of different length share one pool; their tables are scattered and disjoint, entries past a
    sequence's last block are poison.  Block size 24 exercises the non-power-of-two index path."""
    B, heads, kv_heads, D, bs, L = shape
    if dtype == "f32" and D == 256:
        pytest.skip("fp32 D=256 is served by the generic kernel")
    rng = np.random.default_rng(900 + B + L)
    lens = np.array([L, L // 2 + 1, 7, L - 3, 1][:B], np.int32)
    bps = (L + bs - 1) // bs
    nblocks = int(sum((int(x) + bs - 1) // bs for x in lens)) + 4
    k, kf, v, vf = _pool(nblocks, bs, kv_heads, D, dtype, 500)
    q, qf = gen((B, 1, heads, D), dtype, 502)
    bt = _tables(rng, B, bps, nblocks, lens, bs)
    out, info = _launch_paged(q, k, v, bt, dtype=dtype, block_size=bs, seq_q=1, seq_kv=L, heads=heads, kv_heads=kv_heads,
                              head_dim=D, kv_len=lens, chunk=chunk)
    assert info["path"] == N.PATH_DECODE
    ref = O.paged_sdpa(qf.transpose(0, 2, 1, 3), kf, vf, np.where(bt == 0x3fffffff, 0, bt), block_size=bs, seq_kv=L,
                       kv_len=lens)
    compare(out, ref.transpose(0, 2, 1, 3), dtype, f"paged decode {shape}")


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("shape", [(2, 8, 2, 128, 16, 200, 77), (1, 4, 4, 64, 32, 130, 0), (3, 6, 2, 128, 8, 64, 500),
                                   (2, 8, 8, 96, 16, 50, 33)])
def test_paged_prefill_batched(dtype, shape):
    """Chunked prefill: seq_q new queries after start_pos cached keys, per batch entry the same start_pos; D=96 and
    fp32 go through the generic kernel."""
    B, heads, kv_heads, D, bs, nq, start = shape
    rng = np.random.default_rng(1200 + nq)
    L = start + nq
    bps = (L + bs - 1) // bs
    nblocks = B * bps + 3
    k, kf, v, vf = _pool(nblocks, bs, kv_heads, D, dtype, 600)
    q, qf = gen((B, nq, heads, D), dtype, 602)
    bt = _tables(rng, B, bps, nblocks, [L] * B, bs)
    out, info = _launch_paged(q, k, v, bt, dtype=dtype, block_size=bs, seq_q=nq, seq_kv=L, heads=heads,
                              kv_heads=kv_heads, head_dim=D, causal=True, causal_offset=start)
    ref = O.paged_sdpa(qf.transpose(0, 2, 1, 3), kf, vf, bt, block_size=bs, seq_kv=L, causal=True, causal_offset=start)
    compare(out, ref.transpose(0, 2, 1, 3), dtype, f"paged prefill {shape}")


@pytest.mark.parametrize("dtype", ["bf16", "f16"])
@pytest.mark.parametrize("shape", [(2, 8, 2, 128, 16, 300, 77), (1, 4, 4, 64, 32, 130, 0), (3, 6, 2, 128, 8, 64, 500),
                                   (2, 3, 3, 128, 128, 257, 130), (1, 8, 1, 64, 64, 513, 1000), (2, 2, 1, 128, 16, 1, 300)])
def test_paged_prefill_on_the_tcgen05_kernel(dtype, shape):
    """Chunked prefill through the tensor-core kernel: every supported block size (8..128), head pairs and row pairs,
    ragged kv_len (a sequence shorter than the launch's seq_kv: its trailing table entries are poison), a start
    offset that is not a multiple of the block or the tile, and seq_q = 1 forced onto this kernel."""
    B, heads, kv_heads, D, bs, nq, start = shape
    rng = np.random.default_rng(1300 + nq + bs)
    L = start + nq
    lens = np.array([L, max(1, L - 37), max(1, L // 2)][:B], np.int32)
    bps = (L + bs - 1) // bs
    nblocks = int(sum((int(x) + bs - 1) // bs for x in lens)) + 3
    k, kf, v, vf = _pool(nblocks, bs, kv_heads, D, dtype, 650)
    q, qf = gen((B, nq, heads, D), dtype, 652)
    bt = _tables(rng, B, bps, nblocks, lens, bs)
    out, info = _launch_paged(q, k, v, bt, dtype=dtype, block_size=bs, seq_q=nq, seq_kv=L, heads=heads,
                              kv_heads=kv_heads, head_dim=D, causal=True, causal_offset=start, kv_len=lens,
                              path=N.PATH_PREFILL_SM100)
    assert info["path"] == N.PATH_PREFILL_SM100
    ref = O.paged_sdpa(qf.transpose(0, 2, 1, 3), kf, vf, np.where(bt == 0x3fffffff, 0, bt), block_size=bs, seq_kv=L,
                       kv_len=lens, causal=True, causal_offset=start)
    compare(out, ref.transpose(0, 2, 1, 3), dtype, f"paged tcgen05 prefill {shape}")


def test_paged_prefill_identity_table_equals_contiguous_prefill():
    """Size-independent property at a benchmark-sized shape: an identity block table must reproduce the contiguous
    tensor-core prefill bit for bit (same tiles in shared memory, fetched by 8 boxes instead of 1)."""
    B, heads, kv_heads, D, bs, S = 2, 8, 2, 128, 16, 4096
    k, _, v, _ = _pool(B * S // bs, bs, kv_heads, D, "bf16", 720)     # == a [B, S, Hkv, D] cache
    q, _ = gen((B, S, heads, D), "bf16", 722)
    bt = np.arange(B * S // bs, dtype=np.int32).reshape(B, S // bs)
    paged, info = _launch_paged(q, k, v, bt, dtype="bf16", block_size=bs, seq_q=S, seq_kv=S, heads=heads,
                                kv_heads=kv_heads, head_dim=D, causal=True, causal_offset=0)
    assert info["path"] == N.PATH_PREFILL_SM100
    out = torch.full(q.shape, float("nan"), dtype=torch.float32, device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=heads, num_kv_heads=kv_heads, causal=True,
                 causal_bottom_right=False, causal_offset=0)
    stream = torch.cuda.current_stream().cuda_stream
    qo = (S * heads * D, D, heads * D)
    st = (S * kv_heads * D, D, kv_heads * D)
    h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=S, seq_kv=S,
             stream=stream, q_stride=qo, o_stride=qo, k_stride=st, v_stride=st)
    h.poll(stream)
    assert h.last_path == N.PATH_PREFILL_SM100
    h.close()
    assert torch.equal(paged, out)


def test_paged_equals_contiguous_when_table_is_identity():
    """Size-independent property at a serving shape: with block_table = identity the paged launch must reproduce
    the contiguous launch bit for bit (same kernel arithmetic, different addressing)."""
    B, heads, kv_heads, D, bs, L = 8, 32, 8, 128, 16, 4096
    k, _, v, _ = _pool(B * L // bs, bs, kv_heads, D, "bf16", 700)
    q, _ = gen((B, 1, heads, D), "bf16", 702)
    bt = np.arange(B * L // bs, dtype=np.int32).reshape(B, L // bs)
    lens = np.array([L, L - 1, 17, 2048, 4000, 1, 999, 3333], np.int32)
    paged, _ = _launch_paged(q, k, v, bt, dtype="bf16", block_size=bs, seq_q=1, seq_kv=L, heads=heads,
                             kv_heads=kv_heads, head_dim=D, kv_len=lens)
    # the same memory seen as a contiguous [B, L, Hkv, D] cache: strides (B, H, S) = (L*Hkv*D, D, Hkv*D)
    out = torch.full(q.shape, float("nan"), dtype=torch.float32, device="cuda")
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=heads, num_kv_heads=kv_heads)
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = h.workspace_bytes(B, 1, L)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    kl = torch.from_numpy(lens).cuda()
    qo = (heads * D, D, heads * D)
    st = (L * kv_heads * D, D, kv_heads * D)
    h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=1, seq_kv=L,
             stream=stream, kv_len=kl.data_ptr(), q_stride=qo, o_stride=qo, k_stride=st, v_stride=st,
             workspace=ws.data_ptr() if nbytes else None, workspace_bytes=nbytes)
    h.poll(stream)
    h.close()
    assert torch.equal(paged, out)


def test_paged_bad_block_is_skipped_and_reported():
    """An entry outside [0, num_blocks) is not dereferenced: its keys are skipped and poll() says so."""
    heads, D, bs, L = 4, 64, 16, 64
    k, kf, v, vf = _pool(8, bs, heads, D, "bf16", 800)
    q, qf = gen((1, 1, heads, D), "bf16", 802)
    bt = np.array([[3, 100000, 5, 1]], np.int32)
    with pytest.raises(N.AidnError) as e:
        _launch_paged(q, k, v, bt, dtype="bf16", block_size=bs, seq_q=1, seq_kv=L, heads=heads, kv_heads=heads, head_dim=D)
    assert e.value.status == N.EINVAL and "block-table" in e.value.message


def test_paged_argument_errors():
    k, _, v, _ = _pool(4, 16, 2, 64, "bf16", 810)
    q, _ = gen((1, 1, 2, 64), "bf16", 811)
    bt = np.zeros((1, 4), np.int32)
    with pytest.raises(N.AidnError) as e:
        _launch_paged(q, k, v, bt, dtype="bf16", block_size=0, seq_q=1, seq_kv=64, heads=2, kv_heads=2, head_dim=64)
    assert e.value.status == N.EINVAL
    with pytest.raises(N.AidnError) as e:   # two sequences, a table row too short for seq_kv and no kv_len
        _launch_paged(torch.cat([q, q]), k, v, np.zeros((2, 2), np.int32), dtype="bf16", block_size=16, seq_q=1,
                      seq_kv=64, heads=2, kv_heads=2, head_dim=64)
    assert e.value.status == N.EINVAL


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_paged_kv_append_then_prefill(dtype):
    """DevicePagedKVCache.Append's device half: a prompt is appended in three ragged pieces (crossing block
    boundaries, starting mid-block), the pool rows must hold exactly those tokens, untouched rows stay untouched, and
    a paged prefill over the pool equals the contiguous oracle."""
    rng = np.random.default_rng(55)
    heads, kv_heads, D, bs, nblocks = 4, 2, 64, 16, 9
    total = 100
    k, kf = gen((total, kv_heads, D), dtype, 1001)
    v, vf = gen((total, kv_heads, D), dtype, 1002)
    bt = rng.permutation(nblocks)[: (total + bs - 1) // bs].astype(np.int32)
    btd = torch.from_numpy(bt).cuda()
    kp = torch.full((nblocks, bs, kv_heads, D), 9.0, dtype=TORCH_DT[dtype], device="cuda")
    vp = torch.full((nblocks, bs, kv_heads, D), -9.0, dtype=TORCH_DT[dtype], device="cuda")
    row_bytes = kv_heads * D * k.element_size()
    stream = torch.cuda.current_stream().cuda_stream
    at = 0
    for n in (21, 50, 29):
        N.paged_kv_append(k[at:].data_ptr(), v[at:].data_ptr(), kp.data_ptr(), vp.data_ptr(), btd.data_ptr(), at, n, bs,
                          nblocks, row_bytes, stream)
        at += n
    torch.cuda.synchronize()
    flat_k, flat_v = kp.reshape(nblocks * bs, kv_heads, D), vp.reshape(nblocks * bs, kv_heads, D)
    rows = np.array([bt[t // bs] * bs + t % bs for t in range(total)])
    assert torch.equal(flat_k[rows], k) and torch.equal(flat_v[rows], v)
    untouched = np.setdiff1d(np.arange(nblocks * bs), rows)
    assert torch.all(flat_k[untouched] == 9.0) and torch.all(flat_v[untouched] == -9.0)
    q, qf = gen((1, total, heads, D), dtype, 1003)
    out, _ = _launch_paged(q, kp, vp, bt[None], dtype=dtype, block_size=bs, seq_q=total, seq_kv=total, heads=heads,
                           kv_heads=kv_heads, head_dim=D, causal=True, causal_offset=0)
    ref = O.sdpa(qf.transpose(0, 2, 1, 3), kf.transpose(1, 0, 2)[None], vf.transpose(1, 0, 2)[None], causal=True, causal_offset=0)
    compare(out, ref.transpose(0, 2, 1, 3), dtype, "prefill over an appended pool")
    with pytest.raises(N.AidnError) as e:
        N.paged_kv_append(k.data_ptr(), v.data_ptr(), kp.data_ptr(), vp.data_ptr(), btd.data_ptr(), 140, 10, bs, nblocks,
                          row_bytes, stream)
    assert e.value.status == N.EINVAL

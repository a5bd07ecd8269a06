"""ctypes front-end of the CPU oracle (``oracle/sdpa_ref.cpp``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke check and by the benchmark's CPU
baseline leg.  The product package never imports this module.

``sdpa`` takes numpy float32 arrays laid out ``[B,H,S,D]`` (any strides with a unit innermost stride)
and mirrors the semantics of the reference CPU path restated in ``sdpa_ref.cpp``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "libaidn_sdpa_oracle.so")

MASK_NONE, MASK_KEEP_U8, MASK_KEEP_F32, MASK_ADD_F32 = 0, 1, 2, 3


class _Args(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("out", ctypes.c_void_p), ("lse", ctypes.c_void_p), ("weights", ctypes.c_void_p),
        ("batch", ctypes.c_int64), ("q_heads", ctypes.c_int64), ("kv_heads", ctypes.c_int64),
        ("seq_q", ctypes.c_int64), ("seq_kv", ctypes.c_int64),
        ("head_dim", ctypes.c_int64), ("head_dim_v", ctypes.c_int64),
        ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3),
        ("v_stride", ctypes.c_int64 * 3), ("o_stride", ctypes.c_int64 * 3),
        ("scale", ctypes.c_float), ("softcap", ctypes.c_float),
        ("causal", ctypes.c_int32), ("causal_offset", ctypes.c_int64),
        ("mask_kind", ctypes.c_int32), ("mask", ctypes.c_void_p),
        ("mask_stride", ctypes.c_int64 * 4), ("kv_len", ctypes.c_void_p),
        ("accumulate_f64", ctypes.c_int32), ("faithful", ctypes.c_int32), ("threads", ctypes.c_int32),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle into ``oracle/_ref`` (no-op when the library is already newer than its source)."""
    src = os.path.join(_HERE, "sdpa_ref.cpp")
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(src)):
        return _LIB_PATH
    subprocess.check_call(["make", "-C", _HERE, "-B", "CXX=g++"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.aidn_oracle_sdpa.argtypes = [ctypes.POINTER(_Args)]
        _lib.aidn_oracle_sdpa.restype = ctypes.c_int
        _lib.aidn_oracle_max_threads.restype = ctypes.c_int
        _lib.aidn_oracle_f32_to_bf16_array.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
        _lib.aidn_oracle_bf16_to_f32_array.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64]
    return _lib


def max_threads() -> int:
    return int(lib().aidn_oracle_max_threads())


def _strides3(a: np.ndarray) -> Tuple[int, int, int]:
    assert a.dtype == np.float32 and a.ndim == 4
    assert a.shape[3] == 1 or a.strides[3] == 4, "innermost stride must be 1 element"
    return tuple(int(s // 4) for s in a.strides[:3])


def sdpa(q: np.ndarray, k: np.ndarray, v: np.ndarray, *, scale: Optional[float] = None,
         causal: bool = False, causal_offset: Optional[int] = None, softcap: float = 0.0,
         mask: Optional[np.ndarray] = None, mask_kind: int = MASK_NONE,
         kv_len: Optional[np.ndarray] = None, want_lse: bool = False, want_weights: bool = False,
         f64: bool = False, faithful: bool = False, threads: int = 0):
    """Reference attention.  Returns ``out`` or ``(out, lse, weights)`` when either extra is asked for.

    ``mask`` is a 4-D array broadcastable to ``[B,Hq,Sq,Sk]`` (size-1 axes broadcast): ``bool``/``uint8`` with
    ``MASK_KEEP_U8`` (true = attend), ``float32`` with ``MASK_KEEP_F32`` (0.0 = masked) or ``MASK_ADD_F32`` (bias).
    ``causal_offset`` defaults to ``Sk - Sq`` (the SDPA / GQA entry points); pass 0 for the FlashAttention ones.
    """
    q = np.asarray(q, dtype=np.float32)
    k = np.asarray(k, dtype=np.float32)
    v = np.asarray(v, dtype=np.float32)
    B, Hq, Sq, D = q.shape
    Bk, Hkv, Sk, Dk = k.shape
    Dv = v.shape[3]
    assert Bk == B and Dk == D and v.shape[:3] == (B, Hkv, Sk)
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    if causal_offset is None:
        causal_offset = Sk - Sq
    out = np.empty((B, Hq, Sq, Dv), dtype=np.float32)
    lse = np.empty((B, Hq, Sq), dtype=np.float32) if want_lse else None
    weights = np.empty((B, Hq, Sq, Sk), dtype=np.float32) if want_weights else None

    a = _Args()
    a.q, a.k, a.v, a.out = q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data
    a.lse = lse.ctypes.data if lse is not None else None
    a.weights = weights.ctypes.data if weights is not None else None
    a.batch, a.q_heads, a.kv_heads, a.seq_q, a.seq_kv, a.head_dim, a.head_dim_v = B, Hq, Hkv, Sq, Sk, D, Dv
    a.q_stride = (ctypes.c_int64 * 3)(*_strides3(q))
    a.k_stride = (ctypes.c_int64 * 3)(*_strides3(k))
    a.v_stride = (ctypes.c_int64 * 3)(*_strides3(v))
    a.o_stride = (ctypes.c_int64 * 3)(*_strides3(out))
    a.scale, a.softcap = float(scale), float(softcap)
    a.causal, a.causal_offset = int(bool(causal)), int(causal_offset)
    keep = []
    if mask is not None:
        assert mask.ndim == 4
        if mask_kind == MASK_NONE:
            mask_kind = MASK_KEEP_U8 if mask.dtype in (np.bool_, np.uint8) else MASK_ADD_F32
        m = np.ascontiguousarray(mask.astype(np.uint8 if mask_kind == MASK_KEEP_U8 else np.float32))
        keep.append(m)
        full = (B, Hq, Sq, Sk)
        es = m.strides
        item = m.itemsize
        ms = []
        for ax in range(4):
            assert m.shape[ax] in (1, full[ax]), f"mask axis {ax} not broadcastable"
            ms.append(0 if m.shape[ax] == 1 and full[ax] != 1 else es[ax] // item)
        a.mask, a.mask_kind = m.ctypes.data, mask_kind
        a.mask_stride = (ctypes.c_int64 * 4)(*ms)
    else:
        a.mask, a.mask_kind = None, MASK_NONE
    if kv_len is not None:
        kl = np.ascontiguousarray(kv_len, dtype=np.int32)
        assert kl.shape == (B,)
        keep.append(kl)
        a.kv_len = kl.ctypes.data
    else:
        a.kv_len = None
    a.accumulate_f64, a.faithful, a.threads = int(f64), int(faithful), int(threads)
    rc = lib().aidn_oracle_sdpa(ctypes.byref(a))
    if rc != 0:
        raise ValueError("oracle rejected the arguments")
    if want_lse or want_weights:
        return out, lse, weights
    return out


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().aidn_oracle_f32_to_bf16_array(x.ctypes.data, out.ctypes.data, x.size)
    return out


def bf16_bits_to_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().aidn_oracle_bf16_to_f32_array(x.ctypes.data, out.ctypes.data, x.size)
    return out


# ---- paged K/V ------------------------------------------------------------------------------------------------
# The reference's CPU side of a paged cache is "materialise, then attend": PagedKVCache<T>.Materialize
# (src/AiDotNet.Tensors/Engines/Autodiff/PagedKVCache.cs:127-153) gathers a sequence's blocks into contiguous
# [len, heads, headDim] tensors, and the expected values of the GPU tests are standard attention over keys read as
# pool[(blockTable[t / blockSize] * blockSize + t % blockSize), head, :]
# (tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/PagedAttentionCudaTests.cs:70-95, :150-181).

def materialize(cache: np.ndarray, block_table: np.ndarray, block_size: int, seq_kv: int,
                kv_len: Optional[np.ndarray] = None) -> np.ndarray:
    """Gathers ``cache`` [num_blocks, block_size, Hkv, D] through ``block_table`` [B, blocks_per_seq] into a
    contiguous [B, Hkv, seq_kv, D] array.  Positions at or beyond ``kv_len[b]`` are zero (their table entries are
    not read, as a cache only fills the entries a sequence uses)."""
    cache = np.asarray(cache, dtype=np.float32)
    bt = np.asarray(block_table, dtype=np.int64)
    assert cache.ndim == 4 and cache.shape[1] == block_size and bt.ndim == 2
    B = bt.shape[0]
    out = np.zeros((B, cache.shape[2], seq_kv, cache.shape[3]), dtype=np.float32)
    t = np.arange(seq_kv)
    for b in range(B):
        n = seq_kv if kv_len is None else int(min(max(int(kv_len[b]), 0), seq_kv))
        rows = bt[b, t[:n] // block_size] * block_size + t[:n] % block_size
        flat = cache.reshape(-1, cache.shape[2], cache.shape[3])
        out[b, :, :n, :] = flat[rows].transpose(1, 0, 2)
    return out


def paged_sdpa(q: np.ndarray, kcache: np.ndarray, vcache: np.ndarray, block_table: np.ndarray, *, block_size: int,
               seq_kv: int, kv_len: Optional[np.ndarray] = None, **kw):
    """``sdpa`` over K/V materialised from the paged pools; ``q`` is [B, Hq, Sq, D], every keyword of ``sdpa`` applies."""
    k = materialize(kcache, block_table, block_size, seq_kv, kv_len)
    v = materialize(vcache, block_table, block_size, seq_kv, kv_len)
    return sdpa(q, k, v, kv_len=kv_len, **kw)


def paged_attention_rows(q: np.ndarray, kcache: np.ndarray, vcache: np.ndarray, block_table: np.ndarray, heads: int,
                         kv_heads: int, head_dim: int, block_size: int, num_queries: int, start_pos: int,
                         scale: float, decode_len: Optional[int] = None) -> np.ndarray:
    """Direct restatement (float64 numpy, small cases) of the four reference kernels paged_attention_decode,
    _prefill, _decode_gqa and _prefill_gqa (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/
    CudaPagedAttentionKernels.cs:23-160): flat ``q`` [num_queries, heads, head_dim], flat pools, flat block table;
    query qi sees keys 0..start_pos+qi (prefill) or 0..decode_len-1 (decode, num_queries == 1).  Independent of
    ``sdpa`` and ``materialize``: it pins them."""
    q = np.asarray(q, dtype=np.float64).reshape(num_queries, heads, head_dim)
    kc = np.asarray(kcache, dtype=np.float64).reshape(-1, kv_heads, head_dim)
    vc = np.asarray(vcache, dtype=np.float64).reshape(-1, kv_heads, head_dim)
    bt = np.asarray(block_table, dtype=np.int64).reshape(-1)
    out = np.zeros((num_queries, heads, head_dim))
    for qi in range(num_queries):
        key_len = decode_len if decode_len is not None else start_pos + qi + 1
        t = np.arange(key_len)
        rows = bt[t // block_size] * block_size + t % block_size
        for h in range(heads):
            kvh = h // (heads // kv_heads)
            logits = kc[rows, kvh, :] @ q[qi, h] * scale
            w = np.exp(logits - logits.max())
            out[qi, h] = (w / w.sum()) @ vc[rows, kvh, :]
    return out.astype(np.float32)


# ---- packed Q/K/V projection + interleaved RoPE + KV-cache write ------------------------------------------------
def rope_interleaved(x: np.ndarray, cosine: np.ndarray, sine: np.ndarray, seq_len: int, start_position: int) -> np.ndarray:
    """rope_interleaved of the reference (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/Kernels/
    CudaAttentionKernels.cs:1023-1050): ``x`` is [rows, head_dim]; row r sits at position start_position + r % seq_len;
    pair (2i, 2i+1) becomes (e c - o s, e s + o c) with (c, s) = (cosine, sine)[position, i].  float32 arithmetic."""
    x = np.asarray(x, dtype=np.float32)
    rows, head_dim = x.shape
    pos = start_position + np.arange(rows) % seq_len
    c = np.asarray(cosine, np.float32)[pos]          # [rows, head_dim / 2]
    s = np.asarray(sine, np.float32)[pos]
    e, o = x[:, 0::2], x[:, 1::2]
    out = np.empty_like(x)
    out[:, 0::2] = e * c - o * s
    out[:, 1::2] = e * s + o * c
    return out


def qkv_rope_cache(x, weights, bias, cosine, sine, *, heads: int, kv_heads: int, head_dim: int, positions, cache_rows,
                   key_cache: np.ndarray, value_cache: np.ndarray):
    """The composition CudaBackend.QkvProjectionRoPECacheD64 falls back to (CudaBackend.cs:8428-8438): projected =
    x W^T, + bias, RopeInterleaved over the Q and K heads at the token's position, Q returned, the K and V rows copied
    into cache row ``cache_rows[t]``.  ``x`` [tokens, model]; ``weights`` [(heads + 2 kv_heads) head_dim, model] with the
    Q rows first, then K, then V; caches [capacity, kv_heads * head_dim] are updated in place.  Accumulates in float64
    (the check on the GPU's fp32 dot products)."""
    x = np.asarray(x, np.float64)
    w = np.asarray(weights, np.float64)
    y = x @ w.T
    if bias is not None:
        y = y + np.asarray(bias, np.float64)
    y = y.astype(np.float32)
    tokens = x.shape[0]
    q_rows, kv_rows = heads * head_dim, kv_heads * head_dim
    q = np.empty((tokens, q_rows), np.float32)
    for t in range(tokens):
        pos = int(positions[t])
        qk = y[t, :q_rows + kv_rows].reshape(-1, head_dim)
        rot = rope_interleaved(qk, cosine, sine, 1, pos).reshape(-1)
        q[t] = rot[:q_rows]
        row = int(cache_rows[t])
        if 0 <= row < key_cache.shape[0]:
            key_cache[row] = rot[q_rows:]
            value_cache[row] = y[t, q_rows + kv_rows:]
    return q


# ---- attention backward -----------------------------------------------------------------------------------------
def sdpa_backward(q, k, v, dout, *, scale: Optional[float] = None, causal: bool = False,
                  causal_offset: Optional[int] = None, bias: Optional[np.ndarray] = None,
                  keep: Optional[np.ndarray] = None, kv_len: Optional[np.ndarray] = None):
    """dQ, dK, dV of ``sdpa`` in float64 (small cases), restating FlashAttentionBackward of the reference
    (src/AiDotNet.Tensors/Engines/CpuEngine.cs:29474 and the deterministic CUDA kernels,
    CUDA/Kernels/CudaAttentionKernels.cs:251-390): P = softmax(scale Q K^T + bias, masks), dV = P^T dO,
    dP = dO V^T, dS = P (dP - rowsum(dO O)), dQ = scale dS K, dK = scale dS^T Q.  ``q`` [B,Hq,Sq,D],
    ``k``/``v`` [B,Hkv,Sk,D] (grouped-query: the gradients of a KV head sum over its query heads); ``bias`` /
    ``keep`` broadcastable to [B,Hq,Sq,Sk].  Also returns O and the log-sum-exp the GPU call consumes."""
    q, k, v, dout = (np.asarray(a, np.float64) for a in (q, k, v, dout))
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.shape[1], k.shape[2]
    g = Hq // Hkv
    if scale is None:
        scale = 1.0 / np.sqrt(D)
    if causal_offset is None:
        causal_offset = Sk - Sq
    kk, vv = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)
    s = np.einsum("bhid,bhjd->bhij", q, kk) * scale
    if bias is not None:
        s = s + np.asarray(bias, np.float64)
    vis = np.ones((B, Hq, Sq, Sk), bool)
    if keep is not None:
        vis &= np.broadcast_to(np.asarray(keep) != 0, vis.shape)
    if causal:
        vis &= (np.arange(Sk)[None, :] <= np.arange(Sq)[:, None] + causal_offset)[None, None]
    if kv_len is not None:
        vis &= (np.arange(Sk)[None, :] < np.asarray(kv_len)[:, None])[:, None, None, :]
    s = np.where(vis, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    m = np.where(np.isfinite(m), m, 0.0)
    e = np.where(vis, np.exp(s - m), 0.0)
    l = e.sum(axis=-1, keepdims=True)
    p = np.divide(e, l, out=np.zeros_like(e), where=l > 0)
    o = np.einsum("bhij,bhjd->bhid", p, vv)
    lse = np.where(l[..., 0] > 0, m[..., 0] + np.log(np.where(l[..., 0] > 0, l[..., 0], 1.0)), -np.inf)
    dv_full = np.einsum("bhij,bhid->bhjd", p, dout)
    dp = np.einsum("bhid,bhjd->bhij", dout, vv)
    delta = (dout * o).sum(axis=-1, keepdims=True)
    ds = p * (dp - delta)
    dq = np.einsum("bhij,bhjd->bhid", ds, kk) * scale
    dk_full = np.einsum("bhij,bhid->bhjd", ds, q) * scale
    dk = dk_full.reshape(B, Hkv, g, Sk, D).sum(axis=2)
    dv = dv_full.reshape(B, Hkv, g, Sk, D).sum(axis=2)
    return (dq.astype(np.float32), dk.astype(np.float32), dv.astype(np.float32), o.astype(np.float32),
            lse.astype(np.float32))


# ---- fused multi-head attention forward -----------------------------------------------------------------------------
def mha_forward(x, wq, wk, wv, wo, num_heads: int, *, mask: Optional[np.ndarray] = None) -> np.ndarray:
    """MultiHeadAttentionForward of the reference in float64
    (src/AiDotNet.Tensors/Engines/CpuEngine.MultiHeadAttention.cs:155-338 float path, :350-510 the per-head
    attention; contract src/AiDotNet.Tensors/Engines/IEngine.cs:4201-4208): ``x`` [B, S, Dm], each weight
    [Dm, Dm] applied as ``x @ W``; Q/K/V split into ``num_heads`` heads of ``Dm / num_heads`` along the last
    axis; scores scaled by ``1/sqrt(dHead)``; ``mask`` a boolean keep-mask broadcastable to [B, H, S, S] (false
    = -inf before the softmax; a row with no visible key gives zeros, :481-485); heads concatenated as
    [B, S, H*dHead] and multiplied by ``wo``."""
    x, wq, wk, wv, wo = (np.asarray(a, np.float64) for a in (x, wq, wk, wv, wo))
    B, S, Dm = x.shape
    assert Dm % num_heads == 0
    d = Dm // num_heads

    def heads(t):   # [B, S, Dm] -> [B, H, S, d]
        return t.reshape(B, S, num_heads, d).transpose(0, 2, 1, 3)

    q, k, v = heads(x @ wq), heads(x @ wk), heads(x @ wv)
    s = np.einsum("bhid,bhjd->bhij", q, k) / np.sqrt(d)
    vis = np.ones((B, num_heads, S, S), bool)
    if mask is not None:
        m = np.asarray(mask)
        assert m.ndim == 4
        vis &= np.broadcast_to(m != 0, vis.shape)
    s = np.where(vis, s, -np.inf)
    mx = s.max(axis=-1, keepdims=True)
    mx = np.where(np.isfinite(mx), mx, 0.0)
    e = np.where(vis, np.exp(s - mx), 0.0)
    l = e.sum(axis=-1, keepdims=True)
    p = np.divide(e, l, out=np.zeros_like(e), where=l > 0)
    o = np.einsum("bhij,bhjd->bhid", p, v).transpose(0, 2, 1, 3).reshape(B, S, Dm)
    return (o @ wo).astype(np.float32)

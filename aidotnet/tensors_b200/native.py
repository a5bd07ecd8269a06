"""ctypes binding of the C ABI declared in ``include/aidn_sdpa.h``.

This is the same surface a C# ``[DllImport]`` shim binds (see ``bindings/AidnSdpaNative.cs``); Python uses it
for the tests, the smoke check and the benchmark.  There is no fallback: if the CUDA library is missing or a
call fails, an exception is raised.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
# AIDN_SDPA_LIB selects a development variant of the library (see build.build_variant); unset = the shipped one.
LIB_PATH = os.environ.get("AIDN_SDPA_LIB") or os.path.join(_HERE, "lib", "libaidotnet_sdpa_sm100.so")

# aidn_status
OK, EINVAL, EUNSUPPORTED, ECUDA, EWORKSPACE, ETIMEOUT, ENCCL = range(7)
# aidn_dtype
F32, F16, BF16 = 0, 1, 2
# aidn_mask_kind
MASK_NONE, MASK_KEEP_U8, MASK_KEEP_F32, MASK_ADD_F32 = 0, 1, 2, 3
# aidn_path
PATH_AUTO, PATH_GENERIC, PATH_DECODE, PATH_PREFILL_SM100 = 0, 1, 2, 3

EXPORTS = (
    "aidn_sdpa_create", "aidn_sdpa_workspace_bytes", "aidn_sdpa_launch", "aidn_sdpa_poll", "aidn_sdpa_last_path",
    "aidn_sdpa_last_launch_count", "aidn_sdpa_destroy", "aidn_sdpa_last_error", "aidn_sdpa_device_supported",
    "aidn_cast_f32_to_bf16", "aidn_cast_f32_to_f16", "aidn_cast_bf16_to_f32", "aidn_cast_f16_to_f32",
    "aidn_sdpa_decode_noalloc", "aidn_sdpa_launch_paged", "aidn_qkv_rope_cache", "aidn_rope_interleaved",
    "aidn_sdpa_backward", "aidn_sdpa_backward_workspace_bytes", "aidn_paged_kv_append", "aidn_mha_forward",
    "aidn_mha_workspace_bytes", "aidn_peer_export", "aidn_peer_open", "aidn_peer_close",
    "aidn_sdpa_debug_set",   # include/aidn_sdpa_debug.h
)


class SdpaDesc(ctypes.Structure):
    _fields_ = [
        ("device", ctypes.c_int32), ("qkv_dtype", ctypes.c_int32), ("out_dtype", ctypes.c_int32),
        ("head_dim", ctypes.c_int32), ("num_q_heads", ctypes.c_int32), ("num_kv_heads", ctypes.c_int32),
        ("causal", ctypes.c_int32), ("causal_bottom_right", ctypes.c_int32), ("causal_offset", ctypes.c_int64),
        ("mask_kind", ctypes.c_int32), ("emit_lse", ctypes.c_int32), ("softcap", ctypes.c_float),
        ("path", ctypes.c_int32), ("head_begin", ctypes.c_int32), ("head_count", ctypes.c_int32),
        ("decode_chunk", ctypes.c_int32), ("max_batch", ctypes.c_int32), ("max_seq_q", ctypes.c_int64),
        ("max_seq_kv", ctypes.c_int64), ("nccl_comm", ctypes.c_void_p),
    ]


class SdpaArgs(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p), ("mask", ctypes.c_void_p), ("mask_stride", ctypes.c_int64 * 4),
        ("kv_len", ctypes.c_void_p), ("batch", ctypes.c_int64), ("seq_q", ctypes.c_int64), ("seq_kv", ctypes.c_int64),
        ("q_stride", ctypes.c_int64 * 3), ("k_stride", ctypes.c_int64 * 3), ("v_stride", ctypes.c_int64 * 3),
        ("o_stride", ctypes.c_int64 * 3), ("scale", ctypes.c_float), ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_int64), ("gather_output", ctypes.c_int32), ("weights", ctypes.c_void_p),
        ("peer_count", ctypes.c_int32), ("peer_out", ctypes.c_void_p * 8),
    ]


class PagedKv(ctypes.Structure):
    _fields_ = [
        ("block_table", ctypes.c_void_p), ("block_table_stride", ctypes.c_int64), ("block_size", ctypes.c_int32),
        ("num_blocks", ctypes.c_int32),
    ]


class QkvRopeArgs(ctypes.Structure):
    _fields_ = [
        ("input", ctypes.c_void_p), ("weights", ctypes.c_void_p), ("bias", ctypes.c_void_p),
        ("cosine", ctypes.c_void_p), ("sine", ctypes.c_void_p), ("query", ctypes.c_void_p),
        ("key_cache", ctypes.c_void_p), ("value_cache", ctypes.c_void_p), ("positions", ctypes.c_void_p),
        ("cache_rows", ctypes.c_void_p), ("tokens", ctypes.c_int32), ("heads", ctypes.c_int32),
        ("kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("position", ctypes.c_int32),
        ("weight_dtype", ctypes.c_int32), ("query_dtype", ctypes.c_int32), ("cache_dtype", ctypes.c_int32),
        ("cache_capacity", ctypes.c_int64), ("max_position", ctypes.c_int64),
    ]


class SdpaBwdArgs(ctypes.Structure):
    _fields_ = [
        ("fwd", SdpaArgs), ("paged", ctypes.POINTER(PagedKv)), ("dout", ctypes.c_void_p),
        ("do_stride", ctypes.c_int64 * 3), ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
    ]


class MhaArgs(ctypes.Structure):
    _fields_ = [
        ("input", ctypes.c_void_p), ("q_weight", ctypes.c_void_p), ("k_weight", ctypes.c_void_p),
        ("v_weight", ctypes.c_void_p), ("out_weight", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("mask", ctypes.c_void_p), ("mask_stride", ctypes.c_int64 * 4), ("batch", ctypes.c_int64),
        ("seq", ctypes.c_int64), ("input_dtype", ctypes.c_int32), ("weight_dtype", ctypes.c_int32),
        ("out_dtype", ctypes.c_int32), ("reserved", ctypes.c_int32), ("workspace", ctypes.c_void_p),
        ("workspace_bytes", ctypes.c_int64),
    ]


class AidnError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"aidn_sdpa status {status}: {message}")
        self.status = status
        self.message = message


_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Loads the CUDA library.  Raises if it has not been built: there is no CPU path behind this API."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with `python -m aidotnet.tensors_b200.build` (needs nvcc)")
    lib = ctypes.CDLL(LIB_PATH)
    lib.aidn_sdpa_create.argtypes = [ctypes.POINTER(SdpaDesc), ctypes.POINTER(ctypes.c_void_p)]
    lib.aidn_sdpa_create.restype = ctypes.c_int
    lib.aidn_sdpa_workspace_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
    lib.aidn_sdpa_workspace_bytes.restype = ctypes.c_int64
    lib.aidn_sdpa_launch.argtypes = [ctypes.c_void_p, ctypes.POINTER(SdpaArgs), ctypes.c_void_p]
    lib.aidn_sdpa_launch.restype = ctypes.c_int
    lib.aidn_sdpa_poll.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    lib.aidn_sdpa_poll.restype = ctypes.c_int
    lib.aidn_sdpa_last_path.argtypes = [ctypes.c_void_p]
    lib.aidn_sdpa_last_path.restype = ctypes.c_int
    lib.aidn_sdpa_last_launch_count.argtypes = [ctypes.c_void_p]
    lib.aidn_sdpa_last_launch_count.restype = ctypes.c_int
    lib.aidn_sdpa_destroy.argtypes = [ctypes.c_void_p]
    lib.aidn_sdpa_destroy.restype = ctypes.c_int
    lib.aidn_sdpa_last_error.argtypes = []
    lib.aidn_sdpa_last_error.restype = ctypes.c_char_p
    lib.aidn_sdpa_device_supported.argtypes = [ctypes.c_int32]
    lib.aidn_sdpa_device_supported.restype = ctypes.c_int
    lib.aidn_peer_export.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_int64)]
    lib.aidn_peer_export.restype = ctypes.c_int
    lib.aidn_peer_open.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
    lib.aidn_peer_open.restype = ctypes.c_int
    lib.aidn_peer_close.argtypes = [ctypes.c_void_p]
    lib.aidn_peer_close.restype = ctypes.c_int
    for name in ("aidn_cast_f32_to_bf16", "aidn_cast_f32_to_f16", "aidn_cast_bf16_to_f32", "aidn_cast_f16_to_f32"):
        fn = getattr(lib, name)
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        fn.restype = ctypes.c_int
    lib.aidn_sdpa_decode_noalloc.argtypes = [ctypes.POINTER(SdpaDesc), ctypes.POINTER(SdpaArgs), ctypes.c_void_p]
    lib.aidn_sdpa_decode_noalloc.restype = ctypes.c_int
    lib.aidn_sdpa_launch_paged.argtypes = [ctypes.c_void_p, ctypes.POINTER(SdpaArgs), ctypes.POINTER(PagedKv),
                                           ctypes.c_void_p]
    lib.aidn_sdpa_launch_paged.restype = ctypes.c_int
    lib.aidn_sdpa_backward.argtypes = [ctypes.c_void_p, ctypes.POINTER(SdpaBwdArgs), ctypes.c_void_p]
    lib.aidn_sdpa_backward.restype = ctypes.c_int
    lib.aidn_sdpa_backward_workspace_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64]
    lib.aidn_sdpa_backward_workspace_bytes.restype = ctypes.c_int64
    lib.aidn_paged_kv_append.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                         ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int64,
                                         ctypes.c_void_p]
    lib.aidn_paged_kv_append.restype = ctypes.c_int
    lib.aidn_mha_workspace_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32]
    lib.aidn_mha_workspace_bytes.restype = ctypes.c_int64
    lib.aidn_mha_forward.argtypes = [ctypes.c_void_p, ctypes.POINTER(MhaArgs), ctypes.c_void_p]
    lib.aidn_mha_forward.restype = ctypes.c_int
    lib.aidn_qkv_rope_cache.argtypes = [ctypes.POINTER(QkvRopeArgs), ctypes.c_void_p]
    lib.aidn_qkv_rope_cache.restype = ctypes.c_int
    lib.aidn_rope_interleaved.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,
                                          ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.aidn_rope_interleaved.restype = ctypes.c_int
    lib.aidn_sdpa_debug_set.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
    lib.aidn_sdpa_debug_set.restype = ctypes.c_int
    _lib = lib
    return lib


def last_error() -> str:
    return load().aidn_sdpa_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    if status != OK:
        raise AidnError(status, last_error())


def _arr3(values: Optional[Sequence[int]]):
    return (ctypes.c_int64 * 3)(*(values if values is not None else (0, 0, 0)))


class Handle:
    """Owns one ``aidn_sdpa_t``.  Pointers are raw device addresses (``int``); the stream is a ``cudaStream_t``."""

    def __init__(self, *, device: int, qkv_dtype: int, out_dtype: int = F32, head_dim: int, num_q_heads: int,
                 num_kv_heads: Optional[int] = None, causal: bool = False, causal_bottom_right: bool = True,
                 causal_offset: int = 0, mask_kind: int = MASK_NONE, emit_lse: bool = False, softcap: float = 0.0,
                 path: int = PATH_AUTO, head_begin: int = 0, head_count: int = 0, decode_chunk: int = 0,
                 max_batch: int = 0, max_seq_q: int = 0, max_seq_kv: int = 0, nccl_comm: Optional[int] = None):
        self._lib = load()
        d = SdpaDesc()
        d.device, d.qkv_dtype, d.out_dtype, d.head_dim = device, qkv_dtype, out_dtype, head_dim
        d.num_q_heads = num_q_heads
        d.num_kv_heads = num_kv_heads if num_kv_heads else num_q_heads
        d.causal, d.causal_bottom_right, d.causal_offset = int(causal), int(causal_bottom_right), causal_offset
        d.mask_kind, d.emit_lse, d.softcap, d.path = mask_kind, int(emit_lse), softcap, path
        d.head_begin, d.head_count, d.decode_chunk = head_begin, head_count, decode_chunk
        d.max_batch, d.max_seq_q, d.max_seq_kv = max_batch, max_seq_q, max_seq_kv
        d.nccl_comm = nccl_comm
        self.desc = d
        h = ctypes.c_void_p()
        check(self._lib.aidn_sdpa_create(ctypes.byref(d), ctypes.byref(h)))
        self._h = h

    def workspace_bytes(self, batch: int, seq_q: int, seq_kv: int) -> int:
        n = self._lib.aidn_sdpa_workspace_bytes(self._h, batch, seq_q, seq_kv)
        if n < 0:
            raise AidnError(EINVAL, last_error())
        return int(n)

    def launch(self, *, q: int, k: int, v: int, out: int, batch: int, seq_q: int, seq_kv: int, stream: int,
               lse: Optional[int] = None, mask: Optional[int] = None, mask_stride: Sequence[int] = (0, 0, 0, 0),
               kv_len: Optional[int] = None, q_stride=None, k_stride=None, v_stride=None, o_stride=None,
               scale: float = 0.0, workspace: Optional[int] = None, workspace_bytes: int = 0,
               gather_output: bool = False, block_table: Optional[int] = None, block_table_stride: int = 0,
               block_size: int = 0, num_blocks: int = 0, weights: Optional[int] = None,
               peer_out: Sequence[int] = ()) -> None:
        """Enqueues one forward.  With ``block_table`` (a device int32 array) ``k`` / ``v`` are the paged pools
        ``[num_blocks, block_size, Hkv, D]`` and the call goes through ``aidn_sdpa_launch_paged``."""
        a = SdpaArgs()
        a.q, a.k, a.v, a.out, a.lse, a.mask, a.kv_len = q, k, v, out, lse, mask, kv_len
        a.mask_stride = (ctypes.c_int64 * 4)(*mask_stride)
        a.batch, a.seq_q, a.seq_kv = batch, seq_q, seq_kv
        a.q_stride, a.k_stride, a.v_stride, a.o_stride = _arr3(q_stride), _arr3(k_stride), _arr3(v_stride), _arr3(o_stride)
        a.scale, a.workspace, a.workspace_bytes, a.gather_output = scale, workspace, workspace_bytes, int(gather_output)
        a.weights = weights
        a.peer_count = len(peer_out)
        for i, ptr in enumerate(peer_out):
            a.peer_out[i] = ptr
        if block_table is not None:
            pg = PagedKv()
            pg.block_table, pg.block_table_stride = block_table, block_table_stride
            pg.block_size, pg.num_blocks = block_size, num_blocks
            check(self._lib.aidn_sdpa_launch_paged(self._h, ctypes.byref(a), ctypes.byref(pg), ctypes.c_void_p(stream)))
            return
        check(self._lib.aidn_sdpa_launch(self._h, ctypes.byref(a), ctypes.c_void_p(stream)))

    def backward_workspace_bytes(self, batch: int, seq_q: int) -> int:
        n = self._lib.aidn_sdpa_backward_workspace_bytes(self._h, batch, seq_q)
        if n < 0:
            raise AidnError(EINVAL, last_error())
        return int(n)

    def backward(self, *, q: int, k: int, v: int, out: int, lse: int, dout: int, dq: int, dk: int, dv: int, batch: int,
                 seq_q: int, seq_kv: int, stream: int, workspace: int, workspace_bytes: int, mask: Optional[int] = None,
                 mask_stride: Sequence[int] = (0, 0, 0, 0), kv_len: Optional[int] = None, q_stride=None, k_stride=None,
                 v_stride=None, o_stride=None, do_stride=None, scale: float = 0.0) -> None:
        """dQ, dK, dV (dense fp32) from dO, Q, K, V, the forward output ``out`` and its log-sum-exp ``lse``."""
        a = SdpaBwdArgs()
        f = a.fwd
        f.q, f.k, f.v, f.out, f.lse, f.mask, f.kv_len = q, k, v, out, lse, mask, kv_len
        f.mask_stride = (ctypes.c_int64 * 4)(*mask_stride)
        f.batch, f.seq_q, f.seq_kv = batch, seq_q, seq_kv
        f.q_stride, f.k_stride, f.v_stride, f.o_stride = _arr3(q_stride), _arr3(k_stride), _arr3(v_stride), _arr3(o_stride)
        f.scale, f.workspace, f.workspace_bytes = scale, workspace, workspace_bytes
        a.dout, a.do_stride, a.dq, a.dk, a.dv = dout, _arr3(do_stride), dq, dk, dv
        check(self._lib.aidn_sdpa_backward(self._h, ctypes.byref(a), ctypes.c_void_p(stream)))

    def mha_workspace_bytes(self, batch: int, seq: int, input_dtype: int, weight_dtype: int) -> int:
        n = self._lib.aidn_mha_workspace_bytes(self._h, batch, seq, input_dtype, weight_dtype)
        if n < 0:
            raise AidnError(EUNSUPPORTED, last_error())
        return int(n)

    def mha_forward(self, *, input: int, q_weight: int, k_weight: int, v_weight: int, out_weight: int, out: int,
                    batch: int, seq: int, input_dtype: int, weight_dtype: int, out_dtype: int, workspace: int,
                    workspace_bytes: int, stream: int, mask: Optional[int] = None,
                    mask_stride: Sequence[int] = (0, 0, 0, 0)) -> None:
        """Fused projections + attention + output projection ([batch, seq, heads*head_dim] in and out)."""
        a = MhaArgs()
        a.input, a.q_weight, a.k_weight, a.v_weight, a.out_weight, a.out = input, q_weight, k_weight, v_weight, out_weight, out
        a.mask = mask
        a.mask_stride = (ctypes.c_int64 * 4)(*mask_stride)
        a.batch, a.seq = batch, seq
        a.input_dtype, a.weight_dtype, a.out_dtype = input_dtype, weight_dtype, out_dtype
        a.workspace, a.workspace_bytes = workspace, workspace_bytes
        check(self._lib.aidn_mha_forward(self._h, ctypes.byref(a), ctypes.c_void_p(stream)))

    def poll(self, stream: int) -> None:
        check(self._lib.aidn_sdpa_poll(self._h, ctypes.c_void_p(stream)))

    @property
    def last_path(self) -> int:
        return int(self._lib.aidn_sdpa_last_path(self._h))

    @property
    def last_launch_count(self) -> int:
        return int(self._lib.aidn_sdpa_last_launch_count(self._h))

    def debug_set(self, ptr: Optional[int], mode: int = 1) -> None:
        self._lib.aidn_sdpa_debug_set(self._h, ctypes.c_void_p(ptr), mode)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.aidn_sdpa_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def cast(kind: str, src: int, dst: int, n: int, stream: int) -> None:
    check(getattr(load(), f"aidn_cast_{kind}")(ctypes.c_void_p(src), ctypes.c_void_p(dst), n, ctypes.c_void_p(stream)))


def decode_noalloc(desc: SdpaDesc, args: SdpaArgs, stream: int) -> None:
    """Batched decode through the entry point that allocates nothing (split-KV partials in the library's static
    16 MiB array).  For hosts that may not allocate device memory where they decode; calls that overlap on the GPU
    race on the shared array, so keep them on one stream."""
    check(load().aidn_sdpa_decode_noalloc(ctypes.byref(desc), ctypes.byref(args), ctypes.c_void_p(stream)))


def qkv_rope_cache(*, input: int, weights: int, bias: Optional[int], cosine: int, sine: int, query: int, key_cache: int,
                   value_cache: int, tokens: int, heads: int, kv_heads: int, head_dim: int, position: int = 0,
                   positions: Optional[int] = None, cache_rows: Optional[int] = None, weight_dtype: int = F32,
                   query_dtype: int = F32, cache_dtype: int = F32, cache_capacity: int, max_position: int,
                   stream: int) -> None:
    """Packed Q/K/V projection + bias + interleaved RoPE + KV-cache write for ``tokens`` resident tokens."""
    a = QkvRopeArgs()
    a.input, a.weights, a.bias, a.cosine, a.sine = input, weights, bias, cosine, sine
    a.query, a.key_cache, a.value_cache, a.positions, a.cache_rows = query, key_cache, value_cache, positions, cache_rows
    a.tokens, a.heads, a.kv_heads, a.head_dim, a.position = tokens, heads, kv_heads, head_dim, position
    a.weight_dtype, a.query_dtype, a.cache_dtype = weight_dtype, query_dtype, cache_dtype
    a.cache_capacity, a.max_position = cache_capacity, max_position
    check(load().aidn_qkv_rope_cache(ctypes.byref(a), ctypes.c_void_p(stream)))


def rope_interleaved(input: int, cosine: int, sine: int, output: int, rows: int, head_dim: int, seq_len: int,
                     start_position: int, stream: int) -> None:
    check(load().aidn_rope_interleaved(ctypes.c_void_p(input), ctypes.c_void_p(cosine), ctypes.c_void_p(sine),
                                       ctypes.c_void_p(output), rows, head_dim, seq_len, start_position,
                                       ctypes.c_void_p(stream)))


def paged_kv_append(new_keys: int, new_values: int, key_pool: int, value_pool: int, block_table: int, start_position: int,
                    tokens: int, block_size: int, num_blocks: int, row_bytes: int, stream: int) -> None:
    """Scatters ``tokens`` new K / V rows into the paged pools at positions start_position.. of one sequence."""
    check(load().aidn_paged_kv_append(ctypes.c_void_p(new_keys), ctypes.c_void_p(new_values), ctypes.c_void_p(key_pool),
                                      ctypes.c_void_p(value_pool), ctypes.c_void_p(block_table), start_position, tokens,
                                      block_size, num_blocks, row_bytes, ctypes.c_void_p(stream)))

"""Shared helpers of the GPU parity tests: run the CUDA path through the C ABI, run the CPU oracle on the same
inputs, compare with the tolerances of the contract."""
from __future__ import annotations

import numpy as np
import torch

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O

TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
AIDN_DT = {"f32": N.F32, "f16": N.F16, "bf16": N.BF16}

# Contract tolerances: 16-bit inputs vs the fp32 reference on the same (rounded) inputs: max-abs <= 2e-2 and
# mean-abs <= 2e-3; fp32 inputs: <= 1e-5 relative (error over the largest reference magnitude).
TOL_16_MAX, TOL_16_MEAN, TOL_32_REL = 2e-2, 2e-3, 1e-5


def gen(shape, dtype: str, seed: int, scale: float = 0.5):
    """Seeded N(0,1)*scale inputs, rounded to `dtype`; returns (device tensor, fp32 numpy view of the same values)."""
    g = np.random.Generator(np.random.Philox(seed))
    x = (g.standard_normal(shape, dtype=np.float32) * np.float32(scale))
    t = torch.from_numpy(x).to(TORCH_DT[dtype])
    return t.cuda(), t.to(torch.float32).numpy()


# Guard words around every buffer a launch writes (output, log-sum-exp, workspace): a kernel that stores outside its
# buffer is caught here.  The host-side stand-in for a memory checker (compare-sanitizer is not available where these
# tests run); the reference guards its own launches on the host too (Engines/DirectGpu/GpuKernelGuards.cs:10-70).
GUARD = 256
CANARY = 1232.0   # exactly representable in fp32, fp16 and bf16


def guarded(shape, dtype, device, fill=float("nan")):
    """A tensor of `shape` inside a larger allocation with GUARD canary elements on either side.  Returns (flat, body)."""
    n = int(np.prod(shape))
    flat = torch.full((n + 2 * GUARD,), CANARY, dtype=dtype, device=device)
    body = flat[GUARD:GUARD + n].view(shape)
    body.fill_(fill)
    return flat, body


def check_guards(flat, what):
    head, tail = flat[:GUARD], flat[-GUARD:]
    if flat.dtype == torch.uint8:
        ok = bool((head == 0xA5).all()) and bool((tail == 0xA5).all())
    else:
        ok = bool((head == CANARY).all()) and bool((tail == CANARY).all())
    assert ok, f"{what}: a kernel wrote outside its buffer (guard words changed)"


def run_gpu(q, k, v, *, dtype: str, out_dtype: str = "f32", causal=False, bottom_right=True, causal_offset=0,
            softcap=0.0, mask=None, mask_kind=N.MASK_NONE, kv_len=None, want_lse=False, path=N.PATH_AUTO,
            scale=0.0, decode_chunk=0, k_stride=None, v_stride=None, seq_kv=None, num_kv_heads=None,
            head_begin=0, head_count=0, out=None, poll=True, want_weights=False):
    """q [B,Hq,Sq,D], k/v [B,Hkv,Sk,D] CUDA tensors (dense unless strides are given).  Returns (out, lse, handle info)."""
    B, Hq, Sq, D = q.shape
    Hkv = num_kv_heads if num_kv_heads is not None else k.shape[1]
    Sk = seq_kv if seq_kv is not None else k.shape[2]
    dev = q.device.index or 0
    guards = []
    if out is None:
        flat, out = guarded((B, Hq, Sq, D), TORCH_DT[out_dtype], q.device)
        guards.append((flat, "output"))
    lse = None
    if want_lse:
        flat, lse = guarded((B, Hq, Sq), torch.float32, q.device)
        guards.append((flat, "log-sum-exp"))
    weights = None
    if want_weights:   # pre-filled with NaN: every element has to be written, zeros included
        flat, weights = guarded((B, Hq, Sq, Sk), torch.float32, q.device)
        weights.fill_(float("nan"))
        guards.append((flat, "attention weights"))
    mask_stride = (0, 0, 0, 0)
    mt = None
    if mask is not None:
        mt = mask.contiguous()
        full = (B, Hq, Sq, Sk)
        st = mt.stride()
        mask_stride = tuple(0 if (mt.shape[a] == 1 and full[a] != 1) else st[a] for a in range(4))
    klt = kv_len.to(torch.int32).contiguous() if kv_len is not None else None
    h = N.Handle(device=dev, qkv_dtype=AIDN_DT[dtype], out_dtype=AIDN_DT[out_dtype], head_dim=D, num_q_heads=Hq,
                 num_kv_heads=Hkv, causal=causal, causal_bottom_right=bottom_right, causal_offset=causal_offset,
                 mask_kind=mask_kind, emit_lse=want_lse, softcap=softcap, path=path, decode_chunk=decode_chunk,
                 head_begin=head_begin, head_count=head_count)
    stream = torch.cuda.current_stream().cuda_stream
    nbytes = h.workspace_bytes(B, Sq, Sk)
    ws_flat = torch.full((max(nbytes, 16) + 2 * GUARD,), 0xA5, dtype=torch.uint8, device=q.device)
    ws = ws_flat[GUARD:GUARD + max(nbytes, 16)]
    guards.append((ws_flat, "workspace"))
    h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=B, seq_q=Sq, seq_kv=Sk,
             stream=stream, lse=lse.data_ptr() if lse is not None else None,
             mask=mt.data_ptr() if mt is not None else None, mask_stride=mask_stride,
             kv_len=klt.data_ptr() if klt is not None else None, k_stride=k_stride, v_stride=v_stride, scale=scale,
             workspace=ws.data_ptr() if nbytes > 0 else None, workspace_bytes=nbytes,
             weights=weights.data_ptr() if weights is not None else None)
    if poll:
        h.poll(stream)
        for flat, what in guards:
            check_guards(flat, what)
    info = dict(path=h.last_path, launches=h.last_launch_count, weights=weights)
    h.close()
    return out, lse, info


def compare(out: torch.Tensor, ref: np.ndarray, dtype: str, what: str = ""):
    got = out.detach().to(torch.float32).cpu().numpy()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    diff = np.abs(got - ref)
    if dtype == "f32":
        rel = diff.max() / max(np.abs(ref).max(), 1e-30)
        assert rel <= TOL_32_REL, f"{what}: relative error {rel:.3e} > {TOL_32_REL}"
        return rel
    assert diff.max() <= TOL_16_MAX, f"{what}: max-abs {diff.max():.3e} > {TOL_16_MAX}"
    assert diff.mean() <= TOL_16_MEAN, f"{what}: mean-abs {diff.mean():.3e} > {TOL_16_MEAN}"
    return diff.max()


def compare_lse(lse: torch.Tensor, ref: np.ndarray, dtype: str, what: str = ""):
    got = lse.detach().cpu().numpy()
    inf_ref = np.isneginf(ref)
    assert np.array_equal(np.isneginf(got), inf_ref), f"{what}: -inf pattern of LSE differs"
    tol = 1e-4 if dtype == "f32" else 2e-2   # the reference's own half-precision LSE bar is 0.02
    assert np.abs(got[~inf_ref] - ref[~inf_ref]).max(initial=0.0) <= tol, f"{what}: LSE mismatch"


def gen_config(config: int, stream: int, shape, dtype: str, scale: float = 0.5, heads=None):
    """Inputs of a baseline configuration from the generator the benchmark uses (aidotnet/tensors_b200/synth.py):
    (device tensor, fp32 numpy view of the same rounded values)."""
    from aidotnet.tensors_b200 import synth
    t = synth.tensor(config, stream, shape, dtype, scale, heads)
    return t.cuda(), t.to(torch.float32).numpy()


def reference_rows(qf, kf, vf, b, h, rows, *, causal_offset=0, scale=None):
    """float64 attention output for an arbitrary set of query rows of one (batch entry, head): the textbook
    formulation, used where the rows are scattered (the C++ oracle takes contiguous row blocks).  Causal with the
    given offset; K / V of the head's KV group."""
    Hq, Hkv = qf.shape[1], kf.shape[1]
    kvh = h // (Hq // Hkv)
    D = qf.shape[-1]
    scale = 1.0 / np.sqrt(D) if scale is None else scale
    rows = np.asarray(rows)
    qs = qf[b, h, rows].astype(np.float64)
    s = qs @ kf[b, kvh].astype(np.float64).T * scale
    key = np.arange(kf.shape[2])[None, :]
    s = np.where(key <= rows[:, None] + causal_offset, s, -np.inf)
    s -= s.max(axis=1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(axis=1, keepdims=True)
    return p @ vf[b, kvh].astype(np.float64)


def oracle_rows(qf, kf, vf, r0, r1, *, causal, causal_offset, **kw):
    """Oracle output for query rows [r0, r1) only (used where the full tensor would take minutes on the CPU)."""
    return O.sdpa(qf[:, :, r0:r1], kf, vf, causal=causal, causal_offset=causal_offset + r0 if causal else 0, **kw)

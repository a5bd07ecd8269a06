"""Runs the library the way the reference's CUDA backend would: inside a context the caller created itself.

CudaBackend does not use the primary context.  It calls cuCtxCreate, creates its own stream with cuStreamCreate, makes
that context current before every call (src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/CudaBackend.cs:370-375,
EnsureContextCurrent :5253-5272), allocates with cuMemAlloc and hands the library raw CUdeviceptr values.  This script
builds exactly that environment through ctypes on libcuda.so.1 - no torch CUDA call in the default mode - and runs

    create -> launch (tcgen05 prefill) -> poll -> launch (split-KV decode, caller workspace) -> launch (fp32 generic)
           -> aidn_sdpa_decode_noalloc (twice) -> destroy

against the CPU oracle.  With --with-torch the process also holds torch's PRIMARY context on the same GPU and calls the
no-allocation entry point in both contexts alternately: the library's static scratch array has one copy per context, so
each context must be handed its own copy's address.

Exit code 0 = everything matched.  Run by tests/test_gpu_driver_context.py in a child process.
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # CPU side only here (dtype conversion); --with-torch additionally brings up its CUDA context

from aidotnet.tensors_b200 import native as N
from oracle import sdpa_oracle as O

cu = ctypes.CDLL("libcuda.so.1")


def ck(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed with CUresult {rc}")


class Dev:
    """Device memory owned by this script's context (cuMemAlloc / cuMemcpy)."""

    def __init__(self):
        self.ptrs = []

    def alloc(self, nbytes):
        p = ctypes.c_uint64()
        ck(cu.cuMemAlloc_v2(ctypes.byref(p), ctypes.c_size_t(max(nbytes, 16))), "cuMemAlloc")
        self.ptrs.append(p.value)
        return p.value

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.alloc(arr.nbytes)
        ck(cu.cuMemcpyHtoD_v2(ctypes.c_uint64(p), arr.ctypes.data_as(ctypes.c_void_p), ctypes.c_size_t(arr.nbytes)), "cuMemcpyHtoD")
        return p

    def download(self, ptr, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        ck(cu.cuMemcpyDtoH_v2(out.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(ptr), ctypes.c_size_t(out.nbytes)), "cuMemcpyDtoH")
        return out

    def free(self):
        for p in self.ptrs:
            cu.cuMemFree_v2(ctypes.c_uint64(p))
        self.ptrs = []


def bf16(x):
    """(uint16 bit pattern, fp32 value after rounding) of an fp32 array."""
    t = torch.from_numpy(x).to(torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16), t.to(torch.float32).numpy()


def normal(shape, seed, scale=0.5):
    return np.random.Generator(np.random.Philox(seed)).standard_normal(shape, dtype=np.float32) * np.float32(scale)


def close16(got, ref, what):
    err = np.abs(got - ref)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    assert err.max() <= 2e-2 and err.mean() <= 2e-3, f"{what}: max {err.max():.3e} mean {err.mean():.3e}"
    print(f"  ok {what}: max-abs {err.max():.2e}")


def noalloc_decode(mem, stream, seed, tag):
    B, Hq, Hkv, L, D = 3, 8, 2, 1500, 128
    qb, qf = bf16(normal((B, Hq, 1, D), seed))
    kb, kf = bf16(normal((B, Hkv, L, D), seed + 1))
    vb, vf = bf16(normal((B, Hkv, L, D), seed + 2))
    kv = np.array([1500, 64, 999], np.int32)
    d = N.SdpaDesc()
    d.device, d.qkv_dtype, d.out_dtype, d.head_dim, d.num_q_heads, d.num_kv_heads, d.decode_chunk = 0, N.BF16, N.F32, D, Hq, Hkv, 128
    a = N.SdpaArgs()
    a.q, a.k, a.v = mem.upload(qb), mem.upload(kb), mem.upload(vb)
    a.out = mem.alloc(B * Hq * D * 4)
    a.kv_len = mem.upload(kv)
    a.batch, a.seq_q, a.seq_kv = B, 1, L
    N.decode_noalloc(d, a, stream)
    ck(cu.cuStreamSynchronize(ctypes.c_void_p(stream)), "cuStreamSynchronize")
    close16(mem.download(a.out, (B, Hq, 1, D)), O.sdpa(qf, kf, vf, kv_len=kv), f"decode_noalloc {tag}")


def main():
    with_torch = "--with-torch" in sys.argv
    if with_torch:
        torch.zeros(8, device="cuda:0").sum().item()          # the primary context is alive and current now
    ck(cu.cuInit(0), "cuInit")
    dev = ctypes.c_int()
    ck(cu.cuDeviceGet(ctypes.byref(dev), 0), "cuDeviceGet")
    primary = ctypes.c_void_p()
    cu.cuCtxGetCurrent(ctypes.byref(primary))
    ctx = ctypes.c_void_p()
    ck(cu.cuCtxCreate_v2(ctypes.byref(ctx), 0, dev), "cuCtxCreate")    # a NON-primary context, current on this thread
    cur = ctypes.c_void_p()
    cu.cuCtxGetCurrent(ctypes.byref(cur))
    assert cur.value == ctx.value and cur.value != primary.value
    stream_h = ctypes.c_void_p()
    ck(cu.cuStreamCreate(ctypes.byref(stream_h), 1), "cuStreamCreate")  # CU_STREAM_NON_BLOCKING, as the backend's _stream
    stream = stream_h.value
    mem = Dev()
    print(f"non-primary context {ctx.value:#x}" + (f", primary context {primary.value:#x} alive too" if with_torch else ""))

    # --- tcgen05 prefill, grouped-query, causal, log-sum-exp --------------------------------------------------------
    B, Hq, Hkv, S, D = 2, 8, 2, 384, 128
    qb, qf = bf16(normal((B, Hq, S, D), 1))
    kb, kf = bf16(normal((B, Hkv, S, D), 2))
    vb, vf = bf16(normal((B, Hkv, S, D), 3))
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=True, emit_lse=True)
    q, k, v = mem.upload(qb), mem.upload(kb), mem.upload(vb)
    out, lse = mem.alloc(B * Hq * S * D * 4), mem.alloc(B * Hq * S * 4)
    for _ in range(2):      # the second launch re-uses the handle's cached tensor maps
        h.launch(q=q, k=k, v=v, out=out, lse=lse, batch=B, seq_q=S, seq_kv=S, stream=stream)
    h.poll(stream)
    assert h.last_path == N.PATH_PREFILL_SM100
    ref, ref_lse, _ = O.sdpa(qf, kf, vf, causal=True, want_lse=True)
    close16(mem.download(out, (B, Hq, S, D)), ref, "tcgen05 prefill in a cuCtxCreate context")
    assert np.abs(mem.download(lse, (B, Hq, S)) - ref_lse).max() <= 2e-2
    h.close()

    # --- split-KV decode through a handle, caller-provided workspace -----------------------------------------------
    B, Hq, Hkv, L, D = 4, 8, 8, 2000, 128
    qb, qf = bf16(normal((B, Hq, 1, D), 4))
    kb, kf = bf16(normal((B, Hkv, L, D), 5))
    vb, vf = bf16(normal((B, Hkv, L, D), 6))
    kv = np.array([2000, 1, 777, 1300], np.int32)
    h = N.Handle(device=0, qkv_dtype=N.BF16, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, decode_chunk=256)
    nb = h.workspace_bytes(B, 1, L)
    assert nb > 0
    out = mem.alloc(B * Hq * D * 4)
    h.launch(q=mem.upload(qb), k=mem.upload(kb), v=mem.upload(vb), out=out, batch=B, seq_q=1, seq_kv=L, stream=stream,
             kv_len=mem.upload(kv), workspace=mem.alloc(nb), workspace_bytes=nb)
    h.poll(stream)
    assert h.last_path == N.PATH_DECODE and h.last_launch_count == 2
    close16(mem.download(out, (B, Hq, 1, D)), O.sdpa(qf, kf, vf, kv_len=kv), "split-KV decode in a cuCtxCreate context")
    h.close()

    # --- fp32 contract on the generic kernel ------------------------------------------------------------------------
    qf, kf, vf = normal((1, 2, 100, 64), 7, 1.0), normal((1, 2, 100, 64), 8, 1.0), normal((1, 2, 100, 64), 9, 1.0)
    h = N.Handle(device=0, qkv_dtype=N.F32, head_dim=64, num_q_heads=2)
    out = mem.alloc(qf.nbytes)
    h.launch(q=mem.upload(qf), k=mem.upload(kf), v=mem.upload(vf), out=out, batch=1, seq_q=100, seq_kv=100, stream=stream)
    h.poll(stream)
    ref = O.sdpa(qf, kf, vf)
    rel = np.abs(mem.download(out, qf.shape) - ref).max() / np.abs(ref).max()
    assert rel <= 1e-5, rel
    print(f"  ok fp32 generic kernel: rel {rel:.2e}")
    h.close()

    # --- the entry point that allocates nothing: its scratch array has one copy per context -------------------------
    noalloc_decode(mem, stream, 20, "in the cuCtxCreate context (first call)")
    noalloc_decode(mem, stream, 30, "in the cuCtxCreate context (second call)")
    if with_torch:
        popped = ctypes.c_void_p()
        ck(cu.cuCtxPopCurrent_v2(ctypes.byref(popped)), "cuCtxPopCurrent")
        ck(cu.cuCtxSetCurrent(primary), "cuCtxSetCurrent(primary)")
        pmem = Dev()
        noalloc_decode(pmem, torch.cuda.current_stream().cuda_stream, 40, "in torch's primary context")
        pmem.free()
        ck(cu.cuCtxSetCurrent(ctx), "cuCtxSetCurrent(own)")
        noalloc_decode(mem, stream, 50, "back in the cuCtxCreate context")

    mem.free()
    cu.cuStreamDestroy_v2(stream_h)
    cu.cuCtxDestroy_v2(ctx)
    print("driver-context run ok")


if __name__ == "__main__":
    main()

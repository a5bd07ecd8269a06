#!/usr/bin/env python
"""Benchmark of the fused SDPA forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c2o16|c3|c3paged|c4|c4q|c4paged|c4gqa|c4gqatm|c4gqapaged|c5shard|c2bwd|c2bwdfull|c3bwd|mha|mhaq|qkvrope|qkvrope1|qkvrope70b|qkvrope32] [--impl reference]

One "step" is one pass of the attention forward over one synthetic batch of the named configuration.  The
default workload is the Llama-style prefill (B4 H32 S2048 D128, causal, bf16 in, fp32 out); the batched decode
configuration (B64 H32 D128, kv_len in [512,4096]) is measured in the same run and reported under "decode".
With N > 1 every rank runs the same per-GPU workload on its own head/batch shard of an N-times larger job
(no collective on the data path; weak scaling).  Prints ONE JSON line on rank 0.

FLOPs are algorithmic: 4 * D * (visible query-key pairs), i.e. causal work is counted once, not doubled.
Bytes for decode are the valid K and V rows plus Q and O, each once.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, Hq, Hkv, Sq, Sk, D, causal, dtype, kind)
    "c2": dict(B=4, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True, kind="prefill",
               name="llama_prefill_B4_H32_S2048_D128_causal_bf16"),
    "c2o16": dict(B=4, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True, kind="prefill", out16=True,
                  name="llama_prefill_B4_H32_S2048_D128_causal_bf16_in_bf16_out"),
    "c3": dict(B=2, Hq=32, Hkv=8, Sq=8192, Sk=8192, D=128, causal=True, kind="prefill",
               name="gqa_prefill_B2_Hq32_Hkv8_S8192_D128_causal_bf16"),
    "c5shard": dict(B=1, Hq=8, Hkv=1, Sq=32768, Sk=32768, D=128, causal=True, kind="prefill",
                    name="long_context_shard_B1_Hq8_Hkv1_S32768_D128_causal_bf16"),
    "c3paged": dict(B=2, Hq=32, Hkv=8, Sq=8192, Sk=8192, D=128, causal=True, kind="prefill", block_size=16,
                    name="paged_gqa_prefill_B2_Hq32_Hkv8_S8192_D128_block16_causal_bf16"),
    # attention backward (deterministic; tcgen05 dQ and dK/dV kernels for 16-bit inputs) on a quarter of the C2 shape
    "c2bwd": dict(kind="bwd", B=1, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True,
                  name="llama_backward_B1_H32_S2048_D128_causal_bf16"),
    "c2bwdfull": dict(kind="bwd", B=4, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True,
                      name="llama_backward_B4_H32_S2048_D128_causal_bf16"),
    "c3bwd": dict(kind="bwd", B=1, Hq=32, Hkv=8, Sq=8192, Sk=8192, D=128, causal=True,
                  name="gqa_backward_B1_Hq32_Hkv8_S8192_D128_causal_bf16"),
    # the in-library caller of the attention path: Q/K/V projections + attention + output projection in one call
    "mha": dict(kind="mha", B=4, S=2048, heads=32, D=128, name="mha_forward_B4_S2048_dmodel4096_H32_bf16"),
    "mhaq": dict(kind="mha", B=1, S=2048, heads=16, D=128, name="mha_forward_B1_S2048_dmodel2048_H16_bf16"),
    # the decode step in front of attention: packed Q/K/V projection of 8 resident tokens + RoPE + cache write
    "qkvrope": dict(kind="gemv", tokens=8, heads=32, kv_heads=8, D=128, weight="bf16", cache_rows=1 << 16,
                    name="qkv_rope_cache_T8_Hq32_Hkv8_D128_bf16_weights"),
    "qkvrope70b": dict(kind="gemv", tokens=1, heads=64, kv_heads=8, D=128, weight="bf16", cache_rows=1 << 16,
                       name="qkv_rope_cache_T1_Hq64_Hkv8_D128_bf16_weights"),
    "qkvrope1": dict(kind="gemv", tokens=1, heads=32, kv_heads=8, D=128, weight="bf16", cache_rows=1 << 16,
                     name="qkv_rope_cache_T1_Hq32_Hkv8_D128_bf16_weights"),
    "qkvrope32": dict(kind="gemv", tokens=1, heads=64, kv_heads=64, D=64, weight="f32", cache_rows=1 << 12,
                      name="qkv_rope_cache_T1_H64_D64_fp32_weights_reference_contract"),
    "c4q": dict(B=16, Hq=32, Hkv=32, Sq=1, Sk=4096, D=128, causal=False, kind="decode",
                name="batched_decode_quarter_B16_H32_D128_kvlen512-4096_bf16"),
    "c4": dict(B=64, Hq=32, Hkv=32, Sq=1, Sk=4096, D=128, causal=False, kind="decode",
               name="batched_decode_B64_H32_D128_kvlen512-4096_bf16"),
    # the same decode step over a paged pool [blocks, 16, Hkv, D] with a shuffled block table (the serving layout)
    "c4paged": dict(B=64, Hq=32, Hkv=32, Sq=1, Sk=4096, D=128, causal=False, kind="decode", block_size=16,
                    name="paged_decode_B64_H32_D128_block16_kvlen512-4096_bf16"),
    "c4gqa": dict(B=64, Hq=32, Hkv=8, Sq=1, Sk=4096, D=128, causal=False, kind="decode",
                  name="gqa_decode_B64_Hq32_Hkv8_D128_kvlen512-4096_bf16"),
    "c4gqatm": dict(B=64, Hq=32, Hkv=8, Sq=1, Sk=4096, D=128, causal=False, kind="decode", token_major=True,
                    name="gqa_decode_token_major_cache_B64_Hq32_Hkv8_D128_kvlen512-4096_bf16"),
    "c4gqapaged": dict(B=64, Hq=32, Hkv=8, Sq=1, Sk=4096, D=128, causal=False, kind="decode", block_size=16,
                       name="paged_gqa_decode_B64_Hq32_Hkv8_D128_block16_kvlen512-4096_bf16"),
}
# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture each,
# see profiles/).  Prefill C2 was captured directly.  Decode was captured on the B=16 quarter of C4 (525.5 MB of
# traffic for 520.1 MB of algorithmic bytes); every (batch, head) streams its own keys once, so traffic grows in
# proportion to the bytes streamed and a full-size launch is that ratio times its own algorithmic bytes.
NCU_TRAFFIC_BYTES = {"c2": 651.5e6, "c4q": 525.5e6}
NCU_DECODE_TRAFFIC_RATIO = 525.5 / 520.1


def ncu_traffic(workload_key, w, algorithmic_bytes):
    if workload_key in NCU_TRAFFIC_BYTES:
        return NCU_TRAFFIC_BYTES[workload_key]
    if w["kind"] == "decode" and workload_key in ("c4",):
        return NCU_DECODE_TRAFFIC_RATIO * algorithmic_bytes
    return None


METRIC = "attention TFLOP/s/GPU & % bf16 peak (prefill); decode HBM GB/s; 1/2/4/8 GPUs"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), bf16=float(p["bf16_tflops"]), bf16_sustained=float(p["bf16_tflops_sustained"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def visible_pairs(Sq, Sk, causal):
    if not causal:
        return Sq * Sk
    off = Sk - Sq
    return int(np.minimum(Sk, np.maximum(0, np.arange(Sq, dtype=np.int64) + off + 1)).sum())


def algorithmic_flops(w, kv_len=None):
    if w["kind"] == "decode":
        return 4 * w["Hq"] * w["D"] * int(np.sum(kv_len))
    return 4 * w["B"] * w["Hq"] * w["D"] * visible_pairs(w["Sq"], w["Sk"], w["causal"])


def algorithmic_bytes(w, kv_len=None):
    if w["kind"] == "decode":
        kv = 2 * w["Hkv"] * w["D"] * 2 * int(np.sum(kv_len))
        return kv + w["B"] * w["Hq"] * w["D"] * (2 + 4)
    qo = w["B"] * w["Hq"] * w["Sq"] * w["D"] * (2 + (2 if w.get("out16") else 4))
    return qo + 2 * w["B"] * w["Hkv"] * w["Sk"] * w["D"] * 2


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._window = [None, None]
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
                 0x80: "hw_power_brake_slowdown"}
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.samples.append((time.perf_counter(), mhz, r))
                for bit, name in names.items():
                    if r & bit and self._window[0] is not None and self._window[1] is None:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def mark_begin(self):
        self._window[0] = time.perf_counter()

    def mark_end(self):
        self._window[1] = time.perf_counter()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "note": "NVML unavailable"}
        t0, t1 = self._window
        inside = [m for (t, m, _) in self.samples if t0 is not None and t1 is not None and t0 <= t <= t1]
        note = "sampled inside the timed region"
        if not inside:
            inside = [m for (_, m, _) in self.samples]
            note = "timed region shorter than the sampling period; samples span warm-up + timed region"
        return {"sm_mhz": float(np.median(inside)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(inside), "note": note}


def make_inputs(w, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    mk = lambda *s: (torch.randn(s, generator=g, device=device) * 0.5).to(torch.bfloat16)
    q = mk(w["B"], w["Hq"], w["Sq"], w["D"])
    k = mk(w["B"], w["Hkv"], w["Sk"], w["D"])
    v = mk(w["B"], w["Hkv"], w["Sk"], w["D"])
    kv_len = None
    if w["kind"] == "decode":
        kv_len = np.random.Generator(np.random.Philox(seed)).integers(512, w["Sk"] + 1, w["B"]).astype(np.int32)
    return q, k, v, kv_len


def run_gemv(args, w, pk):
    """Times aidn_qkv_rope_cache.  The step is a GEMV: its algorithmic bytes are the packed weights (each read once)
    plus activations and outputs.  Several weight copies are cycled so that no step finds its weights in the L2."""
    from aidotnet.tensors_b200 import native as N
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    g = torch.Generator(device=dev).manual_seed(11)
    T, H, Hkv, D = w["tokens"], w["heads"], w["kv_heads"], w["D"]
    model, rows = H * D, (H + 2 * Hkv) * D
    wdt = torch.bfloat16 if w["weight"] == "bf16" else torch.float32
    copies = max(2, int(400e6 // (rows * model * (2 if w["weight"] == "bf16" else 4))) + 1)
    weights = [(torch.randn(rows, model, generator=g, device=dev) / model ** 0.5).to(wdt) for _ in range(copies)]
    x = torch.randn(T, model, generator=g, device=dev)
    bias = torch.randn(rows, generator=g, device=dev) * 0.1
    max_pos = 4096
    ang = torch.rand(max_pos, D // 2, generator=g, device=dev) * 6.28
    cos, sin = torch.cos(ang), torch.sin(ang)
    cdt = wdt
    q = torch.empty(T, model, dtype=cdt, device=dev)
    kc = torch.zeros(w["cache_rows"], Hkv * D, dtype=cdt, device=dev)
    vc = torch.zeros_like(kc)
    pos = torch.randint(0, max_pos, (T,), generator=g, device=dev, dtype=torch.int32)
    crow = torch.randperm(w["cache_rows"], generator=g, device=dev)[:T].to(torch.int32)
    stream = torch.cuda.current_stream(dev).cuda_stream
    dt = {torch.bfloat16: N.BF16, torch.float32: N.F32}
    # One prebuilt argument block per weight copy: a step is then a single C call (the kernel is a few microseconds
    # long, so per-call Python work would otherwise be what the events time).
    lib = N.load()
    blocks = []
    for wt in weights:
        a = N.QkvRopeArgs()
        a.input, a.weights, a.bias, a.cosine, a.sine = x.data_ptr(), wt.data_ptr(), bias.data_ptr(), cos.data_ptr(), sin.data_ptr()
        a.query, a.key_cache, a.value_cache = q.data_ptr(), kc.data_ptr(), vc.data_ptr()
        a.positions, a.cache_rows = pos.data_ptr(), crow.data_ptr()
        a.tokens, a.heads, a.kv_heads, a.head_dim, a.position = T, H, Hkv, D, 0
        a.weight_dtype, a.query_dtype, a.cache_dtype = dt[wdt], dt[cdt], dt[cdt]
        a.cache_capacity, a.max_position = w["cache_rows"], max_pos
        blocks.append(a)
    import ctypes
    cstream = ctypes.c_void_p(stream)
    def step(i):
        rc = lib.aidn_qkv_rope_cache(ctypes.byref(blocks[i % copies]), cstream)
        if rc != 0:
            raise RuntimeError(N.last_error())
    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    per_step = e0.elapsed_time(e1) / 1e3 / args.steps
    esz = 2 if w["weight"] == "bf16" else 4
    by = rows * model * esz + T * model * 4 + rows * 4 + T * rows * esz
    gbs = by / 1e9 / per_step
    print(json.dumps({
        "metric": "decode-step Q/K/V projection + RoPE + cache write, HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": w["weight"], "data": "synthetic",
        "config": {"workload": w["name"], "l2": "%d weight copies (%.0f MB) cycled, larger than the 126 MB L2" % (copies, copies * rows * model * esz / 1e6)},
        "tokens_per_s": T / per_step,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s", "frac": gbs / pk["hbm"],
                     "traffic": None, "algorithmic": by, "algorithmic_unit": "bytes per launch", "peak_source": pk["source"]},
        "gpu_launches": args.steps}))


def run_bwd(args, w, pk):
    """Times aidn_sdpa_backward (delta + dQ + dK/dV kernels).  FLOP convention: 10*D per visible (query, key) pair
    (five matrix products: S, dP, dV, dQ, dK), causal pairs counted once."""
    from aidotnet.tensors_b200 import native as N
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    q, k, v, _ = make_inputs(w, dev, 5)
    B, Hq, Hkv, Sq, Sk, D = w["B"], w["Hq"], w["Hkv"], w["Sq"], w["Sk"], w["D"]
    out = torch.empty((B, Hq, Sq, D), device=dev)
    lse = torch.empty((B, Hq, Sq), device=dev)
    dout = torch.randn((B, Hq, Sq, D), device=dev)
    dq = torch.empty((B, Hq, Sq, D), device=dev)
    dk = torch.empty((B, Hkv, Sk, D), device=dev)
    dv = torch.empty_like(dk)
    h = N.Handle(device=dev.index, qkv_dtype=N.BF16, head_dim=D, num_q_heads=Hq, num_kv_heads=Hkv, causal=w["causal"],
                 causal_bottom_right=True, emit_lse=True)
    stream = torch.cuda.current_stream(dev).cuda_stream
    common = dict(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), lse=lse.data_ptr(), batch=B,
                  seq_q=Sq, seq_kv=Sk, stream=stream)
    h.launch(**common)
    nb = h.backward_workspace_bytes(B, Sq)
    ws = torch.empty(nb, dtype=torch.uint8, device=dev)
    step = lambda: h.backward(dout=dout.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(), dv=dv.data_ptr(),
                              workspace=ws.data_ptr(), workspace_bytes=nb, **common)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    per_step = e0.elapsed_time(e1) / 1e3 / args.steps
    fl = 10 * B * Hq * D * visible_pairs(Sq, Sk, w["causal"])
    tf = fl / 1e12 / per_step
    print(json.dumps({
        "metric": "attention backward TFLOP/s/GPU", "value": tf, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16 (fp32 accumulation)", "data": "synthetic",
        "config": {"workload": w["name"], "flop_convention": "10*D*visible(q,k) pairs"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16"], "unit": "TFLOP/s", "frac": tf / pk["bf16"],
                     "traffic": None, "algorithmic": fl, "algorithmic_unit": "FLOP per launch",
                     "peak_source": pk["source"] + " (burst)"},
        "gpu_launches": 3 * args.steps}))


def run_mha(args, w, pk):
    """Times aidn_mha_forward with 16-bit input and weights resident in HBM (two projection GEMM launches around one
    attention launch).  FLOP: 4 projections of 2*B*S*dm^2 plus the full (unmasked) attention 4*B*H*S^2*d."""
    from aidotnet.tensors_b200 import native as N
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    B, S, H, D = w["B"], w["S"], w["heads"], w["D"]
    dm = H * D
    g = torch.Generator(device=dev).manual_seed(7)
    x = (torch.randn((B, S, dm), device=dev, generator=g) * 0.5).to(torch.bfloat16)
    ws = [(torch.randn((dm, dm), device=dev, generator=g) / dm ** 0.5).to(torch.bfloat16) for _ in range(4)]
    out = torch.empty((B, S, dm), device=dev)
    h = N.Handle(device=dev.index, qkv_dtype=N.BF16, out_dtype=N.BF16, head_dim=D, num_q_heads=H, num_kv_heads=H)
    nb = h.mha_workspace_bytes(B, S, N.BF16, N.BF16)
    wsb = torch.empty(nb + 1024, dtype=torch.uint8, device=dev)
    base = (wsb.data_ptr() + 1023) // 1024 * 1024
    stream = torch.cuda.current_stream(dev).cuda_stream
    step = lambda: h.mha_forward(input=x.data_ptr(), q_weight=ws[0].data_ptr(), k_weight=ws[1].data_ptr(),
                                 v_weight=ws[2].data_ptr(), out_weight=ws[3].data_ptr(), out=out.data_ptr(), batch=B,
                                 seq=S, input_dtype=N.BF16, weight_dtype=N.BF16, out_dtype=N.F32, workspace=base,
                                 workspace_bytes=nb, stream=stream)
    for _ in range(args.warmup):
        step()
    h.poll(stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    h.poll(stream)
    per_step = e0.elapsed_time(e1) / 1e3 / args.steps
    fl_proj = 4 * 2 * B * S * dm * dm
    fl = fl_proj + 4 * B * H * S * S * D
    tf = fl / 1e12 / per_step
    # end to end: the activations come from pinned host memory and the result goes back, every step, on one stream
    # (the weights are model state and stay resident, as the reference keeps them)
    hx = x.cpu().pin_memory()
    hout = torch.empty(out.shape, dtype=out.dtype).pin_memory()

    def e2e_step():
        x.copy_(hx, non_blocking=True)
        step()
        hout.copy_(out, non_blocking=True)
    for _ in range(max(2, args.warmup)):
        e2e_step()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    torch.cuda.synchronize()
    e2e_s = e0.elapsed_time(e1) / 1e3 / args.steps
    cpu = None
    if not args.no_cpu_baseline:
        # the reference's float path on the host cores: four sgemm + the attention restatement, one batch entry
        from oracle import sdpa_oracle as O
        xf = hx[0].to(torch.float32).numpy()
        wf = [w_.to(torch.float32).cpu().numpy() for w_ in ws]
        t0 = time.perf_counter()
        heads = lambda t: np.ascontiguousarray(t.reshape(1, S, H, D).transpose(0, 2, 1, 3))
        qh, kh, vh = heads(xf @ wf[0]), heads(xf @ wf[1]), heads(xf @ wf[2])
        att = O.sdpa(qh, kh, vh, faithful=True)
        _ = att.transpose(0, 2, 1, 3).reshape(S, dm) @ wf[3]
        dt = time.perf_counter() - t0
        cpu = {"value": fl / B / 1e12 / dt, "unit": "TFLOP/s", "cores": O.max_threads(), "kind": "port",
               "sample": "one batch entry of the workload (%.0f GFLOP): numpy sgemm projections + the attention oracle" % (fl / B / 1e9)}
    print(json.dumps({
        "metric": "multi-head attention forward TFLOP/s/GPU", "value": tf, "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": w["name"], "l2": "weights + activations of a step (%.0f MB) exceed the 126 MB L2"
                   % ((4 * dm * dm * 2 + 5 * B * S * dm * 2 + B * S * dm * 4) / 1e6)},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16"], "unit": "TFLOP/s", "frac": tf / pk["bf16"],
                     "traffic": None, "algorithmic": fl, "algorithmic_unit": "FLOP per step (3 launches)",
                     "projection_share_of_flop": fl_proj / fl, "peak_source": pk["source"]},
        "e2e": {"value": fl / 1e12 / e2e_s, "unit": "TFLOP/s", "h2d_bytes_per_step": hx.numel() * hx.element_size(),
                "d2h_bytes_per_step": hout.numel() * hout.element_size(), "ms_per_step": e2e_s * 1e3,
                "overlap": "none: copy in, three launches, copy out on one stream"},
        "cpu_baseline": cpu,
        "gpu_launches": 3 * args.steps}))


class Runner:
    """One workload bound to one handle of the C ABI; `step()` enqueues one forward pass."""

    def __init__(self, w, device_index, seed, decode_chunk=0):
        from aidotnet.tensors_b200 import native as N
        self.N = N
        self.w = w
        dev = torch.device("cuda", device_index)
        self.q, self.k, self.v, self.kv_len_host = make_inputs(w, dev, seed)
        self.kv_len = torch.from_numpy(self.kv_len_host).to(dev) if self.kv_len_host is not None else None
        out16 = bool(w.get("out16"))   # the reference's contract is an fp32 output; *o16 workloads keep the output in bf16
        self.out = torch.empty((w["B"], w["Hq"], w["Sq"], w["D"]), dtype=torch.bfloat16 if out16 else torch.float32, device=dev)
        self.h = N.Handle(device=device_index, qkv_dtype=N.BF16, out_dtype=N.BF16 if out16 else N.F32, head_dim=w["D"], num_q_heads=w["Hq"],
                          num_kv_heads=w["Hkv"], causal=w["causal"], causal_bottom_right=True,
                          max_batch=w["B"], max_seq_q=w["Sq"], max_seq_kv=w["Sk"], decode_chunk=decode_chunk)
        self.stream = torch.cuda.current_stream(dev).cuda_stream
        self.launches = 0
        self.paged = {}
        if w.get("token_major"):   # the cache stored [B, S, Hkv, D], as a KV-cache append writes it
            self.k = self.k.permute(0, 2, 1, 3).contiguous()
            self.v = self.v.permute(0, 2, 1, 3).contiguous()
            st = (w["Sk"] * w["Hkv"] * w["D"], w["D"], w["Hkv"] * w["D"])
            self.paged = dict(k_stride=st, v_stride=st)
        bs = w.get("block_size")
        if bs:
            # Scatter the logical blocks of every sequence over one shared pool [blocks, bs, Hkv, D].
            nb = w["B"] * w["Sk"] // bs
            perm = torch.randperm(nb, generator=torch.Generator().manual_seed(seed & 0x7fffffff))
            for name in ("k", "v"):
                logical = getattr(self, name).permute(0, 2, 1, 3).reshape(nb, bs, w["Hkv"], w["D"])
                pool = torch.empty_like(logical)
                pool[perm.to(dev)] = logical
                setattr(self, name, pool)
            self.table = perm.to(torch.int32).reshape(w["B"], w["Sk"] // bs).to(dev)
            self.paged = dict(block_table=self.table.data_ptr(), block_table_stride=w["Sk"] // bs, block_size=bs,
                              num_blocks=nb)

    def step(self, q=None, k=None, v=None, out=None, stream=None):
        q = self.q if q is None else q
        k = self.k if k is None else k
        v = self.v if v is None else v
        out = self.out if out is None else out
        self.h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=self.w["B"],
                      seq_q=self.w["Sq"], seq_kv=self.w["Sk"], stream=self.stream if stream is None else stream,
                      kv_len=self.kv_len.data_ptr() if self.kv_len is not None else None, **self.paged)
        self.launches += self.h.last_launch_count

    def time_steps(self, steps, warmup, sampler=None, dist=None):
        for _ in range(warmup):
            self.step()
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = self.launches
        if sampler:
            sampler.mark_begin()
        e0.record()
        for _ in range(steps):
            self.step()
        e1.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.mark_end()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3, self.launches - l0

    def time_e2e(self, steps, warmup):
        """The same C-ABI call with HOST buffers: every step copies its pinned Q/K/V in and its output back inside the
        timed region.  The three phases run on three streams over two sets of device buffers, so the host->device copy
        of step i+1 and the device->host copy of step i-1 overlap the kernel of step i (what a caller that streams
        requests through the library would do); every step still moves all of its bytes."""
        dev = self.q.device
        hq, hk, hv = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
        din = [tuple(torch.empty_like(t) for t in (self.q, self.k, self.v)) for _ in range(2)]
        dout = [torch.empty_like(self.out) for _ in range(2)]
        hout = [torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory() for _ in range(2)]
        s_in, s_c, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        in_ready = [torch.cuda.Event() for _ in range(2)]
        comp_done = [torch.cuda.Event() for _ in range(2)]
        out_free = [torch.cuda.Event() for _ in range(2)]

        def one(i):
            b = i & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(comp_done[b])            # the kernel of step i-2 has read this input set
                for d, h in zip(din[b], (hq, hk, hv)):
                    d.copy_(h, non_blocking=True)
                in_ready[b].record(s_in)
            with torch.cuda.stream(s_c):
                s_c.wait_event(in_ready[b])
                s_c.wait_event(out_free[b])              # step i-2's output has left this output buffer
                self.step(*din[b], out=dout[b], stream=s_c.cuda_stream)
                comp_done[b].record(s_c)
            with torch.cuda.stream(s_out):
                s_out.wait_event(comp_done[b])
                hout[b].copy_(dout[b], non_blocking=True)
                out_free[b].record(s_out)

        for i in range(max(2, warmup)):
            one(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s_in)
        for i in range(steps):
            one(i)
        s_out.wait_stream(s_c)
        s_out.wait_stream(s_in)
        e1.record(s_out)
        torch.cuda.synchronize()
        h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
        d2h = hout[0].numel() * hout[0].element_size()
        return e0.elapsed_time(e1) / 1e3, h2d, d2h


def cpu_reference_time(w, threads, passes=1, sample_batch=None):
    """Times the CPU restatement of the reference path (faithful mode: full-width GEMMs, KV broadcast copy)."""
    from oracle import sdpa_oracle as O
    B = sample_batch or w["B"]
    rng = np.random.Generator(np.random.Philox(7))
    mk = lambda *s: (rng.standard_normal(s, dtype=np.float32) * np.float32(0.5))
    q, k, v = mk(B, w["Hq"], w["Sq"], w["D"]), mk(B, w["Hkv"], w["Sk"], w["D"]), mk(B, w["Hkv"], w["Sk"], w["D"])
    kv = None
    if w["kind"] == "decode":
        kv = np.random.Generator(np.random.Philox(7)).integers(512, w["Sk"] + 1, B).astype(np.int32)
    t0 = time.perf_counter()
    for _ in range(passes):
        O.sdpa(q, k, v, causal=w["causal"], kv_len=kv, faithful=True, threads=threads)
    dt = (time.perf_counter() - t0) / passes
    ws = dict(w, B=B)
    return dt, algorithmic_flops(ws, kv), algorithmic_bytes(ws, kv)


def host_threads():
    """All host cores this process may use (torchrun exports OMP_NUM_THREADS=1, which is not what is wanted here)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference_arm(args, w):
    """`--impl reference`: the reference's CPU attention path (C++ restatement; the .NET original cannot run here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    sample_batch = 1
    times = []
    for i in range(args.warmup + args.steps):
        dt, fl, by = cpu_reference_time(w, threads, 1, sample_batch)
        if i >= args.warmup:
            times.append(dt)
    ms = float(np.mean(times)) * 1e3
    value = (fl / 1e12) / (ms / 1e3) if w["kind"] == "prefill" else (by / 1e9) / (ms / 1e3)
    unit = "TFLOP/s" if w["kind"] == "prefill" else "GB/s"
    sample = f"batch entry 0 of the workload ({sample_batch} of {w['B']} batch entries) per step"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": w["name"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--decode-chunk", type=int, default=0, help="keys per split of the decode kernel (0 = library's choice)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference_arm(args, w)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    pk = peaks()
    if w["kind"] == "gemv":
        if rank == 0:
            run_gemv(args, w, pk)
        return
    if w["kind"] == "bwd":
        if rank == 0:
            run_bwd(args, w, pk)
        return
    if w["kind"] == "mha":
        if rank == 0:
            run_mha(args, w, pk)
        return
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()

    runner = Runner(w, local, 0xA1D00000 + 2 + rank, args.decode_chunk)
    kvh = runner.kv_len_host
    fl, by = algorithmic_flops(w, kvh), algorithmic_bytes(w, kvh)
    secs, launches = runner.time_steps(args.steps, args.warmup, sampler, dist)
    if dist is not None:
        t = torch.tensor([secs], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    clocks = sampler.stop() if sampler else None
    per_step = secs / args.steps
    prefill = w["kind"] == "prefill"
    per_gpu = (fl / 1e12 if prefill else by / 1e9) / per_step
    value = per_gpu * world
    peak = pk["bf16"] if prefill else pk["hbm"]

    e2e_secs, h2d, d2h = runner.time_e2e(max(3, min(args.steps, 20)), 2)
    e2e_steps = max(3, min(args.steps, 20))
    if dist is not None:
        t = torch.tensor([e2e_secs], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs = float(t.item())
    e2e_value = (fl / 1e12 if prefill else by / 1e9) / (e2e_secs / e2e_steps) * world

    decode_obj = None
    if prefill and not args.no_decode:
        wd = WORKLOADS["c4"]
        rd = Runner(wd, local, 0xA1D00004 + rank)
        dsecs, dl = rd.time_steps(max(10, args.steps // 2), 3, None, dist)
        dsteps = max(10, args.steps // 2)
        if dist is not None:
            t = torch.tensor([dsecs], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dsecs = float(t.item())
        dby = algorithmic_bytes(wd, rd.kv_len_host)
        gbs = dby / 1e9 / (dsecs / dsteps)
        decode_obj = {"workload": wd["name"], "value": gbs * world, "unit": "GB/s", "ms_per_step": dsecs / dsteps * 1e3,
                      "tokens_per_s": wd["B"] * world / (dsecs / dsteps), "gpu_launches": dl,
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s",
                                   "frac": gbs / pk["hbm"], "traffic": ncu_traffic("c4", wd, dby),
                                   "traffic_unit": "bytes per launch (ncu, B=16 capture scaled by the bytes streamed)", "algorithmic": dby,
                                   "algorithmic_unit": "bytes per launch", "peak_source": pk["source"]}}
        del rd

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        dt, cfl, cby = cpu_reference_time(w, threads, 1, 1 if prefill else None)
        cpu = {"value": (cfl / 1e12 if prefill else cby / 1e9) / dt, "unit": "TFLOP/s" if prefill else "GB/s",
               "cores": threads, "kind": "port",
               "sample": ("batch entry 0 of the workload (1 of %d batch entries), one pass" % w["B"]) if prefill
               else "the full workload, one pass"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s" if prefill else "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "per_gpu": "one copy of the workload per GPU (batch x head shard of an N-fold job)",
                       "l2": "inputs+outputs larger than the 126 MB L2; no flush",
                       "flop_convention": "4*D*visible(q,k) pairs (causal counted once)"},
            "per_gpu": per_gpu, "pct_of_measured_bf16_peak": (100.0 * per_gpu / pk["bf16"]) if prefill else None,
            "tokens_per_s": w["B"] * w["Sq"] * world / per_step,
            "roofline": {"bound": "tensor" if prefill else "hbm", "achieved": per_gpu, "peak": peak,
                         "unit": "TFLOP/s" if prefill else "GB/s", "frac": per_gpu / peak,
                         "traffic": ncu_traffic(args.workload, w, by), "traffic_unit": "bytes per launch (ncu)",
                         "algorithmic": fl if prefill else by, "algorithmic_unit": "FLOP per launch" if prefill else "bytes per launch",
                         "peak_source": pk["source"] + (" (burst)" if prefill else "")},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s" if prefill else "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_secs / e2e_steps * 1e3,
                    "pipeline": "host->device copy, kernel and device->host copy on three streams over two buffer sets"},
            "gpu_launches": launches, "clocks": clocks, "decode": decode_obj,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

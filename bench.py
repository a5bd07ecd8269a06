#!/usr/bin/env python
"""Benchmark of the fused SDPA forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c1|c3|c5shard|c4|...] [--impl reference]

One "step" is one pass of the attention forward over one synthetic batch of the named configuration.  The default
workload is the Llama-style prefill (B4 H32 S2048 D128, causal, bf16 in, fp32 out), the configuration the metric is
quoted on; the same run also measures, as objects of the same JSON line, the batched decode configuration ("decode":
B64 H32 D128, kv_len in [512,4096]), the fp32 configuration ("c1"), the grouped-query prefill ("c3"), one GPU's shard
of the long-context configuration ("c5shard") and the long-context job itself ("c5": B1 Hq64/Hkv8 S32768, whole on one
GPU, or with --gpus N head-sharded over the N ranks with the all-gather of the output timed and checked).
With N > 1 every rank also runs one copy of the default workload on its own shard of an N-times larger job (no
collective on the data path; weak scaling).  Prints ONE JSON line on rank 0.

Inputs come from one counter-based generator (aidotnet/tensors_b200/synth.py: Philox keyed by configuration, stream,
batch entry and head) that the parity tests use too; after the timed region every workload compares a block of rows of
what it computed with the CPU oracle ("checked").

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
    # cfg = index of the baseline configuration (selects the generator's seed)
    "c1": dict(cfg=1, B=1, Hq=8, Hkv=8, Sq=512, Sk=512, D=64, causal=False, kind="prefill", dtype="f32",
               name="sdpa_fp32_B1_H8_S512_D64_noncausal"),
    "c2": dict(cfg=2, B=4, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True, kind="prefill",
               name="llama_prefill_B4_H32_S2048_D128_causal_bf16"),
    "c2o16": dict(cfg=2, B=4, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True, kind="prefill", out16=True,
                  name="llama_prefill_B4_H32_S2048_D128_causal_bf16_in_bf16_out"),
    "c3": dict(cfg=3, B=2, Hq=32, Hkv=8, Sq=8192, Sk=8192, D=128, causal=True, kind="prefill",
               name="gqa_prefill_B2_Hq32_Hkv8_S8192_D128_causal_bf16"),
    # one GPU's share of configuration 5: the 8 query heads of KV head 3
    "c5shard": dict(cfg=5, B=1, Hq=8, Hkv=1, Sq=32768, Sk=32768, D=128, causal=True, kind="prefill",
                    q_heads=list(range(24, 32)), kv_heads=[3],
                    name="long_context_shard_B1_Hq8_Hkv1_S32768_D128_causal_bf16"),
    "c5": dict(cfg=5, B=1, Hq=64, Hkv=8, Sq=32768, Sk=32768, D=128, causal=True, kind="prefill",
               name="long_context_B1_Hq64_Hkv8_S32768_D128_causal_bf16"),
    "c3paged": dict(cfg=3, B=2, Hq=32, Hkv=8, Sq=8192, Sk=8192, D=128, causal=True, kind="prefill", block_size=16,
                    name="paged_gqa_prefill_B2_Hq32_Hkv8_S8192_D128_block16_causal_bf16"),
    # attention backward (deterministic; tcgen05 dQ and dK/dV kernels for 16-bit inputs) on a quarter of the C2 shape
    "c2bwd": dict(cfg=2, kind="bwd", B=1, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True,
                  name="llama_backward_B1_H32_S2048_D128_causal_bf16"),
    "c2bwdfull": dict(cfg=2, kind="bwd", B=4, Hq=32, Hkv=32, Sq=2048, Sk=2048, D=128, causal=True,
                      name="llama_backward_B4_H32_S2048_D128_causal_bf16"),
    "c3bwd": dict(cfg=3, kind="bwd", B=1, Hq=32, Hkv=8, Sq=8192, Sk=8192, D=128, causal=True,
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
    "c4q": dict(cfg=4, B=16, Hq=32, Hkv=32, Sq=1, Sk=4096, D=128, causal=False, kind="decode",
                name="batched_decode_quarter_B16_H32_D128_kvlen512-4096_bf16"),
    "c4": dict(cfg=4, B=64, Hq=32, Hkv=32, Sq=1, Sk=4096, D=128, causal=False, kind="decode",
               name="batched_decode_B64_H32_D128_kvlen512-4096_bf16"),
    # the same decode step over a paged pool [blocks, 16, Hkv, D] with a shuffled block table (the serving layout)
    "c4paged": dict(cfg=4, B=64, Hq=32, Hkv=32, Sq=1, Sk=4096, D=128, causal=False, kind="decode", block_size=16,
                    name="paged_decode_B64_H32_D128_block16_kvlen512-4096_bf16"),
    "c4gqa": dict(cfg=4, B=64, Hq=32, Hkv=8, Sq=1, Sk=4096, D=128, causal=False, kind="decode",
                  name="gqa_decode_B64_Hq32_Hkv8_D128_kvlen512-4096_bf16"),
    "c4gqatm": dict(cfg=4, B=64, Hq=32, Hkv=8, Sq=1, Sk=4096, D=128, causal=False, kind="decode", token_major=True,
                    name="gqa_decode_token_major_cache_B64_Hq32_Hkv8_D128_kvlen512-4096_bf16"),
    "c4gqapaged": dict(cfg=4, B=64, Hq=32, Hkv=8, Sq=1, Sk=4096, D=128, causal=False, kind="decode", block_size=16,
                       name="paged_gqa_decode_B64_Hq32_Hkv8_D128_block16_kvlen512-4096_bf16"),
}
# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum, one ncu capture each; the
# summaries are under profiles/).  Decode was captured on the B=16 quarter of C4 (525.5 MB of traffic for 520.1 MB of
# algorithmic bytes); every (batch, head) streams its own keys once, so traffic grows in proportion to the bytes
# streamed and a full-size launch is that ratio times its own algorithmic bytes.
NCU_TRAFFIC_BYTES = {"c2": 646.8e6, "c3": 690.8e6, "c5shard": 168.2e6, "c4q": 525.5e6}
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


def make_inputs(w, device, rank=0, q_heads=None, kv_heads=None):
    """Q, K, V of the workload from the shared generator (streams 0, 1, 2 of its configuration; `rank` offsets the
    batch index of the stream so that the copies of a weak-scaling run differ).  q_heads / kv_heads: global head
    indices when only a shard of the heads is materialised."""
    from aidotnet.tensors_b200 import synth
    dt = w.get("dtype", "bf16")
    scale = 1.0 if dt == "f32" else 0.5
    q_heads = q_heads if q_heads is not None else w.get("q_heads")
    kv_heads = kv_heads if kv_heads is not None else w.get("kv_heads")
    cfg = w["cfg"] + 16 * rank
    q = synth.tensor(cfg, synth.STREAM_Q, (w["B"], len(q_heads) if q_heads else w["Hq"], w["Sq"], w["D"]), dt, scale, q_heads)
    k = synth.tensor(cfg, synth.STREAM_K, (w["B"], len(kv_heads) if kv_heads else w["Hkv"], w["Sk"], w["D"]), dt, scale, kv_heads)
    v = synth.tensor(cfg, synth.STREAM_V, (w["B"], len(kv_heads) if kv_heads else w["Hkv"], w["Sk"], w["D"]), dt, scale, kv_heads)
    kv_len = synth.lengths(cfg, w["B"], 512, w["Sk"]) if w["kind"] == "decode" else None
    return q.to(device), k.to(device), v.to(device), kv_len


def oracle_check(w, q, k, v, out, kv_len=None, rows=64, b=None, h=None):
    """Compares `rows` query rows of one (batch entry, head) of `out` with the CPU oracle on the same inputs (read
    back from the device).  Returns {"checked": bool, "max_abs": float, ...}; tolerance as in the parity tests."""
    from oracle import sdpa_oracle as O
    B, Hq, Sq, D = out.shape
    b = B - 1 if b is None else b
    h = Hq - 1 if h is None else h
    group = Hq // k.shape[1]
    kvh = h // group
    r1 = Sq
    r0 = max(0, r1 - rows)
    qf = q[b:b + 1, h:h + 1, r0:r1].float().cpu().numpy()
    kf = k[b:b + 1, kvh:kvh + 1].float().cpu().numpy()
    vf = v[b:b + 1, kvh:kvh + 1].float().cpu().numpy()
    kv = None if kv_len is None else np.asarray(kv_len[b:b + 1], np.int32)
    off = (k.shape[2] - Sq + r0) if w["causal"] else 0
    ref = O.sdpa(qf, kf, vf, causal=w["causal"], causal_offset=off, kv_len=kv)
    got = out[b:b + 1, h:h + 1, r0:r1].float().cpu().numpy()
    err = np.abs(got - ref)
    if w.get("dtype", "bf16") == "f32":
        rel = float(err.max() / max(np.abs(ref).max(), 1e-30))
        return {"checked": bool(np.isfinite(got).all() and rel <= 1e-5), "rel": rel, "rows": [int(r0), int(r1)], "b": b, "h": h}
    ok = bool(np.isfinite(got).all() and err.max() <= 2e-2 and err.mean() <= 2e-3)
    return {"checked": ok, "max_abs": float(err.max()), "mean_abs": float(err.mean()), "rows": [int(r0), int(r1)], "b": b, "h": h}


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
    q, k, v, _ = make_inputs(w, dev)
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

    def __init__(self, w, device_index, rank=0, decode_chunk=0, shard=None, nccl_comm=None):
        """shard = (head_begin, head_count): the handle computes that head range of the FULL tensors of `w`; only the
        shard's heads of Q / K / V are filled in (the rest is never read)."""
        from aidotnet.tensors_b200 import native as N
        self.N = N
        self.w = w
        dev = torch.device("cuda", device_index)
        self.dev = dev
        dt = w.get("dtype", "bf16")
        self.dtype = dt
        if shard is None:
            self.q, self.k, self.v, self.kv_len_host = make_inputs(w, dev, rank)
        else:
            hb, hc = shard
            group = w["Hq"] // w["Hkv"]
            qh = list(range(hb, hb + hc))
            kh = list(range(hb // group, (hb + hc) // group))
            qs, ks, vs, _ = make_inputs(w, dev, 0, qh, kh)
            self.q = torch.zeros((w["B"], w["Hq"], w["Sq"], w["D"]), dtype=qs.dtype, device=dev)
            self.k = torch.zeros((w["B"], w["Hkv"], w["Sk"], w["D"]), dtype=ks.dtype, device=dev)
            self.v = torch.zeros_like(self.k)
            self.q[:, hb:hb + hc] = qs
            self.k[:, kh[0]:kh[-1] + 1] = ks
            self.v[:, kh[0]:kh[-1] + 1] = vs
            self.kv_len_host = None
            del qs, ks, vs
        self.kv_len = torch.from_numpy(self.kv_len_host).to(dev) if self.kv_len_host is not None else None
        out16 = bool(w.get("out16"))   # the reference's contract is an fp32 output; *o16 workloads keep the output in bf16
        self.out = torch.zeros((w["B"], self.q.shape[1], w["Sq"], w["D"]), dtype=torch.bfloat16 if out16 else torch.float32, device=dev)
        adt = {"bf16": N.BF16, "f16": N.F16, "f32": N.F32}[dt]
        self.h = N.Handle(device=device_index, qkv_dtype=adt, out_dtype=N.BF16 if out16 else N.F32, head_dim=w["D"],
                          num_q_heads=self.q.shape[1], num_kv_heads=self.k.shape[1], causal=w["causal"], causal_bottom_right=True,
                          max_batch=w["B"], max_seq_q=w["Sq"], max_seq_kv=w["Sk"], decode_chunk=decode_chunk,
                          head_begin=shard[0] if shard else 0, head_count=shard[1] if shard else 0, nccl_comm=nccl_comm)
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
            perm = torch.randperm(nb, generator=torch.Generator().manual_seed(w["cfg"]))
            for name in ("k", "v"):
                logical = getattr(self, name).permute(0, 2, 1, 3).reshape(nb, bs, w["Hkv"], w["D"])
                pool = torch.empty_like(logical)
                pool[perm.to(dev)] = logical
                setattr(self, name, pool)
            self.table = perm.to(torch.int32).reshape(w["B"], w["Sk"] // bs).to(dev)
            self.paged = dict(block_table=self.table.data_ptr(), block_table_stride=w["Sk"] // bs, block_size=bs,
                              num_blocks=nb)

    def step(self, q=None, k=None, v=None, out=None, stream=None, gather=False, peer_out=()):
        q = self.q if q is None else q
        k = self.k if k is None else k
        v = self.v if v is None else v
        out = self.out if out is None else out
        self.h.launch(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), batch=self.w["B"],
                      seq_q=self.w["Sq"], seq_kv=self.w["Sk"], stream=self.stream if stream is None else stream,
                      kv_len=self.kv_len.data_ptr() if self.kv_len is not None else None, gather_output=gather,
                      peer_out=peer_out, **self.paged)
        self.launches += self.h.last_launch_count

    def time_steps(self, steps, warmup, sampler=None, dist=None, repeats=1, gather=False, peer_out=(), after_step=None):
        """W warm-up steps, then `repeats` loops of exactly `steps` steps, every step bracketed by CUDA events on the
        launching stream.  Returns (seconds of the FIRST loop, launches in it, per-step milliseconds of all loops).
        `after_step` is enqueued behind every step inside the timed region (the rank synchronisation of the fused
        gather)."""
        for _ in range(warmup):
            self.step(gather=gather, peer_out=peer_out)
            if after_step:
                after_step()
        torch.cuda.synchronize()
        per_step = []
        first = None
        first_launches = 0
        for r in range(repeats):
            if dist is not None:
                dist.barrier()
                torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            l0 = self.launches
            if sampler and r == 0:
                sampler.mark_begin()
            ev[0].record()
            for i in range(steps):
                self.step(gather=gather, peer_out=peer_out)
                if after_step:
                    after_step()
                ev[i + 1].record()
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()
                torch.cuda.synchronize()
            if r == 0:
                first = ev[0].elapsed_time(ev[steps]) / 1e3
                first_launches = self.launches - l0
            per_step += [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
        if sampler:
            sampler.mark_end()
        return first, first_launches, per_step

    def time_e2e(self, steps, warmup, copy_only=False):
        """The same C-ABI call with HOST buffers: every step copies its pinned Q/K/V in and its output back inside the
        timed region.  The three phases run on three streams over two sets of device buffers, so the host->device copy
        of step i+1 and the device->host copy of step i-1 overlap the kernel of step i (what a caller that streams
        requests through the library would do); every step still moves all of its bytes.  copy_only: the same copies
        on the same streams without the kernel - the ceiling the host link sets for this pipeline."""
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
                if not copy_only:
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

    def check(self, **kw):
        torch.cuda.synchronize()
        return oracle_check(self.w, self.q, self.k, self.v, self.out, self.kv_len_host, **kw)


def step_stats(per_step_ms, sm_mhz=None):
    a = np.asarray(per_step_ms, np.float64)
    st = {"n": int(a.size), "median_ms": float(np.median(a)), "p95_ms": float(np.percentile(a, 95)), "min_ms": float(a.min())}
    if sm_mhz:
        st["median_ms_x_sm_mhz"] = float(np.median(a) * sm_mhz)
    return st


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
    times = []
    for _ in range(passes):
        t0 = time.perf_counter()
        O.sdpa(q, k, v, causal=w["causal"], kv_len=kv, faithful=True, threads=threads)
        times.append(time.perf_counter() - t0)
    ws = dict(w, B=B)
    return times, algorithmic_flops(ws, kv), algorithmic_bytes(ws, kv)


def host_threads():
    """All host cores this process may use (torchrun exports OMP_NUM_THREADS=1, which is not what is wanted here)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def run_reference_arm(args, w):
    """`--impl reference`: the reference's CPU attention path (C++ restatement; the .NET original cannot run here) on
    the whole workload, every step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    times, fl, by = cpu_reference_time(w, threads, args.warmup + args.steps)
    times = times[args.warmup:]
    ms = float(np.mean(times)) * 1e3
    value = (fl / 1e12) / (ms / 1e3) if w["kind"] == "prefill" else (by / 1e9) / (ms / 1e3)
    unit = "TFLOP/s" if w["kind"] == "prefill" else "GB/s"
    sample = "the whole workload (all %d batch entries) per step" % w["B"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": w["name"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "per_step": step_stats([t * 1e3 for t in times]), "gpu_launches": 0,
    }
    print(json.dumps(line))


def side_workload(key, local, pk, steps, dist=None, world=1):
    """One of the other baseline configurations, measured in the default run: kernel-only value, roofline, check."""
    w = WORKLOADS[key]
    r = Runner(w, local)
    secs, launches, per = r.time_steps(steps, 3, None, dist, repeats=2)
    if dist is not None:
        t = torch.tensor([secs], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t.item())
    fl, by = algorithmic_flops(w, r.kv_len_host), algorithmic_bytes(w, r.kv_len_host)
    tf = fl / 1e12 / (secs / steps)
    f32 = w.get("dtype") == "f32"
    # fp32 inputs run FFMA arithmetic: no measured peak exists for it, the nominal one is 148 SMs x 128 lanes x 2 x 1.965 GHz
    peak = 74.4 if f32 else pk["bf16"]
    obj = {"workload": w["name"], "value": tf * world, "unit": "TFLOP/s", "per_gpu": tf, "ms_per_step": secs / steps * 1e3,
           "steps": steps, "per_step": step_stats(per), "gpu_launches": launches, "tokens_per_s": w["B"] * w["Sq"] * world / (secs / steps),
           "roofline": {"bound": "fp32 FFMA (0.5 GFLOP, latency-bound; reported, not a target)" if f32 else "tensor",
                        "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                        "traffic": ncu_traffic(key, w, by), "traffic_unit": "bytes per launch (ncu)", "algorithmic": fl,
                        "algorithmic_unit": "FLOP per launch", "algorithmic_bytes": by,
                        "peak_source": "nominal fp32 FFMA" if f32 else pk["source"] + " (burst)"},
           "check": r.check()}
    del r
    torch.cuda.empty_cache()
    return obj


def long_context_job(local, rank, world, pk, steps, dist):
    """Configuration 5 as one job: B1, 64 query heads over 8 KV heads, S 32768, causal.  One GPU runs all of it; N ranks
    take `sharding.plan(N, 1, 64, 8)` - whole KV groups, so K/V are never duplicated and the computation needs no
    collective.  Timed twice: the kernel alone, and the same launch with gather_output = 1, i.e. followed on the same
    stream by the library's ncclAllGather that leaves the full [1, 64, S, D] output on every rank."""
    from aidotnet.tensors_b200 import nccl_util, sharding
    w = WORKLOADS["c5"]
    fl, by = algorithmic_flops(w), algorithmic_bytes(w)
    if world == 1:
        r = Runner(w, local)
        secs, launches, per = r.time_steps(steps, 2, None, None, repeats=1)
        tf = fl / 1e12 / (secs / steps)
        obj = {"workload": w["name"], "ranks": 1, "heads_per_rank": 64, "value": tf, "unit": "TFLOP/s", "per_gpu": tf,
               "ms_per_step": secs / steps * 1e3, "steps": steps, "per_step": step_stats(per), "gpu_launches": launches,
               "tokens_per_s": w["Sq"] / (secs / steps),
               "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16"], "unit": "TFLOP/s", "frac": tf / pk["bf16"],
                            "traffic": None, "algorithmic": fl, "algorithmic_unit": "FLOP per launch",
                            "peak_source": pk["source"] + " (burst)"},
               "gather": None, "check": r.check(h=37)}
        del r
        torch.cuda.empty_cache()
        return obj
    plan = sharding.plan(world, w["B"], w["Hq"], w["Hkv"])
    if not sharding.gatherable(plan):
        return {"workload": w["name"], "ranks": world, "skipped": "8 KV groups do not split evenly over %d ranks" % world}
    sh = plan[rank]
    comm = nccl_util.create_comm(rank, world)
    r = Runner(w, local, shard=(sh.head_begin, sh.head_count), nccl_comm=comm)
    secs, launches, per = r.time_steps(steps, 2, None, dist, repeats=1)
    gsecs, _, gper = r.time_steps(steps, 2, None, dist, repeats=1, gather=True)
    t = torch.tensor([secs, gsecs], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    secs, gsecs = float(t[0].item()), float(t[1].item())
    # every rank checks (a) a row block of its own shard against the CPU oracle and (b) a row block of a REMOTE rank's
    # heads in the gathered output against a local recomputation from regenerated inputs
    torch.cuda.synchronize()
    own = oracle_check(w, r.q, r.k, r.v, r.out, None, rows=32, h=sh.head_begin + sh.head_count - 1)
    other = plan[(rank + 1) % world]
    group = w["Hq"] // w["Hkv"]
    rows = 128
    r0 = w["Sq"] - rows
    qh = list(range(other.head_begin, other.head_begin + other.head_count))
    kh = list(range(other.head_begin // group, (other.head_begin + other.head_count) // group))
    dev = torch.device("cuda", local)
    qo, ko, vo, _ = make_inputs(w, dev, 0, qh, kh)
    from aidotnet.tensors_b200 import native as N
    h2 = N.Handle(device=local, qkv_dtype=N.BF16, head_dim=w["D"], num_q_heads=len(qh), num_kv_heads=len(kh), causal=True,
                  causal_bottom_right=False, causal_offset=r0)
    o2 = torch.empty((1, len(qh), rows, w["D"]), device=dev)
    q_rows = qo[:, :, r0:].contiguous()
    h2.launch(q=q_rows.data_ptr(), k=ko.data_ptr(), v=vo.data_ptr(), out=o2.data_ptr(), batch=1, seq_q=rows, seq_kv=w["Sk"],
              stream=r.stream)
    torch.cuda.synchronize()

    def remote_block_diff():
        return float((o2 - r.out[:, other.head_begin:other.head_begin + other.head_count, r0:]).abs().max())

    remote_diff = remote_block_diff()
    remote_ok = bool(remote_diff <= 1e-6)   # the same kernel on the same rows and keys: expected bit-identical
    # Third timing: the gather fused into the kernel.  Every rank maps the other ranks' output tensors (CUDA IPC) and
    # the epilogue stores each output tile to all of them; a one-element all-reduce behind every launch is the rank
    # synchronisation after which the gathered tensor is complete everywhere (inside the timed region).
    from aidotnet.tensors_b200.peer import PeerTensor
    fused = None
    fused_ok = False
    fused_diff = None
    try:
        r.out[:, other.head_begin:other.head_begin + other.head_count].zero_()   # what the NCCL gather left there
        torch.cuda.synchronize()
        dist.barrier()
        peers = PeerTensor(r.out, dist)
        token = torch.zeros(1, device="cuda")
        fsecs, _, fper = r.time_steps(steps, 2, None, dist, repeats=1, peer_out=peers.others,
                                      after_step=lambda: dist.all_reduce(token))
        # and without the per-step barrier (ranks synchronised only around the loop): what the stores themselves cost
        nsecs, _, _ = r.time_steps(steps, 2, None, dist, repeats=1, peer_out=peers.others)
        fused = [fsecs, fper, nsecs]
        torch.cuda.synchronize()
        dist.barrier()
        fused_diff = remote_block_diff()
        fused_ok = bool(fused_diff <= 1e-6)
        peers.close()
    except Exception as exc:   # the mapping is host plumbing outside the C ABI's hot path: report, do not fail the line
        fused = str(exc)
    # The same pair with a 16-bit output tensor (half the bytes to send): kernel alone, then fused.
    out16 = None
    if isinstance(fused, list):
        try:
            r16 = Runner(dict(w, out16=True), local, shard=(sh.head_begin, sh.head_count))
            k16, _, _ = r16.time_steps(steps, 2, None, dist, repeats=1)
            peers16 = PeerTensor(r16.out, dist)
            token16 = torch.zeros(1, device="cuda")
            f16, _, _ = r16.time_steps(steps, 2, None, dist, repeats=1, peer_out=peers16.others,
                                       after_step=lambda: dist.all_reduce(token16))
            torch.cuda.synchronize()
            dist.barrier()
            peers16.close()
            out16 = [k16, f16]
            del r16
        except Exception as exc:
            out16 = str(exc)
    t16 = torch.tensor(out16 if isinstance(out16, list) else [0.0, 0.0], device="cuda")
    dist.all_reduce(t16, op=dist.ReduceOp.MAX)
    t = torch.tensor([fused[0], fused[2]] if isinstance(fused, list) else [0.0, 0.0], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    fsecs, nsecs = float(t[0].item()), float(t[1].item())
    flags = torch.tensor([int(own["checked"]), int(remote_ok), int(fused_ok)], device="cuda")
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    h2.close()
    per_rank_fl = fl / world
    tf = per_rank_fl / 1e12 / (secs / steps)
    out_bytes = w["Hq"] * w["Sq"] * w["D"] * 4
    gather_ms = max(gsecs - secs, 0.0) / steps * 1e3
    recv = out_bytes * (world - 1) / world
    obj = {"workload": w["name"], "ranks": world, "heads_per_rank": sh.head_count, "value": tf * world, "unit": "TFLOP/s",
           "per_gpu": tf, "ms_per_step": secs / steps * 1e3, "steps": steps, "per_step": step_stats(per), "gpu_launches": launches,
           "scaling": "strong (one fixed job split over the ranks); efficiency = (N=1 ms_per_step) / (N x this ms_per_step)",
           "tokens_per_s": w["Sq"] / (secs / steps),
           "roofline": {"bound": "tensor", "achieved": tf, "peak": pk["bf16"], "unit": "TFLOP/s", "frac": tf / pk["bf16"],
                        "traffic": None, "algorithmic": per_rank_fl, "algorithmic_unit": "FLOP per launch and rank",
                        "peak_source": pk["source"] + " (burst)"},
           "gather": {"ms_per_step_with_gather": gsecs / steps * 1e3, "gather_ms": gather_ms, "per_step": step_stats(gper),
                      "bytes_received_per_rank": recv, "nvlink_gbs_per_rank": (recv / 1e9) / (gather_ms / 1e3) if gather_ms > 0 else None,
                      "nvlink_reference_gbs": 770.0, "collective": "ncclAllGather, in place, on the kernel's stream"},
           "fused_gather": ({"ms_per_step": fsecs / steps * 1e3, "extra_ms": max(fsecs - secs, 0.0) / steps * 1e3,
                             "ms_per_step_without_step_barrier": nsecs / steps * 1e3,
                             "per_step": step_stats(fused[1]),
                             "bytes_sent_per_rank": out_bytes / world * (world - 1),
                             "target_ms": max(per_rank_fl / (pk["bf16"] * 1e12), (out_bytes / world * (world - 1)) / 770e9) * 1e3,
                             "frac_of_target": max(per_rank_fl / (pk["bf16"] * 1e12), (out_bytes / world * (world - 1)) / 770e9) / (fsecs / steps),
                             "target": "the slower of FLOP / measured bf16 peak and bytes sent / 770 GB/s (measured peer copy)",
                             "how": "peer_out: the kernel's TMA stores write every tile to all ranks; one-element all-reduce per step as the rank barrier"}
                            if isinstance(fused, list) else {"unavailable": fused}),
           "fused_gather_out16": ({"kernel_ms_per_step": float(t16[0].item()) / steps * 1e3,
                                   "fused_ms_per_step": float(t16[1].item()) / steps * 1e3,
                                   "bytes_sent_per_rank": out_bytes / 2 / world * (world - 1)}
                                  if isinstance(out16, list) else {"unavailable": out16}),
           "fused_gather_ok": bool(flags[2].item() == 1), "fused_gather_max_abs_diff_rank0": fused_diff,
           "gather_ok": bool(flags[1].item() == 1), "gather_check": {"rows": [r0, r0 + rows], "remote_heads": [qh[0], qh[-1]], "max_abs_diff_rank0": remote_diff},
           "check": dict(own, all_ranks=bool(flags[0].item() == 1))}
    del r
    nccl_util.destroy_comm(comm)
    torch.cuda.empty_cache()
    return obj


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="skip the decode / c1 / c3 / c5 objects of the default run")
    ap.add_argument("--repeats", type=int, default=10, help="loops of --steps steps timed for the per-step statistics")
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

    runner = Runner(w, local, rank, args.decode_chunk)
    kvh = runner.kv_len_host
    fl, by = algorithmic_flops(w, kvh), algorithmic_bytes(w, kvh)
    secs, launches, per = runner.time_steps(args.steps, args.warmup, sampler, dist, repeats=max(1, args.repeats))
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
    check = runner.check()

    e2e_steps = max(3, min(args.steps, 20))
    # measured twice, around the copy-only run: with several ranks sharing the host's memory the first pass also pays
    # for bringing the pinned buffers in; the lower of the two (each the max over ranks) is reported, both are printed
    e2e_a, h2d, d2h = runner.time_e2e(e2e_steps, 2)
    copy_secs, _, _ = runner.time_e2e(e2e_steps, 2, copy_only=True)
    e2e_b, _, _ = runner.time_e2e(e2e_steps, 2)
    if dist is not None:
        t = torch.tensor([e2e_a, copy_secs, e2e_b], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_a, copy_secs, e2e_b = float(t[0].item()), float(t[1].item()), float(t[2].item())
    e2e_secs = min(e2e_a, e2e_b)
    e2e_value = (fl / 1e12 if prefill else by / 1e9) / (e2e_secs / e2e_steps) * world

    extra = {}
    if args.workload == "c2" and not args.no_decode:
        wd = WORKLOADS["c4"]
        rd = Runner(wd, local, rank)
        dsteps = max(10, args.steps)
        dsecs, dl, dper = rd.time_steps(dsteps, 3, None, dist, repeats=2)
        if dist is not None:
            t = torch.tensor([dsecs], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dsecs = float(t.item())
        dby = algorithmic_bytes(wd, rd.kv_len_host)
        gbs = dby / 1e9 / (dsecs / dsteps)
        extra["decode"] = {"workload": wd["name"], "value": gbs * world, "unit": "GB/s", "ms_per_step": dsecs / dsteps * 1e3,
                           "steps": dsteps, "per_step": step_stats(dper), "tokens_per_s": wd["B"] * world / (dsecs / dsteps), "gpu_launches": dl,
                           "roofline": {"bound": "hbm", "achieved": gbs, "peak": pk["hbm"], "unit": "GB/s",
                                        "frac": gbs / pk["hbm"], "traffic": ncu_traffic("c4", wd, dby),
                                        "traffic_unit": "bytes per launch (ncu, B=16 capture scaled by the bytes streamed)", "algorithmic": dby,
                                        "algorithmic_unit": "bytes per launch", "peak_source": pk["source"]},
                           "check": rd.check()}
        del rd
        torch.cuda.empty_cache()
        side_steps = max(5, min(args.steps, 20))
        for key in ("c1", "c3", "c5shard"):
            extra[key] = side_workload(key, local, pk, side_steps, dist, world)
        del runner.q, runner.k, runner.v
        torch.cuda.empty_cache()
        extra["c5"] = long_context_job(local, rank, world, pk, 5 if world == 1 else 10, dist)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = host_threads()
        # one warm-up pass, then two timed passes over the whole workload (all batch entries), as the reference arm does
        times, cfl, cby = cpu_reference_time(w, threads, 3)
        dt = float(np.mean(times[1:]))
        cpu = {"value": (cfl / 1e12 if prefill else cby / 1e9) / dt, "unit": "TFLOP/s" if prefill else "GB/s",
               "cores": threads, "kind": "port",
               "sample": "the whole workload (all %d batch entries), mean of two passes after one warm-up pass" % w["B"]}

    if rank == 0:
        mhz = clocks.get("sm_mhz") if clocks else None
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s" if prefill else "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": w.get("dtype", "bf16"), "data": "synthetic",
            "config": {"workload": w["name"], "per_gpu": "one copy of the workload per GPU (batch x head shard of an N-fold job)",
                       "l2": "inputs+outputs larger than the 126 MB L2; no flush",
                       "flop_convention": "4*D*visible(q,k) pairs (causal counted once)",
                       "inputs": "synth.py, seed 0xA1D00000 + configuration, streams Q/K/V = 0/1/2"},
            "per_gpu": per_gpu, "pct_of_measured_bf16_peak": (100.0 * per_gpu / pk["bf16"]) if prefill else None,
            "tokens_per_s": w["B"] * w["Sq"] * world / per_step,
            "per_step": dict(step_stats(per, mhz), loops=max(1, args.repeats), note="value and ms_per_step are the first loop of --steps steps"),
            "roofline": {"bound": "tensor" if prefill else "hbm", "achieved": per_gpu, "peak": peak,
                         "unit": "TFLOP/s" if prefill else "GB/s", "frac": per_gpu / peak,
                         "traffic": ncu_traffic(args.workload, w, by), "traffic_unit": "bytes per launch (ncu)",
                         "algorithmic": fl if prefill else by, "algorithmic_unit": "FLOP per launch" if prefill else "bytes per launch",
                         "algorithmic_bytes": by, "peak_source": pk["source"] + (" (burst)" if prefill else "")},
            "check": check, "checked": bool(check["checked"]),
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s" if prefill else "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_secs / e2e_steps * 1e3,
                    "ms_per_step_runs": [e2e_a / e2e_steps * 1e3, e2e_b / e2e_steps * 1e3],
                    "copy_only_ms": copy_secs / e2e_steps * 1e3, "frac_of_copy_only": copy_secs / e2e_secs,
                    "pipeline": "host->device copy, kernel and device->host copy on three streams over two buffer sets; "
                                "copy_only_ms = the same copies without the kernel (max over ranks)"},
            "gpu_launches": launches, "clocks": clocks,
        }
        line.update(extra)
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()

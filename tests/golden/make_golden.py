"""Generates ``tests/golden/sdpa_golden.npz``.

The reference project stores no golden vectors for attention: its tests recompute scalar references
in-line.  This script replays those test cases (same shapes; same inputs wherever the reference gives
them as closed-form sequences, our own seeded inputs where it used ``System.Random``) through an
independent float64 numpy formulation of softmax attention and stores inputs plus expected outputs.
Both the CPU oracle and the CUDA path are checked against the stored arrays.

Reference test files mirrored (paths relative to the reference project root):
  tests/AiDotNet.Tensors.Tests/Engines/BatchMatMulAndAttentionTests.cs:287-317   (softcap closed form)
  tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/GpuCpuConsistencyTests.cs:895-1061 (cross-attention,
      logit softcap, full boolean mask; inputs are arithmetic sequences)
  tests/AiDotNet.Tensors.Tests/Engines/SdpaMaskBroadcastTests.cs:33-143          (broadcast causal masks)
  tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/RopeGqaOpenClTests.cs:200-279   (GQA, top-left causal)
  tests/AiDotNet.Tensors.Tests/Engines/DirectGpu/FlashDecodeCudaTests.cs:43-126  (decode shape list)
  tests/AiDotNet.Tensors.Tests/Engines/FlashAttentionBiasTests.cs                (3-D / 4-D additive bias, LSE)

Run:  python tests/golden/make_golden.py
"""
import os

import numpy as np


def attention_f64(q, k, v, scale, *, keep=None, bias=None, softcap=0.0, want_lse=False):
    """q [B,Hq,Sq,D], k/v [B,Hkv,Sk,D]; keep/bias broadcastable to [B,Hq,Sq,Sk]. float64 throughout."""
    q, k, v = (np.asarray(x, dtype=np.float64) for x in (q, k, v))
    B, Hq, Sq, _ = q.shape
    Hkv = k.shape[1]
    g = Hq // Hkv
    kk = np.repeat(k, g, axis=1)
    vv = np.repeat(v, g, axis=1)
    s = np.einsum("bhqd,bhkd->bhqk", q, kk) * float(scale)
    if softcap > 0:
        s = softcap * np.tanh(s / softcap)
    if bias is not None:
        s = s + np.asarray(bias, dtype=np.float64)
    if keep is not None:
        s = np.where(np.broadcast_to(keep, s.shape), s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    dead = ~np.isfinite(m)
    e = np.exp(s - np.where(dead, 0.0, m))
    e = np.where(dead, 0.0, e)
    tot = e.sum(axis=-1, keepdims=True)
    w = np.where(tot > 0, e / np.where(tot > 0, tot, 1.0), 0.0)
    out = np.einsum("bhqk,bhkd->bhqd", w, vv)
    lse = np.where(dead[..., 0], -np.inf, m[..., 0] + np.log(np.where(tot[..., 0] > 0, tot[..., 0], 1.0)))
    if want_lse:
        return out, lse, w
    return out, None, w


def seq(n, a, b):
    # the reference builds these in float: (float)a + (float)b * i
    return (np.float32(a) + np.float32(b) * np.arange(n, dtype=np.float32)).astype(np.float32)


def main():
    g = {}

    # --- softcap closed form ------------------------------------------------------------------------
    q = np.array([10.0], np.float32).reshape(1, 1, 1, 1)
    k = np.array([1.0, -1.0], np.float32).reshape(1, 1, 2, 1)
    v = np.array([3.0, 7.0], np.float32).reshape(1, 1, 2, 1)
    cap = 2.0
    t = cap * np.tanh(np.array([10.0, -10.0]) / cap)
    e = np.exp(t - t.max())
    w = e / e.sum()
    g.update(softcap_q=q, softcap_k=k, softcap_v=v, softcap_w=w, softcap_out=np.array([(w * [3.0, 7.0]).sum()]))
    out, _, w2 = attention_f64(q, k, v, 1.0, softcap=cap)
    assert np.allclose(w2.ravel(), w) and np.allclose(out.ravel(), g["softcap_out"])

    # --- GpuCpuConsistency: cross attention / softcap / full bool mask --------------------------------
    B, H, Sq, Sk, D = 2, 2, 2, 3, 3
    q = seq(B * H * Sq * D, -0.2, 0.03).reshape(B, H, Sq, D)
    k = seq(B * H * Sk * D, 0.5, -0.025).reshape(B, H, Sk, D)
    v = seq(B * H * Sk * D, -0.1, 0.04).reshape(B, H, Sk, D)
    out, _, w = attention_f64(q, k, v, 0.75)
    g.update(cross_q=q, cross_k=k, cross_v=v, cross_out=out, cross_w=w)
    mask = np.array([1, 0, 1, 0, 1, 1, 1, 1, 0, 1, 0, 0, 0, 1, 1, 1, 1, 0, 1, 0, 0, 0, 1, 0], np.uint8).reshape(B, H, Sq, Sk)
    out, _, w = attention_f64(q, k, v, 0.75, keep=mask.astype(bool))
    g.update(boolmask_mask=mask, boolmask_out=out, boolmask_w=w)
    q2 = seq(B * H * Sq * D, -0.9, 0.17).reshape(B, H, Sq, D)
    k2 = seq(B * H * Sk * D, 1.3, -0.11).reshape(B, H, Sk, D)
    v2 = seq(B * H * Sk * D, -0.4, 0.09).reshape(B, H, Sk, D)
    out, _, w = attention_f64(q2, k2, v2, 1.5, softcap=2.0)
    g.update(capcross_q=q2, capcross_k=k2, capcross_v=v2, capcross_out=out, capcross_w=w)

    # --- SdpaMaskBroadcast ---------------------------------------------------------------------------
    B, H, S, D = 2, 3, 5, 4
    i = np.arange(B * H * S * D, dtype=np.float64)
    base = np.sin(i * 0.7) * 1.5 + 0.25 * ((i.astype(np.int64) % 7) - 3)
    q = base.astype(np.float32).reshape(B, H, S, D)
    k = (base * 0.5 + 0.1).astype(np.float32).reshape(B, H, S, D)
    v = (base * -0.3 + 0.2).astype(np.float32).reshape(B, H, S, D)
    causal = np.tril(np.ones((S, S), bool))[None, None]
    out, _, _ = attention_f64(q, k, v, 1.0 / np.sqrt(D), keep=causal)
    out_nomask, _, _ = attention_f64(q, k, v, 1.0 / np.sqrt(D))
    g.update(bcast_q=q, bcast_k=k, bcast_v=v, bcast_out=out, bcast_out_nomask=out_nomask)

    # --- GQA (B1 Hq6 Hkv2 S5 D8), top-left causal as the in-test GqaReference ---------------------------
    rng = np.random.Generator(np.random.Philox(23))
    q = rng.uniform(-1, 1, (1, 6, 5, 8)).astype(np.float32)
    k = rng.uniform(-1, 1, (1, 2, 5, 8)).astype(np.float32)
    v = rng.uniform(-1, 1, (1, 2, 5, 8)).astype(np.float32)
    sc = np.float32(1.0) / np.sqrt(np.float32(8))
    out_c, _, _ = attention_f64(q, k, v, sc, keep=np.tril(np.ones((5, 5), bool))[None, None])
    out_n, _, _ = attention_f64(q, k, v, sc)
    g.update(gqa_q=q, gqa_k=k, gqa_v=v, gqa_out_causal=out_c, gqa_out_plain=out_n)

    # --- decode shape list: (heads, kvHeads, headDim, seqLen); K/V stored [seqLen, kvHeads, D] -----------
    shapes = [(4, 4, 64, 40), (8, 8, 32, 100), (4, 4, 64, 7), (4, 4, 64, 64), (6, 6, 48, 77), (8, 2, 64, 50), (8, 1, 64, 40)]
    g["decode_shapes"] = np.array(shapes, np.int64)
    for n, (h, hk, d, L) in enumerate(shapes):
        rng = np.random.Generator(np.random.Philox(0xFDE + h + hk + L))
        kk = rng.uniform(-1, 1, (L, hk, d)).astype(np.float32)
        vv = rng.uniform(-1, 1, (L, hk, d)).astype(np.float32)
        qq = rng.uniform(-1, 1, (h, d)).astype(np.float32)
        out, _, _ = attention_f64(qq[None, :, None, :], kk.transpose(1, 0, 2)[None], vv.transpose(1, 0, 2)[None],
                                  np.float32(1.0) / np.sqrt(np.float32(d)))
        g[f"decode{n}_q"], g[f"decode{n}_k"], g[f"decode{n}_v"] = qq, kk, vv
        g[f"decode{n}_out"] = out[0, :, 0, :]

    # --- FlashAttention additive bias, 3-D (batch-broadcast) and 4-D, with LSE, top-left causal ---------
    rng = np.random.Generator(np.random.Philox(77))
    B, H, S, D = 2, 3, 9, 16
    q = rng.standard_normal((B, H, S, D)).astype(np.float32)
    k = rng.standard_normal((B, H, S, D)).astype(np.float32)
    v = rng.standard_normal((B, H, S, D)).astype(np.float32)
    bias3 = rng.standard_normal((H, S, S)).astype(np.float32)
    bias4 = rng.standard_normal((B, H, S, S)).astype(np.float32)
    sc = 1.0 / np.sqrt(D)
    tri = np.tril(np.ones((S, S), bool))[None, None]
    o3, l3, _ = attention_f64(q, k, v, sc, bias=bias3[None], want_lse=True)
    o4, l4, _ = attention_f64(q, k, v, sc, bias=bias4, keep=tri, want_lse=True)
    g.update(bias_q=q, bias_k=k, bias_v=v, bias3=bias3, bias4=bias4, bias3_out=o3, bias3_lse=l3,
             bias4c_out=o4, bias4c_lse=l4)

    # --- bfloat16 conversion vectors (BFloat16.cs:65-84) ----------------------------------------------
    bits = np.array([0x00000000, 0x80000000, 0x3F800000, 0x3F808000, 0x3F818000, 0x3F807FFF, 0x3F808001,
                     0x7F7FFFFF, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001, 0xFFA00000, 0x00000001,
                     0x00008000, 0x00018000, 0x3EAAAAAB, 0xC2F6E979], np.uint32)
    exp = []
    for b in bits:
        b = int(b)
        if (b & 0x7F800000) == 0x7F800000 and (b & 0x007FFFFF):
            exp.append(((b >> 16) | 0x0040) & 0xFFFF)
        else:
            exp.append(((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF)
    g.update(bf16_in_bits=bits, bf16_out_bits=np.array(exp, np.uint16))

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sdpa_golden.npz")
    np.savez_compressed(path, **g)
    print("wrote", path, os.path.getsize(path), "bytes;", len(g), "arrays")


if __name__ == "__main__":
    main()

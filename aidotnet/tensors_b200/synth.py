"""Seeded synthetic inputs shared by the parity tests and the benchmark.

One counter-based generator: Philox keyed by ``(0xA1D00000 + config, stream, batch entry, head)``, so that any head of
any tensor of a configuration can be produced on its own (a rank that checks another rank's shard regenerates exactly
that head) and in parallel.  Streams: 0 = Q, 1 = K, 2 = V, 3 = sequence lengths, 4+ = extra tensors of a test.
Values are N(0,1) * scale in fp32, rounded to the requested dtype (round to nearest even, what
``NumericOperations/BFloat16.cs:65-84`` of the reference does); 16-bit configurations use scale 0.5, fp32 ones 1.0, the
distributions the baseline configurations name.  No public dataset is involved.
"""
from __future__ import annotations

import concurrent.futures
import os
from typing import Sequence

import numpy as np
import torch

SEED_BASE = 0xA1D00000
STREAM_Q, STREAM_K, STREAM_V, STREAM_LEN = 0, 1, 2, 3
TORCH_DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def _bitgen(config: int, stream: int, b: int, h: int) -> np.random.Philox:
    return np.random.Philox(key=[SEED_BASE + config, (stream << 40) | (b << 20) | h])


def head(config: int, stream: int, b: int, h: int, rows: int, d: int, scale: float = 0.5) -> np.ndarray:
    """fp32 ``[rows, d]`` values of head ``h`` of batch entry ``b`` (before rounding to the tensor's dtype)."""
    g = np.random.Generator(_bitgen(config, stream, b, h))
    return g.standard_normal((rows, d), dtype=np.float32) * np.float32(scale)


def tensor(config: int, stream: int, shape: Sequence[int], dtype: str = "bf16", scale: float = 0.5,
           heads: Sequence[int] | None = None, pin: bool = False) -> torch.Tensor:
    """CPU tensor ``[B, H, S, D]`` of ``dtype``.  ``heads``: the global head index of each of the H heads (default
    0..H-1), for a tensor that holds only a shard of the heads."""
    B, H, S, D = shape
    heads = list(range(H)) if heads is None else list(heads)
    assert len(heads) == H
    out = torch.empty((B, H, S, D), dtype=TORCH_DT[dtype])
    if pin:
        out = out.pin_memory()

    def fill(bh):
        b, j = divmod(bh, H)
        out[b, j].copy_(torch.from_numpy(head(config, stream, b, heads[j], S, D, scale)))

    workers = max(1, min(16, len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else 8))
    if B * H == 1:
        fill(0)
    else:
        with concurrent.futures.ThreadPoolExecutor(workers) as ex:
            list(ex.map(fill, range(B * H)))
    return out


def lengths(config: int, batch: int, lo: int, hi: int) -> np.ndarray:
    """int32 ``[batch]`` sequence lengths, uniform in [lo, hi]."""
    g = np.random.Generator(_bitgen(config, STREAM_LEN, 0, 0))
    return g.integers(lo, hi + 1, batch).astype(np.int32)

"""B200-native fused scaled-dot-product-attention forward behind the reference's GPU-backend attention operator.

``native``  — ctypes binding of the C ABI (include/aidn_sdpa.h)
``backend`` — mirror of the reference's ``CudaBackend`` attention methods on top of it
``sharding`` — head-shard planning for multi-GPU runs
"""
from . import native  # noqa: F401

__all__ = ["native"]

"""Peer mappings of a tensor between the ranks of one node (one process per GPU), for ``aidn_sdpa_args.peer_out``.

Host-side plumbing only: every rank exports the CUDA IPC handle of the allocation that holds its tensor
(``aidn_peer_export``), the handles travel through ``torch.distributed`` (any backend: they are 64 bytes and an
offset), and every rank maps the others' allocations (``aidn_peer_open``).  The reference's counterpart is the
communicator bootstrap of ``NcclComm`` (``CUDA/NcclComm.cs:43-97``): a few bytes exchanged once, outside the hot path.
"""
from __future__ import annotations

import ctypes
from typing import List

import torch

from . import native as N


class PeerTensor:
    """The same tensor on every rank; ``pointers[r]`` is rank r's copy as seen from this rank (own rank: local)."""

    def __init__(self, tensor: torch.Tensor, dist) -> None:
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("PeerTensor needs a contiguous CUDA tensor")
        self.tensor = tensor
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        lib = N.load()
        # Every rank takes part in both exchanges whatever happens to it locally, and all ranks then agree on the
        # outcome: a rank that raised on its own would leave the others waiting in a collective.
        mine, problem = None, None
        try:
            handle = (ctypes.c_ubyte * 64)()
            offset = ctypes.c_int64(0)
            N.check(lib.aidn_peer_export(ctypes.c_void_p(tensor.data_ptr()), handle, ctypes.byref(offset)))
            mine = (bytes(handle), int(offset.value))
        except N.AidnError as exc:
            problem = f"rank {self.rank}: {exc}"
        everyone: List = [None] * self.world
        dist.all_gather_object(everyone, mine)
        self._bases: List[int] = []
        self.pointers: List[int] = []
        if problem is None and all(e is not None for e in everyone):
            try:
                for r, (hbytes, off) in enumerate(everyone):
                    if r == self.rank:
                        self.pointers.append(tensor.data_ptr())
                        continue
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(hbytes)
                    base = ctypes.c_void_p()
                    N.check(lib.aidn_peer_open(buf, ctypes.byref(base)))
                    self._bases.append(base.value)
                    self.pointers.append(base.value + off)
            except N.AidnError as exc:
                problem = f"rank {self.rank}: {exc}"
        elif problem is None:
            problem = f"rank {self.rank}: another rank could not export its tensor"
        verdicts: List = [None] * self.world
        dist.all_gather_object(verdicts, problem)
        failed = [v for v in verdicts if v is not None]
        if failed:
            self.close()
            raise RuntimeError("peer mapping failed: " + "; ".join(failed))

    @property
    def others(self) -> List[int]:
        """Pointers of all ranks but this one: what ``peer_out`` takes."""
        return [p for r, p in enumerate(self.pointers) if r != self.rank]

    def close(self) -> None:
        lib = N.load()
        for base in self._bases:
            lib.aidn_peer_close(ctypes.c_void_p(base))
        self._bases = []

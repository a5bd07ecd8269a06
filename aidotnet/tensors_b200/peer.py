"""Peer mappings of a tensor between the ranks of one node (one process per GPU), for ``aidn_sdpa_args.peer_out``.

Host-side plumbing only: every rank exports the CUDA IPC handle of the allocation that holds its tensor
(``aidn_peer_export``), the handles travel through ``torch.distributed`` (any backend: they are 64 bytes and an
offset), and every rank maps the others' allocations (``aidn_peer_open``).  The reference's counterpart is the
communicator bootstrap of ``NcclComm`` (``CUDA/NcclComm.cs:43-97``): a few bytes exchanged once, outside the hot path.
"""
from __future__ import annotations

import ctypes
from typing import Callable, List, Tuple

import torch

from . import native as N


def exchange_mappings(dist, local_pointer: int, export: Callable[[int], Tuple[bytes, int]],
                      open_mapping: Callable[[bytes], int], close_mapping: Callable[[int], None]) -> Tuple[List[int], List[int]]:
    """The exchange itself, independent of CUDA: returns (pointers by rank, bases this rank has mapped).

    Every rank takes part in both collectives whatever happens to it locally, and all ranks then agree on the outcome:
    a rank that raised on its own would leave the others waiting in a collective.  On failure everything this rank
    mapped is unmapped again and every rank raises the same ``RuntimeError``."""
    rank, world = dist.get_rank(), dist.get_world_size()
    mine, problem = None, None
    try:
        mine = export(local_pointer)
    except Exception as exc:   # noqa: BLE001 - whatever the export raised is reported by all ranks
        problem = f"rank {rank}: {exc}"
    everyone: List = [None] * world
    dist.all_gather_object(everyone, mine)
    bases: List[int] = []
    pointers: List[int] = []
    if problem is None and all(e is not None for e in everyone):
        try:
            for r, (handle, offset) in enumerate(everyone):
                if r == rank:
                    pointers.append(local_pointer)
                    continue
                base = open_mapping(handle)
                bases.append(base)
                pointers.append(base + offset)
        except Exception as exc:   # noqa: BLE001
            problem = f"rank {rank}: {exc}"
    elif problem is None:
        problem = f"rank {rank}: another rank could not export its tensor"
    verdicts: List = [None] * world
    dist.all_gather_object(verdicts, problem)
    failed = [v for v in verdicts if v is not None]
    if failed:
        for base in bases:
            close_mapping(base)
        raise RuntimeError("peer mapping failed: " + "; ".join(failed))
    return pointers, bases


class PeerTensor:
    """The same tensor on every rank; ``pointers[r]`` is rank r's copy as seen from this rank (own rank: local)."""

    def __init__(self, tensor: torch.Tensor, dist) -> None:
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise ValueError("PeerTensor needs a contiguous CUDA tensor")
        self.tensor = tensor
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        lib = N.load()

        def export(ptr: int) -> Tuple[bytes, int]:
            handle = (ctypes.c_ubyte * 64)()
            offset = ctypes.c_int64(0)
            N.check(lib.aidn_peer_export(ctypes.c_void_p(ptr), handle, ctypes.byref(offset)))
            return bytes(handle), int(offset.value)

        def open_mapping(handle: bytes) -> int:
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(handle)
            base = ctypes.c_void_p()
            N.check(lib.aidn_peer_open(buf, ctypes.byref(base)))
            return int(base.value)

        self._bases: List[int] = []
        self.pointers, self._bases = exchange_mappings(dist, tensor.data_ptr(), export, open_mapping, self._close_one)

    @staticmethod
    def _close_one(base: int) -> None:
        N.load().aidn_peer_close(ctypes.c_void_p(base))

    @property
    def others(self) -> List[int]:
        """Pointers of all ranks but this one: what ``peer_out`` takes."""
        return [p for r, p in enumerate(self.pointers) if r != self.rank]

    def close(self) -> None:
        for base in self._bases:
            self._close_one(base)
        self._bases = []

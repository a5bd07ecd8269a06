"""Creates raw ``ncclComm_t`` handles for the optional all-gather of the attention output.

The library's ``desc.nccl_comm`` takes the communicator the reference would create with
``NcclComm.InitRank`` (``src/AiDotNet.Tensors/Engines/DirectGpu/CUDA/NcclComm.cs:84-96``).  ``torch.distributed``
does not expose its communicators, so the multi-GPU harness makes its own through ctypes on the same
``libnccl.so.2`` that torch has loaded, exchanging the unique id over an existing (gloo or nccl) process group.
"""
from __future__ import annotations

import ctypes
from typing import Optional


class _UniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_ubyte * 128)]


_nccl: Optional[ctypes.CDLL] = None


def _lib() -> ctypes.CDLL:
    global _nccl
    if _nccl is None:
        import torch  # noqa: F401  (loads the bundled libnccl.so.2 first so that the soname resolves to it)
        lib = ctypes.CDLL("libnccl.so.2")
        lib.ncclGetUniqueId.argtypes = [ctypes.POINTER(_UniqueId)]
        lib.ncclGetUniqueId.restype = ctypes.c_int
        lib.ncclCommInitRank.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int, _UniqueId, ctypes.c_int]
        lib.ncclCommInitRank.restype = ctypes.c_int
        lib.ncclCommDestroy.argtypes = [ctypes.c_void_p]
        lib.ncclCommDestroy.restype = ctypes.c_int
        lib.ncclGetErrorString.argtypes = [ctypes.c_int]
        lib.ncclGetErrorString.restype = ctypes.c_char_p
        _nccl = lib
    return _nccl


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: {_lib().ncclGetErrorString(rc).decode()}")


def create_comm(rank: int, world: int, group=None) -> int:
    """Collective over ``group`` (default process group): returns this rank's ``ncclComm_t`` as an int.
    The CUDA device of the calling rank must already be current."""
    import torch.distributed as dist
    uid = _UniqueId()
    if rank == 0:
        _check(_lib().ncclGetUniqueId(ctypes.byref(uid)), "ncclGetUniqueId")
    payload = [ctypes.string_at(ctypes.byref(uid), 128) if rank == 0 else None]
    dist.broadcast_object_list(payload, src=0, group=group)
    ctypes.memmove(ctypes.byref(uid), payload[0], 128)
    comm = ctypes.c_void_p()
    _check(_lib().ncclCommInitRank(ctypes.byref(comm), world, uid, rank), "ncclCommInitRank")
    return int(comm.value)


def destroy_comm(comm: int) -> None:
    _check(_lib().ncclCommDestroy(ctypes.c_void_p(comm)), "ncclCommDestroy")

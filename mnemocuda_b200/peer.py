"""Host side of the push collectives (mb200_comm_* / mb200_push_* in include/mnemo_b200.h).

One process per GPU. Each rank lets the library allocate its receive buffer and export a CUDA IPC
handle; the handles are exchanged through torch.distributed (any backend: they are 64 opaque bytes);
the library opens the peers' buffers. After that a collective is one kernel launch per rank that
stores this rank's piece into every peer's buffer over NVLink and waits for the peers' pieces.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import kernels as K


def exchange_handles(local_handle: bytes, group=None) -> list[bytes]:
    """All ranks' 64-byte handles in rank order (torch.distributed object all-gather)."""
    import torch.distributed as dist
    if len(local_handle) != 64:
        raise ValueError("a CUDA IPC handle is 64 bytes")
    world = dist.get_world_size(group)
    out: list = [None] * world
    dist.all_gather_object(out, bytes(local_handle), group=group)
    if any(h is None or len(h) != 64 for h in out):
        raise RuntimeError("handle exchange failed")
    return [bytes(h) for h in out]


class PeerComm:
    """Receive buffers of all ranks mapped into this process; all-reduce / all-gather of small fp32 vectors."""

    def __init__(self, rank: int, world: int, max_floats: int, group=None):
        self.rank, self.world, self.max_floats = rank, world, max_floats
        lib = _lib.lib()
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        K._check(lib.mb200_comm_alloc(world, max_floats, C.byref(ptr), handle), "mb200_comm_alloc")
        self._local = ptr.value
        if world > 1:
            handles = exchange_handles(handle.raw, group)
            blob = b"".join(handles)
        else:
            blob = handle.raw
        comm = C.c_void_p()
        K._check(lib.mb200_comm_create(rank, world, max_floats, self._local, blob, C.byref(comm)), "mb200_comm_create")
        self._comm = comm.value
        if world > 1:
            import torch.distributed as dist
            dist.barrier(group)  # every rank has mapped every buffer before anyone pushes

    def allreduce(self, x: torch.Tensor, out: torch.Tensor, stream=None) -> None:
        """out = sum over ranks of x (fp32, numel a multiple of 4; out may be x)."""
        K._check(_lib.lib().mb200_push_allreduce(self._comm, K._f32(x), K._f32(out), x.numel(), K._stream(stream)),
                 "mb200_push_allreduce")

    def allgather(self, x: torch.Tensor, out: torch.Tensor, stream=None) -> None:
        """out[q * n : (q + 1) * n] = rank q's x."""
        if out.numel() != self.world * x.numel():
            raise ValueError("out must hold world pieces")
        K._check(_lib.lib().mb200_push_allgather(self._comm, K._f32(x), K._f32(out), x.numel(), K._stream(stream)),
                 "mb200_push_allgather")

    def close(self) -> None:
        if self._comm:
            torch.cuda.synchronize()
            _lib.lib().mb200_comm_destroy(self._comm, 1)
            self._comm = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

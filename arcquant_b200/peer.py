"""Receive slots in peer memory for the row-parallel projections of a tensor-parallel group.

Every rank owns a block of device memory, [world, rows_per_rank, cols] bf16, and maps the blocks of all
other ranks of the same machine into its own address space (CUDA IPC handles, exchanged through the
process group).  Slot s of rank d's block is where rank s's GEMM stores the rows of its partial result
that rank d owns (`ops.matmul_scatter`): the tiles cross NVLink while the GEMM is still running, and what
is left of the reduce-scatter is a barrier and one pass over local memory (`ops.sum_partials`).

The reference has no counterpart (its layers run on one GPU).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


class _DeviceBlock:
    """Lets torch view a raw device allocation (the CUDA array interface, 16-bit words)."""

    def __init__(self, ptr: int, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i2", "data": (int(ptr), False), "version": 3}


class PeerSlots:
    def __init__(self, rows_per_rank: int, cols: int, rank: int, world: int, group=None, device=None):
        import torch.distributed as dist

        if world > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        self.rank, self.world, self.rows, self.cols = rank, world, rows_per_rank, cols
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.slot_bytes = rows_per_rank * cols * 2
        self._lib = _lib.load()
        self._own = C.c_void_p()
        self._opened: list[int] = []
        # Every rank takes part in every exchange below whatever happened to it before, and all ranks raise
        # together: a rank that failed alone would leave the others waiting in a collective.
        with torch.cuda.device(self.device):
            err, mine = None, None
            try:
                _lib.check(self._lib.arcq_peer_alloc(self.slot_bytes * world, C.byref(self._own)), "peer slots: allocation")
                handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
                _lib.check(self._lib.arcq_peer_export(self._own, handle), "peer slots: export")
                mine = bytes(handle.raw)
            except Exception as exc:       # reported to the group below
                err = repr(exc)
            handles = [mine]
            if world > 1:
                handles = [None] * world
                dist.all_gather_object(handles, mine, group=group)
            self.base = []
            if err is None and all(h is not None for h in handles):
                try:
                    for d in range(world):
                        if d == rank:
                            self.base.append(int(self._own.value))
                            continue
                        ptr = C.c_void_p()
                        _lib.check(self._lib.arcq_peer_open(handles[d], C.byref(ptr)), f"peer slots: opening rank {d}'s block")
                        self._opened.append(int(ptr.value))
                        self.base.append(int(ptr.value))
                except Exception as exc:
                    err = repr(exc)
            elif err is None:
                err = "a peer could not allocate or export its block"
            errs = [err]
            if world > 1:
                errs = [None] * world
                dist.all_gather_object(errs, err, group=group)
            if any(e is not None for e in errs):
                self.close()
                raise RuntimeError("peer slots unavailable: " + "; ".join(f"rank {i}: {e}" for i, e in enumerate(errs) if e))
        # where this rank's rows for owner d go, and where the partials this rank owns arrive
        self.dests = [self.base[d] + rank * self.slot_bytes for d in range(world)]
        self.sources = [self.base[rank] + s * self.slot_bytes for s in range(world)]

    def local(self) -> torch.Tensor:
        """This rank's block as a bf16 tensor [world, rows_per_rank, cols] (a view, for tests and debugging)."""
        t = torch.as_tensor(_DeviceBlock(self._own.value, (self.world, self.rows, self.cols)), device=self.device)
        return t.view(torch.bfloat16)

    def close(self) -> None:
        """Unmap the peers' blocks and free this rank's (after a barrier of the group: no peer may still be
        writing)."""
        if self._lib is None:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for p in self._opened:
                self._lib.arcq_peer_close(C.c_void_p(p))
            self._opened = []
            if self._own:
                self._lib.arcq_peer_free(self._own)
                self._own = C.c_void_p()
        self._lib = None

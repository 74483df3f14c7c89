"""Peer memory for the collectives of a tensor-parallel group on one NVLink machine.

Every rank owns blocks of device memory (allocated by the library, outside any framework's pool) and maps
the blocks of all other ranks into its own address space (CUDA IPC handles, exchanged through the process
group).  Three uses:

* `PeerSlots`: [world, rows_per_rank, cols] bf16 receive slots.  Slot s of rank d's block is where rank s's
  GEMM stores the rows of its partial result that rank d owns (`ops.matmul_scatter`): the tiles cross NVLink
  while the GEMM is still running, and what is left of the reduce-scatter is a barrier and one pass over local
  memory (`ops.sum_partials`).
* `PeerGathered`: the gathered packed codes and block scales of a sequence-parallel activation: every rank
  quantizes its token rows into its own copy and stores them into every other rank's
  (`ops.rmsnorm_quantize_x_multi`), so the all-gather is over when those stores and a barrier are.
* `PeerBarrier`: that barrier - flags in peer memory, one small kernel per rank (`ops.peer_barrier`).

The reference has no counterpart (its layers run on one GPU).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib, ops


class _DeviceBlock:
    """Lets torch view a raw device allocation (the CUDA array interface, bytes)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False), "version": 3}


class PeerBlock:
    """`nbytes` of zeroed device memory on every rank of the group, each rank's block mapped by all others:
    `base[d]` is the address of rank d's block in this process."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None, device=None):
        import torch.distributed as dist

        if world > 8:
            raise ValueError("at most 8 ranks (one NVLink domain)")
        self.rank, self.world, self.nbytes = rank, world, int(nbytes)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._lib = None
        self._own = C.c_void_p()
        self._opened: list[int] = []
        self.base: list[int] = []
        # Every rank takes part in every exchange below whatever happened to it before, and all ranks raise
        # together: a rank that failed alone would leave the others waiting in a collective.
        err, mine = None, None
        try:
            mine = self._make_own()
        except Exception as exc:       # reported to the group below
            err = repr(exc)
        handles = [mine]
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
        if err is None and all(h is not None for h in handles):
            try:
                for d in range(world):
                    self.base.append(int(self._own.value) if d == rank else self._open(handles[d], d))
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
            raise RuntimeError("peer memory unavailable: " + "; ".join(f"rank {i}: {e}" for i, e in enumerate(errs) if e))

    # the two device-side steps (a test replaces them with fakes to exercise the failure paths on CPU)
    def _make_own(self) -> bytes:
        """Allocate and zero this rank's block; the handle the peers open it with."""
        self._lib = _lib.load()
        with torch.cuda.device(self.device):
            _lib.check(self._lib.arcq_peer_alloc(self.nbytes, C.byref(self._own)), "peer block: allocation")
            self.local_bytes().zero_()
            torch.cuda.synchronize()        # zeroed before any peer can learn the address
            handle = C.create_string_buffer(_lib.PEER_HANDLE_BYTES)
            _lib.check(self._lib.arcq_peer_export(self._own, handle), "peer block: export")
        return bytes(handle.raw)

    def _open(self, handle: bytes, owner: int) -> int:
        ptr = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self._lib.arcq_peer_open(handle, C.byref(ptr)), f"peer block: opening rank {owner}'s")
        self._opened.append(int(ptr.value))
        return int(ptr.value)

    def local_bytes(self) -> torch.Tensor:
        """This rank's block as a uint8 tensor (a view)."""
        return torch.as_tensor(_DeviceBlock(self._own.value, self.nbytes), device=self.device)

    def close(self) -> None:
        """Unmap the peers' blocks and free this rank's (after a barrier of the group: no peer may still be
        using them)."""
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


class PeerSlots(PeerBlock):
    def __init__(self, rows_per_rank: int, cols: int, rank: int, world: int, group=None, device=None):
        self.rows, self.cols = rows_per_rank, cols
        self.slot_bytes = rows_per_rank * cols * 2
        super().__init__(self.slot_bytes * world, rank, world, group, device)
        # where this rank's rows for owner d go, and where the partials this rank owns arrive
        self.dests = [self.base[d] + rank * self.slot_bytes for d in range(world)]
        self.sources = [self.base[rank] + s * self.slot_bytes for s in range(world)]

    def local(self) -> torch.Tensor:
        """This rank's slots as a bf16 tensor [world, rows_per_rank, cols] (a view)."""
        return self.local_bytes().view(torch.bfloat16).reshape(self.world, self.rows, self.cols)


class PeerGathered(PeerBlock):
    """Packed codes [rows_per_rank * world, k_eff / 2] and their scale buffer on every rank; rank r's quantizer
    writes rows [r * rows_per_rank, (r + 1) * rows_per_rank) of every rank's copy."""

    def __init__(self, rows_per_rank: int, k_eff: int, rank: int, world: int, group=None, device=None):
        if rows_per_rank % 128:
            raise ValueError("token shards must be whole 128-row scale tiles")
        total = rows_per_rank * world
        self.q_bytes = (total * (k_eff // 2) + 255) // 256 * 256
        self.sf_bytes = ops.sf_bytes(total, k_eff)
        super().__init__(self.q_bytes + self.sf_bytes, rank, world, group, device)
        tile = ((k_eff // 16 + 3) // 4) * 512
        q_off = rank * rows_per_rank * (k_eff // 2)
        sf_off = self.q_bytes + rank * (rows_per_rank // 128) * tile
        # this rank's copy first: the quantizer's primary output
        order = [rank] + [d for d in range(world) if d != rank]
        self.q_dests = [self.base[d] + q_off for d in order]
        self.sf_dests = [self.base[d] + sf_off for d in order]
        mine = self.local_bytes()
        self.q = mine[:total * (k_eff // 2)].reshape(total, k_eff // 2)
        self.sf = mine[self.q_bytes:self.q_bytes + self.sf_bytes]


class PeerBarrier(PeerBlock):
    def __init__(self, rank: int, world: int, group=None, device=None):
        super().__init__(256, rank, world, group, device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)

    def __call__(self) -> None:
        ops.peer_barrier(self.base, self.rank, self.counter)

"""Host-side bookkeeping for running the quantized linears tensor-parallel (one process per GPU).

Column-parallel linears (qkv, gate_up) shard N: every rank quantizes the full, replicated
activation with the layer's global channel order, so nothing changes for the quantizer.

Row-parallel linears (o_proj, down_proj) shard K.  The reference's channel order is a single
permutation over all K input channels and cannot be applied across ranks: a rank that owns the
slice [start, stop) can only reorder inside it.  Each rank therefore gets
  * a local order: the entries of the global order that fall in its slice, kept in their global
    (ascending-importance) sequence, re-based to the slice - so its locally most important channels
    are last, as the kernels expect;
  * a local number of augmented residual channels KE_r: the global KE split evenly, rounded up to
    a multiple of 64 so that K_local + KE_r stays a multiple of 64 (what the GEMM needs).
The partial products are summed with one all-reduce.  Results differ slightly between TP degrees
(different 16-channel groups, different residual sets); each is a valid ARC quantization.
"""
from __future__ import annotations

import torch


def shard_range(n: int, tp: int, rank: int):
    if n % tp:
        raise ValueError(f"{n} does not split over {tp} ranks")
    step = n // tp
    return rank * step, (rank + 1) * step


def local_reorder_index(global_index: torch.Tensor, start: int, stop: int) -> torch.Tensor:
    """int16 [stop-start]: global order restricted to [start, stop), re-based."""
    g = global_index.to(torch.int64).cpu()
    keep = g[(g >= start) & (g < stop)] - start
    if keep.numel() != stop - start:
        raise ValueError("global_index is not a permutation")
    return keep.to(torch.int16)


def shard_select_num(select_num: int, tp: int, k_local: int) -> int:
    """Residual channels kept by one K shard (multiple of 64, at most k_local)."""
    if select_num == 0:
        return 0
    if k_local % 64:
        raise ValueError("K shards must be multiples of 64 channels")
    per = -(-select_num // tp)
    ke = max(64, -(-per // 64) * 64)
    return min(ke, k_local)


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the tensor-parallel group (NCCL on GPUs, gloo in the CPU tests)."""
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t

"""Mixtral-architecture sparse-MoE block on ARC-NVFP4 expert linears, expert-parallel.

Semantics of the reference block (model/qMixtralLayer.py:435-473, 524-543 of ARCQuant): bf16 router,
fp32 softmax, top-2, renormalised routing weights; every expert quantizes its own batch of tokens
with its own per-call global scale and its own channel orders (w1/w3 share one, w2 has another);
outputs are scaled by the routing weight and summed per token.  What replaces the reference's
serial Python loop over all experts on one device:

  * the routed rows of all local experts form ONE padded buffer, expert after expert, every expert's
    run starting at a multiple of 256 rows.  Where the runs start and how long they are is computed
    with tensor operations and stays on the device: no count ever travels to the host, nothing in
    `dispatch` / `combine` synchronises;
  * one absmax launch, one quantizer launch and one GEMM launch per projection serve all experts
    (`ops.absmax_grouped`, `ops.reorder_quantize_x_grouped`, `ops.matmul_grouped`): per-expert global
    scale, channel order and weight matrix are picked on the device from the run a row belongs to.
    w1 and w3 of an expert are one fused [gate;up] matrix over the shared quantized activation;
  * tokens and experts are sharded over the expert-parallel group; rows travel to the rank that owns
    their expert with one all-to-all of fixed-capacity blocks (bf16 rows - the experts' channel orders
    differ, so rows cannot be quantized at the source) and come back with a second one.  The counts
    travel as a small all-to-all of their own and are consumed on the device.

The dispatcher is plain torch + torch.distributed, so its bookkeeping runs (and is tested) on CPU
with gloo; the expert arithmetic needs the CUDA library.
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import ops
from .qlinear import NVFP4_reorder_quantize_x

TILE = 256   # rows: every expert's run starts on a tile of the grouped GEMM


@dataclass
class MoEConfig:
    hidden: int = 4096
    ffn: int = 14336
    n_experts: int = 8
    top_k: int = 2
    select_num: int = 128


def route_top_k(x: torch.Tensor, router_w: torch.Tensor, top_k: int):
    """(expert ids [T,k], weights [T,k] in x.dtype), as model/qMixtralLayer.py:441-447."""
    logits = F.linear(x, router_w)
    probs = F.softmax(logits, dim=1, dtype=torch.float)
    w, ids = torch.topk(probs, top_k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return ids, w.to(x.dtype)


def _counts(ids: torch.Tensor, n: int) -> torch.Tensor:
    """int64 [n]: how often each of 0..n-1 occurs (values >= n are ignored).  No host synchronisation
    (torch.bincount would need the maximum on the host)."""
    return (ids.unsqueeze(1) == torch.arange(n, device=ids.device).unsqueeze(0)).sum(0)


def padded_layout(slot_expert: torch.Tensor, n_groups: int, tile: int = TILE):
    """Places `n` slots (slot i belongs to expert slot_expert[i], or to nobody if that is >= n_groups) into
    a padded buffer: expert after expert, every run starting at a multiple of `tile` rows, slots of one
    expert in their original order.  Returns
      dest       int64 [n]: padded row of every slot (`rows_bound` for slots of nobody),
      row_slot   int64 [rows_bound]: slot held by every padded row (0 for padding rows),
      groups     int32 [2 * n_groups]: first row and number of rows of every run,
      tile_group int32 [rows_bound / tile]: run of every tile, -1 for tiles without rows,
      rows_bound int: size of the padded buffer - the only number the host knows, a worst-case bound."""
    n, dev = slot_expert.numel(), slot_expert.device
    rows_bound = (n + tile - 1) // tile * tile + n_groups * tile
    if slot_expert.is_cuda and n_groups <= 64 and n <= (1 << 20):       # one small launch does all of it
        dest, row_slot, groups, tile_group = ops.moe_layout(slot_expert.to(torch.int64).contiguous(), n_groups, tile,
                                                            rows_bound)
        return dest, row_slot, groups, tile_group, rows_bound
    order = torch.argsort(slot_expert, stable=True)
    sorted_e = slot_expert[order]
    counts = _counts(slot_expert, n_groups)
    pad = (counts + tile - 1) // tile * tile
    offs = torch.cumsum(pad, 0) - pad
    starts = torch.cumsum(counts, 0) - counts
    se = sorted_e.clamp(max=n_groups - 1)
    ar = torch.arange(n, device=dev)
    dest_sorted = torch.where(sorted_e < n_groups, offs[se] + ar - starts[se], torch.full_like(ar, rows_bound))
    dest = torch.empty_like(dest_sorted)
    dest[order] = dest_sorted
    row_slot = torch.zeros(rows_bound + 1, dtype=torch.int64, device=dev)
    row_slot[dest] = ar
    groups = torch.cat([offs, counts]).to(torch.int32)
    tile_start = torch.arange(rows_bound // tile, device=dev) * tile
    e_of = (torch.searchsorted(offs, tile_start, right=True) - 1).clamp(min=0)
    tile_group = torch.where(tile_start < (offs + counts)[e_of], e_of, torch.full_like(e_of, -1)).to(torch.int32)
    return dest, row_slot[:rows_bound], groups, tile_group, rows_bound


@dataclass
class RoutedBatch:
    """Device-resident description of the rows the local experts work on."""
    src: torch.Tensor          # [*, hidden]: the rows are read from here (this rank's tokens, or the receive buffer)
    row_map: torch.Tensor      # int32 [rows_bound]: row of `src` held by every padded row (0 for padding)
    groups: torch.Tensor       # int32 [2 * local experts]
    tile_group: torch.Tensor   # int32 [rows_bound / TILE]
    rows_bound: int
    n_local: int               # local experts
    state: dict                # what `combine` needs

    def rows(self) -> torch.Tensor:
        """The padded buffer materialised: [rows_bound, hidden] (padding rows hold a copy of row 0)."""
        return self.src.index_select(0, self.row_map.long())

    def row_expert(self) -> torch.Tensor:
        """int64 [rows_bound]: local expert of every padded row, -1 for padding."""
        e = self.tile_group.long().repeat_interleave(TILE)
        ends = (self.groups[:self.n_local] + self.groups[self.n_local:]).long()
        r = torch.arange(self.rows_bound, device=e.device)
        return torch.where((e >= 0) & (r < ends[e.clamp(min=0)]), e, torch.full_like(e, -1))


class ExpertParallelDispatcher:
    """Moves token rows to the ranks that own their experts and back (all-to-all of fixed-capacity
    blocks), and lays the rows out by local expert - without a host synchronisation.

    capacity: rows one rank may send to one peer (the same number on every rank).  Default: the largest
    number of routed copies any rank holds at the first call (agreed once with an all-reduce and kept) -
    the worst case, every copy of a rank going to one peer, so nothing can overflow; pass it explicitly
    when later calls may be larger.
    capacity_factor: instead of the worst case, `capacity_factor` times the even share (copies / ranks,
    rounded up to 128 rows): the all-to-alls then move that much less padding.  Copies beyond a block's
    capacity are dropped (they contribute zero) and `overflowed()` reports it - the caller then repeats the
    step with a dispatcher of larger capacity."""

    def __init__(self, n_experts: int, ep_rank: int = 0, ep_size: int = 1, group=None, capacity: int | None = None,
                 capacity_factor: float | None = None):
        if n_experts % ep_size:
            raise ValueError("experts must split evenly over the expert-parallel group")
        self.E, self.rank, self.ep, self.group = n_experts, ep_rank, ep_size, group
        self.e_local = n_experts // ep_size
        self.capacity = capacity
        self.capacity_factor = capacity_factor
        self._overflow = None          # device flag, sticky

    def overflowed(self) -> bool:
        """True if any call so far dropped copies for lack of capacity (reads the device: synchronises)."""
        return self._overflow is not None and bool(self._overflow.item())

    def _agree_capacity(self, n_copies: int, device) -> int:
        import torch.distributed as dist

        if self.capacity is None:            # first call only: one small all-reduce and one host read
            t = torch.tensor([n_copies], dtype=torch.int64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            self.capacity = int(t.item())
            if self.capacity_factor is not None:
                share = -(-self.capacity // self.ep)
                self.capacity = min(self.capacity, -(-int(share * self.capacity_factor) // 128) * 128)
                n_copies = 0          # (a factor below the worst case can overflow: flagged, not raised)
        if self.capacity_factor is None and n_copies > self.capacity:
            raise ValueError(f"{n_copies} routed copies exceed the dispatcher's capacity {self.capacity}; "
                             "construct it with capacity=<largest number of copies per rank>")
        return self.capacity

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor) -> RoutedBatch:
        """x [T,H]: this rank's tokens; ids [T,k]: global expert of every copy."""
        import torch.distributed as dist

        T, k = ids.shape
        flat = ids.reshape(-1)
        if self.ep == 1:
            dest, row_slot, groups, tile_group, rows_bound = padded_layout(flat, self.e_local)
            row_map = torch.div(row_slot, k, rounding_mode="floor").to(torch.int32)
            return RoutedBatch(x, row_map, groups, tile_group, rows_bound, self.e_local,
                               dict(T=T, k=k, copy_row=dest))
        n = flat.numel()
        cap = self._agree_capacity(n, x.device)
        # send side: copies sorted by (destination rank, expert), block s of `cap` rows goes to rank s
        order = torch.argsort(flat, stable=True)
        sorted_e = flat[order]
        counts = _counts(flat, self.E)
        per_rank = counts.reshape(self.ep, self.e_local).sum(1)
        rank_start = torch.cumsum(per_rank, 0) - per_rank
        dst = torch.div(sorted_e, self.e_local, rounding_mode="floor")
        in_block = torch.arange(n, device=x.device) - rank_start[dst]
        kept = in_block < cap                                     # (always, at worst-case capacity)
        if self.capacity_factor is not None:
            over = (~kept).any()
            self._overflow = over if self._overflow is None else (self._overflow | over)
            counts = _counts(torch.where(kept, sorted_e, torch.full_like(sorted_e, self.E)), self.E)
        dummy = self.ep * cap                                      # where dropped copies point: a row of zeros
        send_slot_sorted = torch.where(kept, dst * cap + in_block, torch.full_like(in_block, dummy))
        copy_slot = torch.empty_like(send_slot_sorted)
        copy_slot[order] = send_slot_sorted                       # slot of every copy, in copy order
        slot_token = torch.zeros(self.ep * cap + 1, dtype=torch.int64, device=x.device)
        slot_token[send_slot_sorted] = torch.div(order, k, rounding_mode="floor")
        send = x.index_select(0, slot_token[:dummy])
        recv_counts = torch.empty_like(counts)
        dist.all_to_all_single(recv_counts, counts, group=self.group)      # [source rank, local expert]
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=self.group)               # equal blocks: no sizes needed
        # receive side: slot i of block s holds a row of the local expert whose cumulative count first exceeds i
        cs = torch.cumsum(recv_counts.reshape(self.ep, self.e_local), 1)   # [ep, e_local]
        i = torch.arange(cap, device=x.device)
        slot_expert = (i.reshape(1, cap, 1) >= cs.reshape(self.ep, 1, self.e_local)).sum(-1).reshape(-1)
        dest, row_slot, groups, tile_group, rows_bound = padded_layout(slot_expert, self.e_local)
        return RoutedBatch(recv, row_slot.to(torch.int32), groups, tile_group, rows_bound, self.e_local,
                           dict(T=T, k=k, copy_row=copy_slot, slot_row=dest.clamp(max=rows_bound - 1)))

    def combine(self, y_rows: torch.Tensor, weights: torch.Tensor, batch: RoutedBatch) -> torch.Tensor:
        """y_rows [rows_bound, H]: expert outputs in the padded layout.  -> [T,H] weighted sums."""
        import torch.distributed as dist

        st = batch.state
        T, k = st["T"], st["k"]
        if self.ep > 1:
            back = y_rows.index_select(0, st["slot_row"])                  # slot order again (padding: any row)
            ret = back.new_zeros((back.shape[0] + 1, back.shape[1]))       # last row: what dropped copies read
            dist.all_to_all_single(ret[:-1], back, group=self.group)
        else:
            ret = y_rows
        pos = st["copy_row"].reshape(T, k)                                  # row of `ret` holding copy j of token t
        if ret.is_cuda and ret.dtype == torch.bfloat16:
            return ops.moe_combine(ret.contiguous(), pos.to(torch.int32).contiguous(),
                                   weights.to(torch.bfloat16).contiguous())
        out = torch.zeros((T, ret.shape[1]), dtype=ret.dtype, device=ret.device)
        for j in range(k):
            out += ret.index_select(0, pos[:, j]) * weights[:, j:j + 1].to(ret.dtype)
        return out


class MoEPeerBuffers:
    """What one rank of `PeerExpertDispatcher` needs: the addresses of every rank's receive buffer
    [ep * cap, hidden] bf16, slot table [ep * cap] int64 and return buffer [ep * cap + 1, hidden] bf16 (its last row
    stays zero: what dropped copies read), this rank's own three as tensors, and a barrier of the group."""

    def __init__(self, cap: int, hidden: int, rank: int, ep: int, group=None, device=None):
        from .peer import PeerBarrier, PeerBlock

        self.cap, self.hidden, self.rank, self.ep = cap, hidden, rank, ep
        self._blocks = []
        try:     # all four blocks or none (a failure is raised on every rank together, see peer.PeerBlock)
            for nbytes in (ep * cap * hidden * 2, ep * cap * 8, (ep * cap + 1) * hidden * 2):
                self._blocks.append(PeerBlock(nbytes, rank, ep, group, device))
            self.barrier = PeerBarrier(rank, ep, group, device)
        except Exception:
            for b in self._blocks:
                b.close()
            raise
        self.recv_base, self.meta_base, self.ret_base = (b.base for b in self._blocks)
        self.recv = self._blocks[0].local_bytes().view(torch.bfloat16).reshape(ep * cap, hidden)
        self.meta = self._blocks[1].local_bytes().view(torch.int64)
        self.ret = self._blocks[2].local_bytes().view(torch.bfloat16).reshape(ep * cap + 1, hidden)

    def close(self) -> None:
        for b in self._blocks + [self.barrier]:
            b.close()

    @staticmethod
    def local_group(cap: int, hidden: int, ep: int, device) -> list:
        """`ep` buffer sets in one process, each seeing the others' tensors as its peers (no barrier): all ranks
        of a group emulated on one GPU, phase by phase."""
        out = []
        for r in range(ep):
            b = MoEPeerBuffers.__new__(MoEPeerBuffers)
            b.cap, b.hidden, b.rank, b.ep = cap, hidden, r, ep
            b.recv = torch.zeros((ep * cap, hidden), dtype=torch.bfloat16, device=device)
            b.meta = torch.zeros((ep * cap,), dtype=torch.int64, device=device)
            b.ret = torch.zeros((ep * cap + 1, hidden), dtype=torch.bfloat16, device=device)
            b.barrier = lambda: None
            b._blocks = []
            out.append(b)
        for b in out:
            b.recv_base = [o.recv.data_ptr() for o in out]
            b.meta_base = [o.meta.data_ptr() for o in out]
            b.ret_base = [o.ret.data_ptr() for o in out]
        return out


class PeerExpertDispatcher(ExpertParallelDispatcher):
    """`ExpertParallelDispatcher` without collectives: every rank stores its routed rows (and the local expert of
    each) straight into the memory of the ranks that own the experts, and the experts' output rows straight
    back; a barrier through flags in peer memory follows each direction.  Three small launches and a barrier
    replace the sort / scatter / gather / all-to-all sequence of the parent on the way out, one launch and a
    barrier on the way back.  The capacity of a block is fixed at construction."""

    def __init__(self, n_experts: int, buffers: MoEPeerBuffers):
        super().__init__(n_experts, buffers.rank, buffers.ep, None, buffers.cap, None)
        self.buf = buffers
        self._overflow = torch.zeros(1, dtype=torch.int32, device=buffers.recv.device)

    def overflowed(self) -> bool:
        return bool(self._overflow.item())

    # the two halves of `dispatch` (separate so that a test can run all ranks of a group in one process)
    def send(self, x: torch.Tensor, ids: torch.Tensor) -> dict:
        b = self.buf
        T, k = ids.shape
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        slot = ops.ep_send_layout(flat, self.e_local, self.ep, b.cap, self.rank, b.meta_base, self._overflow)
        ops.ep_rows(x, None, k, T, slot, flat.numel(), b.cap, self.ep, self.rank, b.recv_base)
        return dict(T=T, k=k, copy_row=slot)

    def receive(self, state: dict) -> RoutedBatch:
        b = self.buf
        dest, row_slot, groups, tile_group, rows_bound = padded_layout(b.meta, self.e_local)
        state = dict(state, slot_row=dest, rows_bound=rows_bound)
        return RoutedBatch(b.recv, row_slot.to(torch.int32), groups, tile_group, rows_bound, self.e_local, state)

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor) -> RoutedBatch:
        state = self.send(x, ids)
        self.buf.barrier()          # every rank's rows and slot tables have arrived
        return self.receive(state)

    # and of `combine`
    def send_back(self, y_rows: torch.Tensor, batch: RoutedBatch) -> None:
        b, st = self.buf, batch.state
        ops.ep_rows(y_rows, st["slot_row"].to(torch.int32), 1, st["rows_bound"], None, self.ep * b.cap, b.cap, self.ep,
                    self.rank, b.ret_base)

    def finish(self, weights: torch.Tensor, batch: RoutedBatch) -> torch.Tensor:
        st = batch.state
        pos = st["copy_row"].reshape(st["T"], st["k"])
        return ops.moe_combine(self.buf.ret, pos.contiguous(), weights.to(torch.bfloat16).contiguous())

    def combine(self, y_rows: torch.Tensor, weights: torch.Tensor, batch: RoutedBatch) -> torch.Tensor:
        self.send_back(y_rows, batch)
        self.buf.barrier()          # every expert's rows have come home
        return self.finish(weights, batch)


def random_moe_weights(cfg: MoEConfig, seed: int = 0, std: float = 0.02):
    g = torch.Generator().manual_seed(seed)

    def w(n, k):
        return (torch.randn(n, k, generator=g) * std).to(torch.bfloat16)

    out = {"router": (torch.randn(cfg.n_experts, cfg.hidden, generator=g)).to(torch.bfloat16) * 0.05, "experts": []}
    for _ in range(cfg.n_experts):
        out["experts"].append({
            "w1": w(cfg.ffn, cfg.hidden), "w3": w(cfg.ffn, cfg.hidden), "w2": w(cfg.hidden, cfg.ffn),
            "w1_index": torch.randperm(cfg.hidden, generator=g).to(torch.int16),
            "w2_index": torch.randperm(cfg.ffn, generator=g).to(torch.int16),
        })
    return out


def _stack(linears):
    """Packed weights of several linears of one shape behind one another: (codes [E*N, K/2], scales, global
    scales [E], channel orders [E, KQ]).  The linears' own buffers become views of the stacked ones."""
    n, kb = linears[0].W.shape
    k_eff = kb * 2
    span = (n // 128) * ((k_eff // 16 + 3) // 4) * 512          # bytes of the scale tiles of one matrix
    W = torch.cat([l.W for l in linears], 0)
    SF = torch.cat([l.SFW[:span] for l in linears], 0)
    for e, l in enumerate(linears):
        l.W = W[e * n:(e + 1) * n]
        l.SFW = SF[e * span:(e + 1) * span]
    scale = torch.stack([l.scale for l in linears]).contiguous()
    index = torch.stack([l.index for l in linears]).contiguous()
    return W, SF, scale, index


class QMixtralMoEBlockEP(torch.nn.Module):
    def __init__(self, cfg: MoEConfig, weights: dict, ep_rank: int = 0, ep_size: int = 1, group=None, device="cuda",
                 capacity: int | None = None, capacity_factor: float | None = None):
        super().__init__()
        from .llama_layer import PackedLinear

        self.cfg = cfg
        self.dispatcher = ExpertParallelDispatcher(cfg.n_experts, ep_rank, ep_size, group, capacity, capacity_factor)
        dev = torch.device(device)
        self.router = weights["router"].to(dev)
        self.experts = []
        e0 = ep_rank * self.dispatcher.e_local
        # gate (w1) and up (w3) interleaved in blocks of 128 channels: SiLU(gate) * up and its maximum come out of
        # the GEMM's epilogue (same bits as the GEMM followed by a SiLU pass over [rows, 2 * ffn])
        self.fuse_swiglu = cfg.ffn % 128 == 0
        for e in range(e0, e0 + self.dispatcher.e_local):
            ew = weights["experts"][e]
            wgu = ops.interleave_gate_up(ew["w1"], ew["w3"]) if self.fuse_swiglu else torch.cat([ew["w1"], ew["w3"]], 0)
            gu = PackedLinear(wgu.to(dev), ew["w1_index"], cfg.select_num)
            dn = PackedLinear(ew["w2"].to(dev).contiguous(), ew["w2_index"], cfg.select_num)
            self.experts.append((gu, dn))
        # one launch per projection for all local experts needs whole scale tiles per expert (N % 128)
        # and row widths the grouped quantizer covers (512..16384 channels)
        ok_width = lambda kq: kq % 16 == 0 and 512 <= kq <= 16384
        self.grouped = (2 * cfg.ffn) % 128 == 0 and cfg.hidden % 128 == 0 and ok_width(cfg.hidden) and ok_width(cfg.ffn)
        if self.grouped:
            self.gu_W, self.gu_SF, self.gu_scale, self.gu_index = _stack([gu for gu, _ in self.experts])
            self.dn_W, self.dn_SF, self.dn_scale, self.dn_index = _stack([dn for _, dn in self.experts])

    def peer_capacity(self, tokens_per_rank: int, capacity_factor: float | None = 2.0) -> int:
        """Rows one rank may send to one peer: all its copies (worst case), or `capacity_factor` times the even
        share, rounded up to 128."""
        copies = tokens_per_rank * self.cfg.top_k
        if capacity_factor is None:
            return copies
        share = -(-copies // self.dispatcher.ep)
        return min(copies, -(-int(share * capacity_factor) // 128) * 128)

    def enable_peer_dispatch(self, tokens_per_rank: int, capacity_factor: float | None = 2.0) -> None:
        """From now on rows travel to the experts' ranks and back as stores into peer memory
        (`PeerExpertDispatcher`) instead of all-to-all collectives.  Collective call; the ranks share one machine."""
        d = self.dispatcher
        if d.ep == 1:
            return
        buf = MoEPeerBuffers(self.peer_capacity(tokens_per_rank, capacity_factor), self.cfg.hidden, d.rank, d.ep, d.group,
                             self.router.device)
        self.dispatcher = PeerExpertDispatcher(self.cfg.n_experts, buf)
        self.dispatcher.group = d.group

    def disable_peer_dispatch(self) -> None:
        d = self.dispatcher
        if isinstance(d, PeerExpertDispatcher):
            d.buf.close()
            self.dispatcher = ExpertParallelDispatcher(self.cfg.n_experts, d.rank, d.ep, d.group, d.capacity, None)

    @torch.no_grad()
    def expert_forward_grouped(self, batch: RoutedBatch) -> torch.Tensor:
        """All local experts in five launches: [rows_bound, hidden] in the padded layout of `batch`."""
        cfg, E = self.cfg, self.dispatcher.e_local
        ke = cfg.select_num
        s1 = ops.absmax_grouped(batch.src, batch.row_map, batch.groups, E) / (448.0 * 6.0)   # per-expert scales
        a, sfa = ops.reorder_quantize_x_grouped(batch.src, batch.row_map, s1, self.gu_index, batch.groups,
                                                batch.rows_bound, ke)
        if self.fuse_swiglu:        # SiLU * up and the per-expert maxima in the GEMM's epilogue
            act, amax2 = ops.matmul_grouped_swiglu(a, self.gu_W, sfa, self.gu_SF, batch.tile_group, batch.groups, E,
                                                   2 * cfg.ffn, s1, self.gu_scale)
        else:
            h = ops.matmul_grouped(a, self.gu_W, sfa, self.gu_SF, batch.tile_group, E, 2 * cfg.ffn, s1, self.gu_scale)
            if cfg.ffn % 256 == 0:  # SiLU * up and the per-expert maxima in one pass, empty tiles skipped
                act, amax2 = ops.silu_mul_grouped(h, batch.tile_group, batch.groups, E)
            else:
                act, _ = ops.silu_mul(h, with_amax=False)
                amax2 = ops.absmax_grouped(act, None, batch.groups, E)
        s2 = amax2 / (448.0 * 6.0)
        b, sfb = ops.reorder_quantize_x_grouped(act, None, s2, self.dn_index, batch.groups, batch.rows_bound, ke)
        return ops.matmul_grouped(b, self.dn_W, sfb, self.dn_SF, batch.tile_group, E, cfg.hidden, s2, self.dn_scale)

    n_streams = 4   # per-expert path: a few streams hide the launch gaps of the experts' small kernels

    @torch.no_grad()
    def expert_forward(self, rows: torch.Tensor, per_expert) -> torch.Tensor:
        """The reference's organisation - one quantize / GEMM sequence per expert on `per_expert[e]`
        consecutive rows - kept as the yardstick of the grouped path (needs the counts on the host)."""
        out = torch.empty_like(rows)
        start = 0
        use_streams = rows.is_cuda and self.n_streams > 1 and len(self.experts) > 1
        if use_streams:
            if not hasattr(self, "_streams"):
                self._streams = [torch.cuda.Stream(rows.device) for _ in range(self.n_streams)]
            cur = torch.cuda.current_stream(rows.device)
            for s in self._streams:
                s.wait_stream(cur)
        for i, ((gu, dn), n) in enumerate(zip(self.experts, per_expert)):
            if n == 0:
                continue
            ctx = torch.cuda.stream(self._streams[i % self.n_streams]) if use_streams else contextlib.nullcontext()
            with ctx:
                xb = rows[start:start + n]
                a, sfa, sx = NVFP4_reorder_quantize_x(xb, gu.index, gu.select_num, mode=16)
                if self.fuse_swiglu:
                    act, amax = ops.matmul_swiglu(a, gu.W, sfa, gu.SFW, sx, gu.scale)
                else:
                    act, amax = ops.silu_mul(gu.gemm(a, sfa, sx))
                b, sfb, sa = NVFP4_reorder_quantize_x(act, dn.index, dn.select_num, mode=16, amax=amax)
                out[start:start + n] = dn.gemm(b, sfb, sa)
            start += n
        if use_streams:
            for s in self._streams:
                cur.wait_stream(s)
        return out

    @torch.no_grad()
    def expert_forward_padded(self, batch: RoutedBatch) -> torch.Tensor:
        """The per-expert path on a padded batch (reads the run sizes on the host): what
        `expert_forward_grouped` must reproduce."""
        E = self.dispatcher.e_local
        g = batch.groups.tolist()
        rows = batch.rows()
        out = torch.zeros_like(rows)
        for e in range(E):
            off, cnt = g[e], g[E + e]
            if cnt:
                out[off:off + cnt] = self.expert_forward(rows[off:off + cnt].contiguous(), [0] * e + [cnt])
        return out

    @torch.no_grad()
    def forward(self, x: torch.Tensor, routing=None) -> torch.Tensor:
        """x: this rank's tokens [T, hidden] (bf16).  routing: optional precomputed
        (expert ids [T,k], weights [T,k]) - otherwise the block's own router decides."""
        ids, w = routing if routing is not None else route_top_k(x, self.router, self.cfg.top_k)
        batch = self.dispatcher.dispatch(x, ids)
        y = self.expert_forward_grouped(batch) if self.grouped else self.expert_forward_padded(batch)
        return self.dispatcher.combine(y, w, batch)

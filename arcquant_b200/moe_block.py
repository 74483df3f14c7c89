"""Mixtral-architecture sparse-MoE block on ARC-NVFP4 expert linears, expert-parallel.

Semantics of the reference block (model/qMixtralLayer.py:435-473, 524-543 of ARCQuant): bf16 router,
fp32 softmax, top-2, renormalised routing weights; every expert quantizes its own batch of tokens
with its own per-call global scale and its own channel orders (w1/w3 share one, w2 has another);
outputs are scaled by the routing weight and summed per token.  What replaces the reference's
serial Python loop over all experts on one device:

  * tokens and experts are sharded over the expert-parallel group; rows travel to the rank that
    owns their expert with one all-to-all (bf16 rows - the experts' channel orders differ, so rows
    cannot be quantized at the source), and come back with a second one;
  * w1 and w3 of an expert are one fused [gate;up] GEMM over the shared quantized activation.

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


class ExpertParallelDispatcher:
    """Moves token rows to the ranks that own their experts and back (all-to-all), and groups the
    received rows by local expert."""

    def __init__(self, n_experts: int, ep_rank: int = 0, ep_size: int = 1, group=None):
        if n_experts % ep_size:
            raise ValueError("experts must split evenly over the expert-parallel group")
        self.E, self.rank, self.ep, self.group = n_experts, ep_rank, ep_size, group
        self.e_local = n_experts // ep_size

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor):
        """x [T,H], ids [T,k]  ->  (rows grouped by local expert [R,H], rows per local expert (list),
        state for `combine`)."""
        import torch.distributed as dist

        T, k = ids.shape
        flat = ids.reshape(-1)
        order = torch.argsort(flat, stable=True)               # (token,slot) pairs sorted by expert
        token_of = torch.div(order, k, rounding_mode="floor")
        send_rows = x.index_select(0, token_of)
        counts = torch.bincount(flat, minlength=self.E)        # rows per expert, this rank's tokens
        if self.ep == 1:
            state = dict(order=order, T=T, k=k, regroup=None, send_splits=None, recv_splits=None)
            return send_rows, counts.tolist(), state
        recv_counts = torch.empty_like(counts)                 # [src rank, local expert] flattened
        dist.all_to_all_single(recv_counts, counts, group=self.group)
        send_splits = counts.reshape(self.ep, self.e_local).sum(1).tolist()
        rc = recv_counts.reshape(self.ep, self.e_local)
        recv_splits = rc.sum(1).tolist()
        recv_rows = x.new_empty((int(sum(recv_splits)), x.shape[1]))
        dist.all_to_all_single(recv_rows, send_rows, recv_splits, send_splits, group=self.group)
        # received rows are ordered (src rank, expert); regroup to (expert, src rank)
        rc_cpu = rc.cpu()
        starts = torch.zeros(self.ep * self.e_local + 1, dtype=torch.int64)
        starts[1:] = torch.cumsum(rc_cpu.reshape(-1), 0)
        pieces = []
        for e in range(self.e_local):
            for s in range(self.ep):
                j = s * self.e_local + e
                pieces.append(torch.arange(int(starts[j]), int(starts[j + 1])))
        regroup = torch.cat(pieces).to(x.device) if pieces else torch.zeros(0, dtype=torch.int64, device=x.device)
        rows = recv_rows.index_select(0, regroup)
        per_expert = rc_cpu.sum(0).tolist()
        state = dict(order=order, T=T, k=k, regroup=regroup, send_splits=send_splits, recv_splits=recv_splits)
        return rows, per_expert, state

    def combine(self, y_rows: torch.Tensor, weights: torch.Tensor, state) -> torch.Tensor:
        """y_rows: expert outputs in the grouped order `dispatch` returned.  -> [T,H] weighted sums."""
        import torch.distributed as dist

        if self.ep > 1:
            back = torch.empty_like(y_rows)
            back.index_copy_(0, state["regroup"], y_rows)      # undo the regrouping
            ret = y_rows.new_empty((int(sum(state["send_splits"])), y_rows.shape[1]))
            dist.all_to_all_single(ret, back, state["send_splits"], state["recv_splits"], group=self.group)
        else:
            ret = y_rows
        T, k, order = state["T"], state["k"], state["order"]
        if ret.is_cuda and ret.dtype == torch.bfloat16:
            # one gather per token instead of a scatter-add per copy: row of `ret` holding copy j of token t
            pos = torch.empty_like(order)
            pos[order] = torch.arange(order.numel(), device=order.device)
            from . import ops
            return ops.moe_combine(ret.contiguous(), pos.reshape(T, k).to(torch.int32).contiguous(),
                                   weights.to(torch.bfloat16).contiguous())
        token_of = torch.div(order, k, rounding_mode="floor")
        w = weights.reshape(-1).index_select(0, order).unsqueeze(1)
        out = torch.zeros((T, ret.shape[1]), dtype=ret.dtype, device=ret.device)
        out.index_add_(0, token_of, ret * w.to(ret.dtype))
        return out


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


class QMixtralMoEBlockEP(torch.nn.Module):
    def __init__(self, cfg: MoEConfig, weights: dict, ep_rank: int = 0, ep_size: int = 1, group=None, device="cuda"):
        super().__init__()
        from .llama_layer import PackedLinear

        self.cfg = cfg
        self.dispatcher = ExpertParallelDispatcher(cfg.n_experts, ep_rank, ep_size, group)
        dev = torch.device(device)
        self.router = weights["router"].to(dev)
        self.experts = []
        e0 = ep_rank * self.dispatcher.e_local
        for e in range(e0, e0 + self.dispatcher.e_local):
            ew = weights["experts"][e]
            gu = PackedLinear(torch.cat([ew["w1"], ew["w3"]], 0).to(dev), ew["w1_index"], cfg.select_num)
            dn = PackedLinear(ew["w2"].to(dev).contiguous(), ew["w2_index"], cfg.select_num)
            self.experts.append((gu, dn))

    n_streams = 4   # experts are independent: a few streams hide the launch gaps of their small kernels

    @torch.no_grad()
    def expert_forward(self, rows: torch.Tensor, per_expert) -> torch.Tensor:
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
                h = gu.gemm(a, sfa, sx)
                act, amax = ops.silu_mul(h)
                b, sfb, sa = NVFP4_reorder_quantize_x(act, dn.index, dn.select_num, mode=16, amax=amax)
                out[start:start + n] = dn.gemm(b, sfb, sa)
            start += n
        if use_streams:
            for s in self._streams:
                cur.wait_stream(s)
        return out

    @torch.no_grad()
    def forward(self, x: torch.Tensor, routing=None) -> torch.Tensor:
        """x: this rank's tokens [T, hidden] (bf16).  routing: optional precomputed
        (expert ids [T,k], weights [T,k]) - otherwise the block's own router decides."""
        ids, w = routing if routing is not None else route_top_k(x, self.router, self.cfg.top_k)
        rows, per_expert, state = self.dispatcher.dispatch(x, ids)
        y = self.expert_forward(rows, per_expert)
        return self.dispatcher.combine(y, w, state)

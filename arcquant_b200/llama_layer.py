"""Llama-architecture decoder layer on ARC-NVFP4 linears, tensor-parallel over 1/2/4/8 GPUs.

Call order of the reference layer (model/qLlamaLayer.py:136-178, 281-372, 423-443 of ARCQuant) with
its two fusions made explicit: q/k/v share one quantized activation, so they are ONE GEMM over a
fused [q;k;v] weight, and likewise gate/up; the two RMSNorms are fused into the quantizer
(`rmsnorm_quantize_x`, as the reference's benchmark model does, benchmarks/modeling_arc.py:222-227).

    x --rmsnorm+quant(q order)--> qkv GEMM --RoPE, causal GQA attention--> quant(o order) --> o GEMM
      --all-reduce--> +x --rmsnorm+quant(up order)--> gate_up GEMM --SiLU*up--> quant(down order)
      --> down GEMM --all-reduce--> +h

Column-parallel GEMMs (qkv, gate_up) shard N, row-parallel ones (o, down) shard K (see tp.py);
one NCCL all-reduce follows each row-parallel GEMM.  Attention itself (RoPE, SDPA) is torch.
"""
from __future__ import annotations

import contextlib
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import ops, tp
from .qlinear import NVFP4_reorder_quantize_w, NVFP4_reorder_quantize_x


@dataclass
class LlamaLayerConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    rope_theta: float = 500000.0
    eps: float = 1e-5
    select_num: int = 128


def random_layer_weights(cfg: LlamaLayerConfig, seed: int = 0, device="cpu", std: float = 0.02):
    """Random-init weights of one layer, identical for every TP degree (one generator, full shapes)."""
    g = torch.Generator().manual_seed(seed)

    def w(n, k):
        return (torch.randn(n, k, generator=g) * std).to(torch.bfloat16).to(device)

    hd = cfg.n_heads * cfg.head_dim
    kvd = cfg.n_kv_heads * cfg.head_dim
    return {
        "wq": w(hd, cfg.hidden), "wk": w(kvd, cfg.hidden), "wv": w(kvd, cfg.hidden), "wo": w(cfg.hidden, hd),
        "w_gate": w(cfg.ffn, cfg.hidden), "w_up": w(cfg.ffn, cfg.hidden), "w_down": w(cfg.hidden, cfg.ffn),
        "ln1": (1.0 + 0.1 * torch.randn(cfg.hidden, generator=g)).to(torch.bfloat16).to(device),
        "ln2": (1.0 + 0.1 * torch.randn(cfg.hidden, generator=g)).to(torch.bfloat16).to(device),
    }


def random_reorder_indices(cfg: LlamaLayerConfig, seed: int = 1):
    """Synthetic stand-in for the calibrated channel orders (one per quantize site)."""
    g = torch.Generator().manual_seed(seed)
    hd = cfg.n_heads * cfg.head_dim
    return {
        "q": torch.randperm(cfg.hidden, generator=g).to(torch.int16),
        "o": torch.randperm(hd, generator=g).to(torch.int16),
        "up": torch.randperm(cfg.hidden, generator=g).to(torch.int16),
        "down": torch.randperm(cfg.ffn, generator=g).to(torch.int16),
    }


_ROPE_CACHE: dict = {}


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float):
    """cos / sin tables [len(positions), head_dim] in fp32.  The tables of the last few position
    tensors are kept (keyed by storage, length and version counter: a tensor that was written to in
    place is a new key), so a prefill loop that passes the same positions to every layer and step
    builds them once instead of with a dozen small kernels per layer."""
    key = (positions.data_ptr(), positions.numel(), positions._version, str(positions.device), positions.dtype,
           head_dim, float(theta))
    hit = _ROPE_CACHE.get(key)
    if hit is not None and hit[0] is positions:
        return hit[1], hit[2]
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=positions.device, dtype=torch.float32) / head_dim))
    ang = positions.to(torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([ang, ang], dim=-1)
    cos, sin = emb.cos(), emb.sin()
    if len(_ROPE_CACHE) >= 8:
        _ROPE_CACHE.pop(next(iter(_ROPE_CACHE)))
    _ROPE_CACHE[key] = (positions, cos, sin)   # holding the tensor keeps its storage address unique
    return cos, sin


def apply_rope(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """t: [B, H, S, D]; rotate-half convention of the HF Llama the reference wraps."""
    tf = t.float()
    half = t.shape[-1] // 2
    rot = torch.cat([-tf[..., half:], tf[..., :half]], dim=-1)
    return (tf * cos + rot * sin).to(t.dtype)


class PackedLinear(torch.nn.Module):
    """Packed NVFP4 weight + the channel order / KE its activation must be quantized with.

    Codes, block scales, the per-tensor scale, the int16 channel order and KE are registered buffers:
    a layer's ``state_dict`` carries everything needed to run it, and ``from_packed`` rebuilds the
    linear from those buffers without touching the bf16 weight again (the reference re-derives them
    from the bf16 checkpoint at every load, model/qLinearLayer.py:25-28,55)."""

    BUFFERS = ("W", "SFW", "scale", "index", "select_num_t")

    def __init__(self, weight: torch.Tensor | None, index: torch.Tensor | None, select_num: int = 0):
        super().__init__()
        if weight is None:      # filled by from_packed
            return
        dev = weight.device
        idx = index.to(torch.int16).to(dev).contiguous()
        W, SFW, scale = NVFP4_reorder_quantize_w(weight.contiguous(), idx, select_num, mode=16)
        self._set(W, SFW, scale.reshape(()), idx, select_num)

    def _set(self, W, SFW, scale, index, select_num: int):
        self.register_buffer("W", W)
        self.register_buffer("SFW", SFW)
        self.register_buffer("scale", scale.to(torch.float32).reshape(()))
        self.register_buffer("index", index.to(torch.int16))
        self.register_buffer("select_num_t", torch.tensor(int(select_num), dtype=torch.int32))
        self.select_num = int(select_num)

    @classmethod
    def from_packed(cls, state: dict, prefix: str = "", device=None) -> "PackedLinear":
        """Rebuild from the buffers of a saved ``state_dict`` (keys ``prefix + name``)."""
        missing = [n for n in cls.BUFFERS if prefix + n not in state]
        if missing:
            raise KeyError(f"packed linear '{prefix}': missing {missing}")
        get = lambda n: state[prefix + n] if device is None else state[prefix + n].to(device)
        W, SFW, index = get("W"), get("SFW"), get("index")
        select_num = int(state[prefix + "select_num_t"])
        kq = index.numel()
        if W.dtype != torch.uint8 or SFW.dtype != torch.uint8 or index.dtype != torch.int16:
            raise ValueError(f"packed linear '{prefix}': wrong buffer dtypes")
        if W.dim() != 2 or W.shape[1] * 2 != kq + select_num:
            raise ValueError(f"packed linear '{prefix}': codes [{tuple(W.shape)}] do not match KQ {kq} + KE {select_num}")
        self = cls(None, None)
        self._set(W.contiguous(), SFW.contiguous(), get("scale"), index.contiguous(), select_num)
        return self

    def gemm(self, qx, sfx, scale_x=None, residual=None):
        """x W^T (+ residual, added in the GEMM's epilogue: for prefill-sized batches)."""
        if residual is not None:
            return ops.matmul_residual(qx, self.W, sfx, self.SFW, self.scale if scale_x is None else scale_x,
                                       None if scale_x is None else self.scale, residual)
        if scale_x is None:
            return ops.matmul_dev_alpha(qx, self.W, sfx, self.SFW, self.scale, None)
        return ops.matmul_dev_alpha(qx, self.W, sfx, self.SFW, scale_x, self.scale)


class PhaseTimer:
    """Per-phase device time of a step (CUDA events around each phase; eager runs only - it synchronises
    when read).  Phases: quantize, gemm, attention, glue, collective."""

    def __init__(self):
        self.spans = []

    @contextlib.contextmanager
    def phase(self, name: str):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        yield
        e1.record()
        self.spans.append((name, e0, e1))

    def totals(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for name, e0, e1 in self.spans:
            out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
        self.spans = []
        return out


class QLlamaDecoderLayerTP(torch.nn.Module):
    timer: PhaseTimer | None = None     # set to a PhaseTimer to attribute the time of eager steps

    def _ph(self, name: str):
        return self.timer.phase(name) if self.timer is not None else contextlib.nullcontext()

    def __init__(self, cfg: LlamaLayerConfig, weights: dict, indices: dict, tp_rank: int = 0, tp_size: int = 1,
                 group=None, device="cuda", fuse_swiglu: bool = True):
        """fuse_swiglu: pack gate and up interleaved in blocks of 128 channels so that SiLU(gate) * up (and its
        max|.|) is computed in the gate_up GEMM's epilogue instead of a pass of its own over [tokens, 2 * ffn];
        same bits either way.  Needs ffn / tp_size to be a multiple of 128; meant for prefill-sized batches
        (the fused GEMM always runs the CTA-pair kernel)."""
        super().__init__()
        self.cfg, self.rank, self.tp, self.group = cfg, tp_rank, tp_size, group
        self.fuse_swiglu = bool(fuse_swiglu) and (cfg.ffn // tp_size) % 128 == 0
        if cfg.n_heads % tp_size or cfg.n_kv_heads % tp_size or cfg.ffn % tp_size:
            raise ValueError("heads / kv heads / ffn must split over the tensor-parallel group")
        dev = torch.device(device)
        D = cfg.head_dim
        self.h_local = cfg.n_heads // tp_size
        self.kv_local = cfg.n_kv_heads // tp_size
        q0, q1 = tp.shard_range(cfg.n_heads * D, tp_size, tp_rank)
        k0, k1 = tp.shard_range(cfg.n_kv_heads * D, tp_size, tp_rank)
        f0, f1 = tp.shard_range(cfg.ffn, tp_size, tp_rank)
        to = lambda t: t.to(dev)
        # column-parallel: rows of this rank's heads / ffn slice, global channel order
        wqkv = torch.cat([to(weights["wq"][q0:q1]), to(weights["wk"][k0:k1]), to(weights["wv"][k0:k1])], dim=0)
        self.qkv = PackedLinear(wqkv, indices["q"], cfg.select_num)
        if self.fuse_swiglu:
            wgu = ops.interleave_gate_up(to(weights["w_gate"][f0:f1]), to(weights["w_up"][f0:f1]))
        else:
            wgu = torch.cat([to(weights["w_gate"][f0:f1]), to(weights["w_up"][f0:f1])], dim=0)
        self.gate_up = PackedLinear(wgu, indices["up"], cfg.select_num)
        self.register_buffer("fuse_swiglu_t", torch.tensor(int(self.fuse_swiglu), dtype=torch.int32))
        # row-parallel: K slice with its local order and local KE
        self.o = PackedLinear(to(weights["wo"][:, q0:q1]).contiguous(), tp.local_reorder_index(indices["o"], q0, q1),
                              tp.shard_select_num(cfg.select_num, tp_size, q1 - q0))
        self.down = PackedLinear(to(weights["w_down"][:, f0:f1]).contiguous(),
                                 tp.local_reorder_index(indices["down"], f0, f1),
                                 tp.shard_select_num(cfg.select_num, tp_size, f1 - f0))
        self.register_buffer("ln1", to(weights["ln1"]).contiguous())
        self.register_buffer("ln2", to(weights["ln2"]).contiguous())
        self.f_local = f1 - f0

    @classmethod
    def from_packed(cls, cfg: LlamaLayerConfig, state: dict, tp_rank: int = 0, tp_size: int = 1, group=None,
                    device="cuda") -> "QLlamaDecoderLayerTP":
        """Rebuild one rank's layer from the ``state_dict`` of a layer built for the same
        (tp_rank, tp_size): packed codes, scales, channel orders and norm gains, no bf16 weights."""
        self = cls.__new__(cls)
        torch.nn.Module.__init__(self)
        self.cfg, self.rank, self.tp, self.group = cfg, tp_rank, tp_size, group
        if cfg.n_heads % tp_size or cfg.n_kv_heads % tp_size or cfg.ffn % tp_size:
            raise ValueError("heads / kv heads / ffn must split over the tensor-parallel group")
        dev = torch.device(device)
        self.h_local = cfg.n_heads // tp_size
        self.kv_local = cfg.n_kv_heads // tp_size
        self.f_local = cfg.ffn // tp_size
        for name in ("qkv", "gate_up", "o", "down"):
            setattr(self, name, PackedLinear.from_packed(state, name + ".", dev))
        want = {"qkv": (self.h_local + 2 * self.kv_local) * cfg.head_dim, "gate_up": 2 * self.f_local,
                "o": cfg.hidden, "down": cfg.hidden}
        for name, rows in want.items():
            if getattr(self, name).W.shape[0] != rows:
                raise ValueError(f"{name}: {getattr(self, name).W.shape[0]} output rows, expected {rows} for tp_size {tp_size}")
        self.register_buffer("ln1", state["ln1"].to(dev).contiguous())
        self.register_buffer("ln2", state["ln2"].to(dev).contiguous())
        self.fuse_swiglu = bool(int(state["fuse_swiglu_t"])) if "fuse_swiglu_t" in state else False
        self.register_buffer("fuse_swiglu_t", torch.tensor(int(self.fuse_swiglu), dtype=torch.int32))
        return self

    def _gate_up_act(self, a: torch.Tensor, sfa: torch.Tensor):
        """(silu(gate) * up [tokens, ffn / tp], its max|.|) from the quantized input of the gate/up projection."""
        if self.fuse_swiglu:
            return ops.matmul_swiglu(a, self.gate_up.W, sfa, self.gate_up.SFW, self.gate_up.scale, None)
        return ops.silu_mul(self.gate_up.gemm(a, sfa))

    # ---- halves of the layer up to (and excluding) the all-reduce: usable for in-process emulation
    @torch.no_grad()
    def attn_partial(self, x2d: torch.Tensor, bsz: int, seq: int, positions: torch.Tensor,
                     residual: torch.Tensor | None = None) -> torch.Tensor:
        cfg, D = self.cfg, self.cfg.head_dim
        with self._ph("quantize"):
            a, sfa = ops.rmsnorm_quantize_x(x2d, self.ln1, cfg.eps, self.qkv.index, self.qkv.select_num)
        with self._ph("gemm"):
            qkv = self.qkv.gemm(a, sfa)
        nq, nk = self.h_local * D, self.kv_local * D
        # rotary embedding in place on the q and k columns of the fused output (they are adjacent);
        # attention reads strided views of it, grouped-query heads are not materialised
        with self._ph("glue"):
            cos, sin = rope_tables(positions, D, cfg.rope_theta)
            ops.rope_inplace(qkv, cos, sin, self.h_local + self.kv_local, D)
        with self._ph("attention"):
            q = qkv[:, :nq].reshape(bsz, seq, self.h_local, D).transpose(1, 2)
            k = qkv[:, nq:nq + nk].reshape(bsz, seq, self.kv_local, D).transpose(1, 2)
            v = qkv[:, nq + nk:].reshape(bsz, seq, self.kv_local, D).transpose(1, 2)
            attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.h_local != self.kv_local)
            attn = attn.transpose(1, 2).reshape(bsz * seq, nq).contiguous()
        with self._ph("quantize"):
            qa, sfo, so = NVFP4_reorder_quantize_x(attn, self.o.index, self.o.select_num, mode=16)
        with self._ph("gemm"):
            return self.o.gemm(qa, sfo, so, residual)

    @torch.no_grad()
    def mlp_partial(self, h2d: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.cfg
        with self._ph("quantize"):
            a, sfa = ops.rmsnorm_quantize_x(h2d, self.ln2, cfg.eps, self.gate_up.index, self.gate_up.select_num)
        with self._ph("gemm"):
            act, amax = self._gate_up_act(a, sfa)      # silu(gate) * up and its max|.| with the GEMM
        with self._ph("quantize"):
            qd, sfd, sd = NVFP4_reorder_quantize_x(act, self.down.index, self.down.select_num, mode=16, amax=amax)
        with self._ph("gemm"):
            return self.down.gemm(qd, sfd, sd, residual)

    @torch.no_grad()
    def forward(self, x: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
        bsz, seq, hidden = x.shape
        if positions is None:
            positions = torch.arange(seq, device=x.device)
        x2d = x.reshape(bsz * seq, hidden).contiguous()
        if self.tp > 1 and x2d.shape[0] >= 2 * self.overlap_rows and self._dist_ready():
            return self._forward_overlapped(x2d, bsz, seq, positions).reshape(bsz, seq, hidden)
        if self.tp == 1 and self.fuse_residual and x2d.shape[0] >= 1024:
            # one rank, a prefill-sized batch: both residual additions happen in the epilogues of the o and down GEMMs
            h = self.attn_partial(x2d, bsz, seq, positions, residual=x2d)
            return self.mlp_partial(h, residual=h).reshape(bsz, seq, hidden)
        y = self.attn_partial(x2d, bsz, seq, positions)
        if self.tp > 1:      # (an unsharded layer inside a multi-rank process talks to nobody)
            with self._ph("collective"):
                y = tp.all_reduce_sum(y, self.group)
        with self._ph("glue"):
            h = x2d + y
        y = self.mlp_partial(h)
        if self.tp > 1:
            with self._ph("collective"):
                y = tp.all_reduce_sum(y, self.group)
        with self._ph("glue"):
            out = h + y
        return out.reshape(bsz, seq, hidden)

    overlap_rows = 4096   # rows per chunk of the overlapped schedule (a multiple of 128)
    fuse_residual = True  # one rank: residual additions in the GEMM epilogues (same bits as separate additions)

    # ---- sequence-parallel form: the residual stream is sharded by tokens over the group
    def _gather_quantized(self, q_s: torch.Tensor, sf_s: torch.Tensor, rows_s: int, k_eff: int):
        """All-gather of packed codes and block scales of every rank's token shard (whole 128-row scale
        tiles, so the shards' scale bytes concatenate): 0.56 bytes per element on the wire instead of
        the 2 of a bf16 activation."""
        import torch.distributed as dist

        tile = ((k_eff // 16 + 3) // 4) * 512
        span_s = (rows_s // 128) * tile
        q = torch.empty((rows_s * self.tp, k_eff // 2), dtype=torch.uint8, device=q_s.device)
        sf = torch.empty((ops.sf_bytes(rows_s * self.tp, k_eff),), dtype=torch.uint8, device=q_s.device)
        dist.all_gather_into_tensor(q, q_s, group=self.group)
        dist.all_gather_into_tensor(sf[:span_s * self.tp], sf_s[:span_s], group=self.group)
        return q, sf

    @torch.no_grad()
    def forward_sequence_parallel(self, x_shard: torch.Tensor, bsz: int, seq: int,
                                  positions: torch.Tensor | None = None) -> torch.Tensor:
        """x_shard: this rank's contiguous run of bsz*seq/tp tokens [tokens/tp, hidden] (a multiple of
        128 rows); returns the same rows of the layer's output.  RMSNorm + quantize run on the shard
        only (not replicated), the packed result is all-gathered for the column-parallel GEMMs, and the
        row-parallel GEMMs end in a reduce-scatter instead of an all-reduce.  Same arithmetic as
        `forward` row for row."""
        import torch.distributed as dist

        cfg, D = self.cfg, self.cfg.head_dim
        T, rows_s = bsz * seq, x_shard.shape[0]
        if rows_s * self.tp != T or rows_s % 128:
            raise ValueError("token shards must be equal and multiples of 128 rows")
        if positions is None:
            positions = torch.arange(seq, device=x_shard.device)
        k_eff = cfg.hidden + self.qkv.select_num
        a, sfa = self._quantize_gathered(x_shard, self.ln1, self.qkv, rows_s, k_eff, self.peer_g1)
        with self._ph("gemm"):
            qkv = self.qkv.gemm(a, sfa)
        nq, nk = self.h_local * D, self.kv_local * D
        with self._ph("glue"):
            cos, sin = rope_tables(positions, D, cfg.rope_theta)
            ops.rope_inplace(qkv, cos, sin, self.h_local + self.kv_local, D)
        with self._ph("attention"):
            q = qkv[:, :nq].reshape(bsz, seq, self.h_local, D).transpose(1, 2)
            k = qkv[:, nq:nq + nk].reshape(bsz, seq, self.kv_local, D).transpose(1, 2)
            v = qkv[:, nq + nk:].reshape(bsz, seq, self.kv_local, D).transpose(1, 2)
            attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.h_local != self.kv_local)
            attn = attn.transpose(1, 2).reshape(T, nq).contiguous()
        with self._ph("quantize"):
            qa, sfo, so = NVFP4_reorder_quantize_x(attn, self.o.index, self.o.select_num, mode=16)
        h_s = self._reduce_rows(self.o, qa, sfo, so, x_shard, self.peer_o)
        a, sfa = self._quantize_gathered(h_s, self.ln2, self.gate_up, rows_s, k_eff, self.peer_g2)
        with self._ph("gemm"):
            act, amax = self._gate_up_act(a, sfa)
        with self._ph("quantize"):
            qd, sfd, sd = NVFP4_reorder_quantize_x(act, self.down.index, self.down.select_num, mode=16, amax=amax)
        return self._reduce_rows(self.down, qd, sfd, sd, h_s, self.peer_down)

    # ---- row-parallel projection + reduce-scatter + residual
    peer_o = None       # peer.PeerSlots of the o / down projections once `enable_peer_scatter` has run
    peer_down = None
    peer_g1 = None      # peer.PeerGathered: quantized input of the qkv / gate_up projections
    peer_g2 = None
    peer_barrier = None

    def enable_peer_scatter(self, total_rows: int) -> None:
        """Sequence-parallel steps over `total_rows` tokens from now on send the partial results of the o and down
        projections straight from the GEMM's epilogue into the owning rank's memory (`ops.matmul_scatter`) and
        finish the reduce-scatter with a barrier and one local pass that also adds the residual
        (`ops.sum_partials`), instead of a GEMM into local memory followed by NCCL's reduce-scatter and an
        addition; the fused RMSNorm quantizers store their rows into every rank's gathered buffers
        (`ops.rmsnorm_quantize_x_multi`) instead of an all-gather behind them; and the ranks meet at barriers
        through flags in peer memory (`ops.peer_barrier`).  No NCCL call is left in the step.
        Collective call: every rank of the group, same arguments.  The ranks must share one machine."""
        from .peer import PeerBarrier, PeerGathered, PeerSlots

        rows_s = total_rows // self.tp
        if rows_s * self.tp != total_rows or rows_s % 128:
            raise ValueError("token shards must be equal and multiples of 128 rows")
        dev = self.ln1.device
        # (two blocks: the barrier of one projection and the all-gather that follows it separate a block's
        # readers from its next writers)
        k_eff = self.cfg.hidden + self.qkv.select_num
        made = {}
        try:     # all five blocks or none (a failure is raised on every rank together, see peer.PeerBlock)
            made["peer_o"] = PeerSlots(rows_s, self.cfg.hidden, self.rank, self.tp, self.group, dev)
            made["peer_down"] = PeerSlots(rows_s, self.cfg.hidden, self.rank, self.tp, self.group, dev)
            made["peer_g1"] = PeerGathered(rows_s, k_eff, self.rank, self.tp, self.group, dev)
            made["peer_g2"] = PeerGathered(rows_s, k_eff, self.rank, self.tp, self.group, dev)
            made["peer_barrier"] = PeerBarrier(self.rank, self.tp, self.group, dev)
        except Exception:
            for block in made.values():
                block.close()
            raise
        for name, block in made.items():
            setattr(self, name, block)

    def disable_peer_scatter(self) -> None:
        for name in ("peer_o", "peer_down", "peer_g1", "peer_g2", "peer_barrier"):
            slots = getattr(self, name)
            if slots is not None:
                slots.close()
            setattr(self, name, None)

    def _reduce_rows(self, lin: PackedLinear, q, sf, scale_x, residual_s: torch.Tensor, slots) -> torch.Tensor:
        """residual_s + (this rank's token rows of the sum over ranks of x_r W_r^T)."""
        import torch.distributed as dist

        if slots is not None and slots.rows == residual_s.shape[0]:
            with self._ph("gemm"):
                ops.matmul_scatter(q, lin.W, sf, lin.SFW, scale_x, lin.scale, slots.dests)
            with self._ph("collective"):
                self.peer_barrier()      # every rank's GEMM, and with it every store into this rank's slots, is complete
            with self._ph("glue"):
                out = torch.empty_like(residual_s)
                return ops.sum_partials(slots.sources, residual_s.numel(), out, residual_s)
        with self._ph("gemm"):
            y = lin.gemm(q, sf, scale_x)
        y_s = torch.empty_like(residual_s)
        with self._ph("collective"):
            dist.reduce_scatter_tensor(y_s, y, op=dist.ReduceOp.SUM, group=self.group)
        with self._ph("glue"):
            return residual_s + y_s

    def _quantize_gathered(self, x_s: torch.Tensor, gain: torch.Tensor, lin: PackedLinear, rows_s: int, k_eff: int,
                           gathered):
        """(codes [rows_s * tp, k_eff / 2], scales) of RMSNorm(x) over all ranks' token shards."""
        if gathered is not None and gathered.q.shape[0] == rows_s * self.tp:
            with self._ph("quantize"):
                ops.rmsnorm_quantize_x_multi(x_s, gain, self.cfg.eps, lin.index, lin.select_num, gathered.q_dests,
                                             gathered.sf_dests)
            with self._ph("collective"):
                self.peer_barrier()      # every rank's rows have arrived in this rank's copy
            return gathered.q, gathered.sf
        with self._ph("quantize"):
            a_s, sfa_s = ops.rmsnorm_quantize_x(x_s, gain, self.cfg.eps, lin.index, lin.select_num)
        with self._ph("collective"):
            return self._gather_quantized(a_s, sfa_s, rows_s, k_eff)

    # ---- the same with communication hidden behind compute
    @staticmethod
    def pipelined_shard_rows(total_rows: int, tp_size: int, tp_rank: int, chunks: int) -> torch.Tensor:
        """Rows of the [total_rows, hidden] residual stream that rank `tp_rank` holds in the pipelined
        sequence-parallel form: the stream is cut into `chunks` runs of whole sequences and every rank owns
        its 1/tp slice of EVERY run (so each run's collectives involve all ranks evenly)."""
        tc = total_rows // chunks
        rc = tc // tp_size
        base = torch.arange(chunks).repeat_interleave(rc) * tc + tp_rank * rc
        return base + torch.arange(rc).repeat(chunks)

    @torch.no_grad()
    def forward_sequence_parallel_pipelined(self, x_shard: torch.Tensor, bsz: int, seq: int,
                                            positions: torch.Tensor | None = None, chunks: int = 4) -> torch.Tensor:
        """`forward_sequence_parallel` with its collectives overlapped with compute.  The batch is cut into
        `chunks` runs of whole sequences; x_shard holds this rank's slice of every run
        (`pipelined_shard_rows`).  Everything between two per-tensor scales is independent per row, so
        inside each of the three segments that the two scales (o and down inputs) delimit, the all-gather
        or reduce-scatter of one run (NCCL, asynchronous) runs under the GEMMs, attention and quantizers
        of its neighbours.  Row for row the arithmetic is that of `forward_sequence_parallel`."""
        import torch.distributed as dist

        cfg, D, C = self.cfg, self.cfg.head_dim, chunks
        T = bsz * seq
        if bsz % C or x_shard.shape[0] * self.tp != T or (T // C // self.tp) % 128:
            raise ValueError("runs must be whole sequences and every rank's slice of a run a multiple of 128 rows")
        if positions is None:
            positions = torch.arange(seq, device=x_shard.device)
        tc, rc = T // C, T // C // self.tp            # rows of a run, rows of this rank's slice of it
        bc = bsz // C
        k_eff = cfg.hidden + self.qkv.select_num
        tile = ((k_eff // 16 + 3) // 4) * 512
        span = (rc // 128) * tile
        nq, nk = self.h_local * D, self.kv_local * D
        dev = x_shard.device
        xs = x_shard.reshape(C, rc, cfg.hidden)

        def gather_async(q_s, sf_s):
            q = torch.empty((tc, k_eff // 2), dtype=torch.uint8, device=dev)
            sf = torch.empty((ops.sf_bytes(tc, k_eff),), dtype=torch.uint8, device=dev)
            w1 = dist.all_gather_into_tensor(q, q_s, group=self.group, async_op=True)
            w2 = dist.all_gather_into_tensor(sf[:span * self.tp], sf_s[:span], group=self.group, async_op=True)
            return q, sf, (w1, w2)

        # segment A: fused RMSNorm + quantize of the slices, all-gather, qkv GEMM, attention per run
        pend = []
        for c in range(C):
            a_s, sfa_s = ops.rmsnorm_quantize_x(xs[c], self.ln1, cfg.eps, self.qkv.index, self.qkv.select_num)
            pend.append(gather_async(a_s, sfa_s))
        cos, sin = rope_tables(positions, D, cfg.rope_theta)
        attn = torch.empty((C, tc, nq), dtype=torch.bfloat16, device=dev)
        amax = []
        for c in range(C):
            a, sfa, works = pend[c]
            for w in works:
                w.wait()
            qkv = self.qkv.gemm(a, sfa)
            ops.rope_inplace(qkv, cos, sin, self.h_local + self.kv_local, D)
            q = qkv[:, :nq].reshape(bc, seq, self.h_local, D).transpose(1, 2)
            k = qkv[:, nq:nq + nk].reshape(bc, seq, self.kv_local, D).transpose(1, 2)
            v = qkv[:, nq + nk:].reshape(bc, seq, self.kv_local, D).transpose(1, 2)
            o = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.h_local != self.kv_local)
            attn[c].copy_(o.transpose(1, 2).reshape(tc, nq))
            amax.append(ops.absmax(attn[c]))
        scale_o = torch.stack(amax).max() / (448.0 * 6.0)
        # segment B: o projection + reduce-scatter, residual, RMSNorm + quantize, all-gather, gate_up, SiLU
        ys = torch.empty_like(xs)
        pend = []
        for c in range(C):
            qa, sfo = ops.reorder_quantize_x(attn[c], self.o.index, self.o.select_num, mode=16, scale=scale_o)
            y = self.o.gemm(qa, sfo, scale_o)
            pend.append((y, dist.reduce_scatter_tensor(ys[c], y, op=dist.ReduceOp.SUM, group=self.group, async_op=True)))
        hs = torch.empty_like(xs)
        gathers = []
        for c in range(C):
            pend[c][1].wait()
            torch.add(xs[c], ys[c], out=hs[c])
            a_s, sfa_s = ops.rmsnorm_quantize_x(hs[c], self.ln2, cfg.eps, self.gate_up.index, self.gate_up.select_num)
            gathers.append(gather_async(a_s, sfa_s))
        acts, amax = [], []
        for c in range(C):
            a, sfa, works = gathers[c]
            for w in works:
                w.wait()
            act, am = self._gate_up_act(a, sfa)
            acts.append(act)
            amax.append(am)
        scale_d = torch.stack(amax).max() / (448.0 * 6.0)
        # segment C: down projection + reduce-scatter, residual
        pend = []
        for c in range(C):
            qd, sfd = ops.reorder_quantize_x(acts[c], self.down.index, self.down.select_num, mode=16, scale=scale_d)
            y = self.down.gemm(qd, sfd, scale_d)
            pend.append((y, dist.reduce_scatter_tensor(ys[c], y, op=dist.ReduceOp.SUM, group=self.group, async_op=True)))
        out = torch.empty_like(xs)
        for c in range(C):
            pend[c][1].wait()
            torch.add(hs[c], ys[c], out=out[c])
        return out.reshape(C * rc, cfg.hidden)

    def _dist_ready(self) -> bool:
        import torch.distributed as dist
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    @torch.no_grad()
    def _attn_core(self, x2d, bsz, seq, positions):
        """Everything of the attention half before the row-parallel o projection."""
        cfg, D = self.cfg, self.cfg.head_dim
        a, sfa = ops.rmsnorm_quantize_x(x2d, self.ln1, cfg.eps, self.qkv.index, self.qkv.select_num)
        qkv = self.qkv.gemm(a, sfa)
        nq, nk = self.h_local * D, self.kv_local * D
        cos, sin = rope_tables(positions, D, cfg.rope_theta)
        ops.rope_inplace(qkv, cos, sin, self.h_local + self.kv_local, D)
        q = qkv[:, :nq].reshape(bsz, seq, self.h_local, D).transpose(1, 2)
        k = qkv[:, nq:nq + nk].reshape(bsz, seq, self.kv_local, D).transpose(1, 2)
        v = qkv[:, nq + nk:].reshape(bsz, seq, self.kv_local, D).transpose(1, 2)
        attn = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=self.h_local != self.kv_local)
        return attn.transpose(1, 2).reshape(bsz * seq, nq).contiguous()

    @torch.no_grad()
    def _forward_overlapped(self, x2d, bsz, seq, positions):
        """Same arithmetic as `forward`'s plain path - per-tensor scales are taken over the whole
        tensor first, everything after them is independent per row - but the two row-parallel
        projections run in chunks of rows whose all-reduces (NCCL, asynchronous) overlap the GEMMs
        and element-wise work of the other chunks."""
        import torch.distributed as dist

        cfg = self.cfg
        T = x2d.shape[0]
        bounds = [(r, min(r + self.overlap_rows, T)) for r in range(0, T, self.overlap_rows)]
        attn = self._attn_core(x2d, bsz, seq, positions)
        scale_o = ops.absmax(attn) / (448.0 * 6.0)
        o_parts, works = [], []
        for r0, r1 in bounds:
            qa, sfo = ops.reorder_quantize_x(attn[r0:r1], self.o.index, self.o.select_num, mode=16, scale=scale_o)
            y = self.o.gemm(qa, sfo, scale_o)
            works.append(dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            o_parts.append(y)
        h = torch.empty_like(x2d)
        acts, amaxes = [], []
        for (r0, r1), y, w in zip(bounds, o_parts, works):
            w.wait()
            torch.add(x2d[r0:r1], y, out=h[r0:r1])
            a, sfa = ops.rmsnorm_quantize_x(h[r0:r1], self.ln2, cfg.eps, self.gate_up.index, self.gate_up.select_num)
            act, amax = self._gate_up_act(a, sfa)
            acts.append(act)
            amaxes.append(amax)
        scale_d = torch.stack(amaxes).max() / (448.0 * 6.0)
        d_parts, works = [], []
        for act in acts:
            qd, sfd = ops.reorder_quantize_x(act, self.down.index, self.down.select_num, mode=16, scale=scale_d)
            y = self.down.gemm(qd, sfd, scale_d)
            works.append(dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            d_parts.append(y)
        out = torch.empty_like(x2d)
        for (r0, r1), y, w in zip(bounds, d_parts, works):
            w.wait()
            torch.add(h[r0:r1], y, out=out[r0:r1])
        return out

"""Torch restatement of the reference's CPU-runnable "fake-quant" path.

TEST / BASELINE INFRASTRUCTURE ONLY (never imported by the shipped package).
This is the arm that is *timed* on the host cores next to the GPU numbers; it
is not the bit-exact oracle (that is ``arcq_oracle.c``): the reference's fake
path rounds e2m1 ties towards the more negative candidate, divides by the
block scale instead of multiplying by its reciprocal and has no subnormal
block scales, so its values differ from the CUDA kernels' on a small fraction
of elements.

Follows, function by function (paths relative to the ARCQuant source tree):

  model/quantize.py:14-22     nearest of the 15 e2m1 values by argmin
  model/quantize.py:40-49     block scale: clamp [2e-3, 448], 3-bit mantissa rounding
  model/quantize.py:145-172   NVFP4 group quantize -> dequantised values
  model/quantize.py:287-312   weights: cat([q(w), q(w[:, -KE:])])
  model/quantize.py:314-343   activations: cat([q(x), q((x-q(x))[:, -KE:])]) * s
  benchmarks/modeling_arc.py:237-242  fp32 RMSNorm

The callers (model/qLlamaLayer.py:84-86) hand these functions an input that
is already gathered by ``reorder_index``, so the critical channels are the
last KE columns.
"""
from __future__ import annotations

import torch

_E2M1 = [-6.0, -4.0, -3.0, -2.0, -1.5, -1.0, -0.5, 0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def quantize_e2m1(t: torch.Tensor, chunk_rows: int = 1 << 16) -> torch.Tensor:
    """Nearest representable value; a tie picks the lower-index (more negative)
    candidate, as ``argmin`` does.  Row-chunked so the 15-way difference tensor
    stays bounded."""
    vals = torch.tensor(_E2M1, dtype=t.dtype, device=t.device)
    flat = t.reshape(-1)
    out = torch.empty_like(flat)
    step = chunk_rows * 16
    for s in range(0, flat.numel(), step):
        part = flat[s:s + step]
        d = (part.unsqueeze(-1) - vals).abs()
        out[s:s + step] = vals[d.argmin(dim=-1)]
    return out.view_as(t)


def quantize_ue4m3(t: torch.Tensor) -> torch.Tensor:
    t = t.clamp(min=2e-3, max=448.0)
    e = torch.floor(torch.log2(t + 1e-9))
    m = t / (2 ** e) - 1.0
    qm = torch.round(m * 8) / 8
    return (1 + qm) * (2 ** e)


def quantize_nvfp4_tensor(t: torch.Tensor, group: int = 16) -> torch.Tensor:
    shape = t.shape
    assert shape[-1] % group == 0
    g = t.reshape(-1, group)
    amax = g.abs().max(dim=1, keepdim=True)[0]
    scale = amax / 6.0
    scale[scale == 0] = 1e-9
    s = quantize_ue4m3(scale)
    q = quantize_e2m1(g / s) * s
    return q.view(shape)


def fake_reorder_quantize_x(x: torch.Tensor, ke: int):
    """x is already gathered.  Returns (values [M, KQ+KE], global scale).
    As in the reference the result is multiplied back by the global scale only
    when ke > 0."""
    dt = x.dtype
    scale = torch.max(x).to(torch.float32) / (448.0 * 6.0)
    xf = x.to(torch.float32) / scale
    q = quantize_nvfp4_tensor(xf)
    if ke == 0:
        return q.to(dt), scale
    err = xf - q
    qe = quantize_nvfp4_tensor(err[:, -ke:].contiguous())
    return (torch.cat([q, qe], dim=1) * scale).to(dt), scale


def fake_reorder_quantize_w(w: torch.Tensor, ke: int):
    """w is already gathered.  The result is never multiplied back by the scale."""
    dt = w.dtype
    scale = torch.max(w).to(torch.float32) / (448.0 * 6.0)
    wf = w.to(torch.float32) / scale
    q = quantize_nvfp4_tensor(wf)
    if ke == 0:
        return q.to(dt), scale
    return torch.cat([q, q[:, -ke:]], dim=1).to(dt), scale


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    dt = x.dtype
    h = x.to(torch.float32)
    var = h.pow(2).mean(-1, keepdim=True)
    h = h * torch.rsqrt(var + eps)
    return weight * h.to(dt)


def fake_quantize_activations(x: torch.Tensor, idx: torch.Tensor, ke: int, gamma=None, eps: float = 1e-5):
    """(RMSNorm ->) gather -> fake ARC-NVFP4.  Returns values with every scale
    applied, i.e. an approximation of the (normalised, gathered) input with the
    residual block appended."""
    if gamma is not None:
        x = rmsnorm(x, gamma, eps)
    xg = torch.index_select(x, 1, idx.to(torch.int64))
    q, s = fake_reorder_quantize_x(xg, ke)
    if ke == 0:
        q = (q.to(torch.float32) * s).to(x.dtype)
    return q


def fake_linear(x: torch.Tensor, w: torch.Tensor, idx: torch.Tensor, ke: int) -> torch.Tensor:
    """Y = X W^T through the fake path, with the scales the reference's
    functions leave off applied by this harness."""
    i64 = idx.to(torch.int64)
    qx, sx = fake_reorder_quantize_x(torch.index_select(x, 1, i64), ke)
    qw, sw = fake_reorder_quantize_w(torch.index_select(w, 1, i64), ke)
    y = torch.nn.functional.linear(qx, qw).to(torch.float32) * sw
    if ke == 0:
        y = y * sx
    return y.to(x.dtype)

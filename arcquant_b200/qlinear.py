"""Host-side mirror of the reference's quantized linear (model/qLinearLayer.py and the
``NVFP4_reorder_quantize_x`` helper of model/qLlamaLayer.py:73-77 in ARCQuant): same names, same
argument meaning, same return tuples - with the host synchronisations taken out (the product of
the two per-tensor scales stays on the device and is read by the GEMM's epilogue).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops

FP4_MAX = 6.0
FP8_MAX = 448.0


def NVFP4_reorder_quantize_x(x: torch.Tensor, reorder_index: torch.Tensor, select_num: int, mode=None, amax=None):
    """(qx, scale_x, scale): per-tensor scale = max|x| / (448*6) as a 0-dim fp32 CUDA tensor,
    ``x / scale`` in bf16 as the reference forms it, then the fused reorder + NVFP4 + ARC kernel.
    One pass for the amax (``arcq_absmax_bf16``) instead of ``torch.max(x.abs())``; a caller that
    already has max|x| on the device (``ops.silu_mul``) passes it as ``amax``."""
    scale = (ops.absmax(x) if amax is None else amax) / (FP8_MAX * FP4_MAX)
    qx, scale_x = ops.reorder_quantize_x(x, reorder_index, select_num, mode=mode, scale=scale)   # x / scale, fused
    return qx, scale_x, scale


def NVFP4_reorder_quantize_w(w: torch.Tensor, reorder_index: torch.Tensor, select_num: int, mode=None):
    """(qw, scale_w, scale).  The reference takes the SIGNED maximum of the weight here
    (model/qLinearLayer.py:26); kept for drop-in parity."""
    scale = torch.max(w).float() / (FP8_MAX * FP4_MAX)
    qw, scale_w = ops.reorder_quantize_w(w / scale, reorder_index, select_num, mode=mode)
    return qw, scale_w, scale


class QLinearLayer(nn.Module):
    """NVFP4 linear with ARC-augmented K.  ``forward`` takes the tuple the reference's layers pass
    around: ``(qx, scale_x, scale, bsz, q_len)``.

    Unlike the reference the packed weight, its scales and the global scale are registered
    buffers, so they travel through ``state_dict`` instead of being re-derived at every load."""

    def __init__(self, originalLayer: nn.Linear, select_num: int, reorder_index: torch.Tensor,
                 out_reorder_index=None, quant_type: str = "NVFP4"):
        super().__init__()
        if quant_type != "NVFP4":
            raise NotImplementedError("only the NVFP4 path exists in this library")
        self.in_features = originalLayer.in_features
        self.out_features = originalLayer.out_features
        self.select_num = select_num
        self.quant_type = quant_type
        w = originalLayer.weight.data
        if not w.is_cuda:
            w = w.cuda()
        if originalLayer.bias is not None:
            self.register_buffer("bias", originalLayer.bias.detach().to(w.device).clone())
        else:
            self.bias = None
        idx = reorder_index.to(torch.int16).to(w.device)
        W, scale_w, scale = NVFP4_reorder_quantize_w(w.to(torch.bfloat16).contiguous(), idx, select_num)
        self.register_buffer("W", W)
        self.register_buffer("scale_w", scale_w)
        self.register_buffer("scale", scale.reshape(()))

    @torch.no_grad()
    def forward(self, x):
        qx, scale_x, scale, bsz, q_len = x
        if isinstance(scale, torch.Tensor) and scale.is_cuda:
            y = ops.matmul_dev_alpha(qx, self.W, scale_x, self.scale_w, scale, self.scale)
        else:
            y = ops.matmul(qx, self.W, scale_x, self.scale_w, float(scale) * float(self.scale))
        if self.bias is not None:
            y = y + self.bias
        if bsz is not None:
            return y.reshape(bsz, q_len, -1)
        return y.reshape(q_len, -1)

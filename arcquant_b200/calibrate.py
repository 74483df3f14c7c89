"""Calibration of channel orders and residual widths from activations, on whatever device they live on.

The reference derives both from forward passes over a calibration set: the per-channel maximum of
|x| at the input of every projection (``get_act_stats`` with the max metric, utilize.py:80-116 of
ARCQuant, running maximum over the samples), the channel order = ascending argsort of that statistic
(reorder_indices.py), and the number of residual channels from the share of elements that exceed an
eighth of their row's maximum, rounded up to a multiple of 64 (``search_select_proportions``,
utilize.py:546-551).  The same rules here, as three small functions that a caller hooks onto the
inputs of its linears; the results feed `llama_layer.PackedLinear` / `checkpoint`.
"""
from __future__ import annotations

import math

import torch


class ChannelAbsMax:
    """Running per-channel max |x| over any number of batches [..., channels], and with it the running
    count behind the residual-width rule.  bf16 batches on a CUDA device take one pass of
    `arcq_calib_stats_bf16` (both statistics at once, accumulated on the device); anything else takes the
    eager torch formulation."""

    def __init__(self):
        self.value: torch.Tensor | None = None
        self._above: torch.Tensor | None = None      # elements larger than an eighth of their row's maximum
        self._seen = 0                               # elements seen

    @torch.no_grad()
    def update(self, x: torch.Tensor) -> None:
        x2 = x.detach().reshape(-1, x.shape[-1])
        k = x2.shape[1]
        if x2.is_cuda and x2.dtype == torch.bfloat16 and k % 8 == 0 and k <= 32768 and x2.is_contiguous():
            from . import ops

            if self.value is None:
                self.value = torch.zeros(k, dtype=torch.float32, device=x2.device)
            if self._above is None:
                self._above = torch.zeros((), dtype=torch.int64, device=x2.device)
            ops.calib_stats(x2, self.value, self._above)
        else:
            cur = x2.abs().amax(dim=0).float()
            self.value = cur if self.value is None else torch.maximum(self.value, cur.to(self.value.device))
            thr = x2.max(dim=-1, keepdim=True)[0] * 0.125
            n = (x2 > thr).sum().to(torch.int64)
            self._above = n if self._above is None else self._above + n.to(self._above.device)
        self._seen += x2.numel()

    def reorder_index(self) -> torch.Tensor:
        """int16 [channels]: channels by ascending statistic - the largest (critical) channels last."""
        if self.value is None:
            raise RuntimeError("no batch seen")
        if self.value.numel() > 32752:
            raise ValueError("more channels than an int16 order can hold")
        return torch.argsort(self.value).to(torch.int16)

    def select_num(self, granule: int = 64) -> int:
        """The residual width the rule of `select_num_rule` gives for everything seen so far."""
        if self.value is None:
            raise RuntimeError("no batch seen")
        k = self.value.numel()
        ratio = float(self._above) / self._seen
        return min(math.ceil(k * ratio / granule) * granule, k)


@torch.no_grad()
def select_num_rule(x: torch.Tensor, reorder_index: torch.Tensor | None = None, granule: int = 64) -> int:
    """Residual channels for activations x [..., channels]: the share of elements larger than an eighth
    of their row's (signed) maximum decides how many channels get a residual, in units of `granule`.
    The statistic does not depend on the channel order; `reorder_index` is accepted for symmetry with
    the reference, which applies it first."""
    keys = x.detach().reshape(-1, x.shape[-1])
    if reorder_index is not None:
        keys = keys[:, reorder_index.to(keys.device).long()]
    in_features = keys.shape[1]
    threshold = keys.max(dim=-1, keepdim=True)[0] * 0.125
    ratio = float((keys > threshold).sum()) / keys.numel()
    select_num = math.ceil(in_features * ratio / granule) * granule
    return min(select_num, in_features)


def average_bits(in_features: int, select_num: int) -> float:
    """4.5 bits per stored element (e2m1 + a ue4m3 scale per 16) over the augmented width."""
    return 4.5 * (in_features + select_num) / in_features

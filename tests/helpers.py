"""Shared input builders for the parity tests (CPU tensors; the GPU tests move them)."""
from __future__ import annotations

import numpy as np
import torch

from arcquant_b200 import synth


def scaled_activations(tokens: int, hidden: int, seed: int, n_outliers: int | None = None):
    """bf16 activations already divided by the per-tensor global scale, plus a calibrated index."""
    if n_outliers is None:
        n_outliers = max(1, hidden // 100)
    out = synth.outlier_channels(hidden, n_outliers, seed + 7)
    x = synth.activations(tokens, hidden, seed, out)
    calib = synth.activations(256, hidden, seed + 13, out)
    idx = synth.reorder_index_from_stats(calib.abs().amax(dim=0))
    xs = (x / synth.global_scale(x)).contiguous()
    return xs, idx


def adversarial_rows(hidden: int) -> torch.Tensor:
    """Rows that sit on every rounding boundary: e2m1 ties of both signs, signed zeros, values
    that underflow to (signed) zero, block scales at the ue4m3 subnormal floor and at the 448 cap,
    ue4m3 ties, and an all-zero row."""
    rows = []
    base = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -6.0])
    rows.append(base.repeat(hidden // 16))                                   # scale exactly 1
    rows.append((base * 0.5).repeat(hidden // 16))
    rows.append((base * 3.0).repeat(hidden // 16))                           # non power-of-two scale
    z = torch.zeros(hidden); z[1::2] = -0.0
    rows.append(z)                                                           # zeros of both signs
    tiny = torch.full((hidden,), 1e-4); tiny[::3] = -1e-4; tiny[::16] = 0.011
    rows.append(tiny)                                                        # subnormal block scales
    huge = torch.full((hidden,), 3000.0); huge[::2] = -2900.0; huge[::16] = 3.0e4
    rows.append(huge)                                                        # scale clamps at 448
    t = torch.linspace(-8, 8, hidden)
    rows.append(t)
    g = torch.Generator().manual_seed(5)
    rows.append(torch.randn(hidden, generator=g) * 6.375)                    # amax/6 near ue4m3 ties
    rows.append(torch.randn(hidden, generator=g) * 0.01)
    return torch.stack(rows).to(torch.bfloat16)


def valid_sf(sf, rows: int, k_eff: int):
    from oracle import oracle as O

    off = O.sf_valid_offsets(rows, k_eff)
    a = sf if isinstance(sf, np.ndarray) else sf.cpu().numpy()
    return a[off]

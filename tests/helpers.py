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


def steady_state_rows(tokens: int, ctas: int = 148, ring: int = 8, extra: int = 24, seed: int = 0) -> torch.Tensor:
    """Rows that exercise the persistent quantizer's steady state: a CTA b of `ctas` takes the row
    pairs b, b + ctas, b + 2 ctas, ...; its k-th pair occupies ring stage k % ring.  Returned are both
    rows of the pairs k = 0, ring-1, ring, ring+1, middle, last-1, last of several CTAs (first, second,
    middle, last), plus the first and last rows of the tensor and `extra` random rows."""
    npairs = (tokens + 1) // 2
    per_cta = max(1, npairs // ctas)
    ks = sorted({0, ring - 1, ring, ring + 1, per_cta // 2, per_cta - 2, per_cta - 1})
    rows = set(range(min(4, tokens))) | set(range(max(0, tokens - 4), tokens))
    for b in (0, 1, ctas // 2, ctas - 1):
        for k in ks:
            pair = b + k * ctas
            if 0 <= pair < npairs:
                rows.update(r for r in (2 * pair, 2 * pair + 1) if r < tokens)
    g = torch.Generator().manual_seed(seed)
    rows.update(torch.randint(0, tokens, (extra,), generator=g).tolist())
    return torch.tensor(sorted(rows), dtype=torch.int64)


def sampled_rows_match_oracle(q, sf, rows: torch.Tensor, q_oracle: np.ndarray, sf_oracle: np.ndarray, k_eff: int):
    """Codes and every valid scale byte of the sampled rows of a large launch (q, sf: device tensors of
    the whole launch) against the oracle run on those rows alone (row j of the oracle = row rows[j])."""
    qg = q[rows.to(q.device)].cpu().numpy()
    bad = np.argwhere(qg != q_oracle)
    assert bad.size == 0, f"{len(bad)} code bytes differ, first (sample, byte) {bad[:4].tolist()}, rows {rows[bad[:4, 0]].tolist()}"
    ncols = k_eff // 16
    natoms = (ncols + 3) // 4
    c = np.arange(ncols, dtype=np.int64)[None, :]

    def offsets(r):
        r = np.asarray(r, dtype=np.int64)[:, None]
        return ((r // 128) * natoms + c // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (c % 4)

    og = offsets(rows.numpy())
    oo = offsets(np.arange(len(rows)))
    sg = sf.cpu().numpy()[og]
    so = np.asarray(sf_oracle)[oo]
    bad = np.argwhere(sg != so)
    assert bad.size == 0, f"{len(bad)} scale bytes differ, first (sample, column) {bad[:4].tolist()}, rows {rows[bad[:4, 0]].tolist()}"


def sf_take_rows(sf, rows, k_eff: int) -> np.ndarray:
    """Scale bytes of the sampled rows of a packed operand, re-laid out as the scale buffer of an operand
    that consists of those rows only (row j of the result = row rows[j] of the source)."""
    from oracle import oracle as O

    src = sf if isinstance(sf, np.ndarray) else sf.cpu().numpy()
    rows = np.asarray(rows, dtype=np.int64)
    ncols = k_eff // 16
    natoms = (ncols + 3) // 4
    c = np.arange(ncols, dtype=np.int64)[None, :]

    def offsets(r):
        r = np.asarray(r, dtype=np.int64)[:, None]
        return ((r // 128) * natoms + c // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (c % 4)

    out = np.zeros(O.sf_alloc_bytes(len(rows), k_eff), np.uint8)
    out[offsets(np.arange(len(rows)))] = src[offsets(rows)]
    return out

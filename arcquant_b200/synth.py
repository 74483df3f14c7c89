"""Seeded synthetic inputs with the shapes and value distributions of the
workloads this library is measured on.

The reference evaluates on WikiText-2 / lm-eval with real checkpoints; neither
is available offline, so every test and benchmark here draws from these
generators instead: N(0,1) activations with ~1 % outlier channels scaled by 50,
N(0, 0.02) weights, N(1, 0.1) RMSNorm gains, and a channel order obtained the
way the reference calibrates it (per-channel max |x| over a calibration batch,
ascending, so the outliers sit last: utilize.py:22-64 of the reference).
"""
from __future__ import annotations

import torch


def outlier_channels(hidden: int, count: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(hidden, generator=g)[:count]


def activations(tokens: int, hidden: int, seed: int, outliers: torch.Tensor | None = None,
                outlier_scale: float = 50.0, device="cpu") -> torch.Tensor:
    """bf16 [tokens, hidden] ~ N(0,1); the given channels are multiplied by 50."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g, device=device, dtype=torch.float32)
    if outliers is not None and len(outliers):
        x[:, outliers.to(x.device)] *= outlier_scale
    return x.to(torch.bfloat16)


def weights(n: int, k: int, seed: int, std: float = 0.02, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(n, k, generator=g, device=device, dtype=torch.float32) * std).to(torch.bfloat16)


def rms_gain(hidden: int, seed: int, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device).manual_seed(seed)
    return (1.0 + 0.1 * torch.randn(hidden, generator=g, device=device, dtype=torch.float32)).to(torch.bfloat16)


def reorder_index_from_stats(absmax: torch.Tensor) -> torch.Tensor:
    """Ascending argsort of the per-channel statistic -> int16 index, critical
    (largest) channels last."""
    assert absmax.numel() < 32768
    return torch.argsort(absmax.float().cpu(), stable=True).to(torch.int16)


def calibrate_reorder_index(hidden: int, outliers: torch.Tensor, seed: int, samples: int = 128,
                            seq: int = 2048, device="cpu") -> torch.Tensor:
    """Per-channel max |x| over ``samples`` x ``seq`` calibration tokens of the
    same distribution, drawn chunk by chunk."""
    stat = torch.zeros(hidden, dtype=torch.float32, device=device)
    for s in range(samples):
        x = activations(seq, hidden, seed * 100003 + s, outliers, device=device)
        stat = torch.maximum(stat, x.abs().amax(dim=0).float())
    return reorder_index_from_stats(stat)


def config1(seed: int = 0):
    """Single linear: X [512,4096] with 40 outlier channels, W [4096,4096], KE 128."""
    torch.manual_seed(seed)
    x = torch.randn(512, 4096, dtype=torch.float32)
    cols = torch.randperm(4096)[:40]
    x[:, cols] *= 50.0
    x = x.to(torch.bfloat16)
    w = (torch.randn(4096, 4096, dtype=torch.float32) * 0.02).to(torch.bfloat16)
    idx = reorder_index_from_stats(x.abs().amax(dim=0))
    return x, w, idx, 128


def global_scale(t: torch.Tensor) -> torch.Tensor:
    """Per-tensor scale amax/(6*448) as a 0-dim fp32 tensor (qLlamaLayer.py:74)."""
    return t.abs().max().float() / (448.0 * 6.0)

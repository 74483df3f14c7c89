"""Calibration rules against direct restatements of the reference's formulas (utilize.py:108,546-551;
reorder_indices.py): running channel maximum, ascending order, residual-width rule."""
import math

import torch

from arcquant_b200 import calibrate


def test_running_channel_maximum_and_order():
    g = torch.Generator().manual_seed(0)
    batches = [torch.randn(3, 17, 96, generator=g) * (1 + i) for i in range(4)]
    stat = calibrate.ChannelAbsMax()
    for b in batches:
        stat.update(b.to(torch.bfloat16))
    want = torch.stack([b.to(torch.bfloat16).reshape(-1, 96).abs().float().amax(0) for b in batches]).amax(0)
    assert torch.equal(stat.value, want)
    idx = stat.reorder_index()
    assert idx.dtype == torch.int16
    assert torch.equal(idx.long(), torch.argsort(want))
    assert want[idx.long()[-1]] == want.max()          # the largest channel comes last


def test_select_num_rule():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(64, 512, generator=g)
    x[:, :5] *= 40                                       # a few outlier channels raise the row maxima
    thr = x.max(dim=-1, keepdim=True)[0] * 0.125
    ratio = float((x > thr).sum()) / x.numel()
    want = min(math.ceil(512 * ratio / 64) * 64, 512)
    assert calibrate.select_num_rule(x) == want
    perm = torch.randperm(512, generator=g)
    assert calibrate.select_num_rule(x, perm) == want    # order-independent
    flat = torch.ones(4, 128)                            # every element exceeds an eighth of its row's maximum
    assert calibrate.select_num_rule(flat) == 128
    assert calibrate.average_bits(4096, 128) == 4.5 * 4224 / 4096

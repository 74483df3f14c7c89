"""The oracle's quantizer: pinned against outputs of the reference's own fake-quant path (golden
fixtures generated from the reference), and checked for the properties the reference kernels have."""
import hashlib
import json
import os

import numpy as np
import torch

from arcquant_b200 import synth
from oracle import fake_port as FP
from oracle import oracle as O
from tests.helpers import adversarial_rows, scaled_activations


def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a, dtype="<f4").tobytes()).hexdigest()


def _config1_slice(gold):
    x, w, idx, ke = synth.config1()
    rows = gold["rows"]
    xs = (x[:rows] / synth.global_scale(x)).contiguous()
    ws = (w[:rows] / synth.global_scale(w)).contiguous()
    return xs, ws, idx, ke


def test_oracle_structure_equals_reference_fake_path(golden_dir):
    """Same gather, 16-groups, block scales, e2m1 grid and residual structure as the reference:
    run with the fake path's arithmetic knobs (division, tie towards the more negative value, fp32
    residual) the oracle reproduces the reference's fake-quant values bit for bit."""
    gold = json.load(open(os.path.join(golden_dir, "reference_fake_config1.json")))
    xs, _, idx, ke = _config1_slice(gold)
    fv = O.fake_values(xs, idx.numpy(), ke)
    assert _sha(fv) == gold["x_values_sha256"]
    sl = np.load(os.path.join(golden_dir, "reference_fake_config1_slice.npz"))
    assert np.array_equal(fv[:4], sl["x_values"])


def test_kernel_arithmetic_differs_from_fake_path_only_at_ties_and_reciprocal(golden_dir):
    gold = json.load(open(os.path.join(golden_dir, "reference_fake_config1.json")))
    xs, _, idx, ke = _config1_slice(gold)
    kq = xs.shape[1]
    fv = O.fake_values(xs, idx.numpy(), ke)
    q, sf = O.quantize_x(xs, idx.numpy(), ke)
    deq = O.dequant(q, sf)
    g0 = (kq - ke) // 16
    main = np.concatenate([deq[:, :16 * g0]] + [deq[:, 16 * g0 + 32 * j:16 * g0 + 32 * j + 16] for j in range(ke // 16)], 1)
    mism = main != fv[:, :kq]
    assert mism.mean() < 0.015                       # ~0.7 % on this input
    # wherever they differ the two candidates are adjacent grid points (a tie or a 1-ulp product)
    xg = torch.index_select(xs, 1, idx.to(torch.int64)).float().numpy()
    worst = np.abs(main - fv[:, :kq])[mism]
    step = np.abs(xg).reshape(xg.shape[0], -1, 16).max(-1).repeat(16, axis=1)[mism] / 6 * 2.2
    assert (worst <= np.maximum(step, 1e-6)).all()


def test_fake_port_equals_reference_fake_path(golden_dir):
    gold = json.load(open(os.path.join(golden_dir, "reference_fake_config1.json")))
    xs, ws, idx, ke = _config1_slice(gold)
    i64 = idx.to(torch.int64)
    qx, sx = FP.fake_reorder_quantize_x(torch.index_select(xs, 1, i64), ke)
    qw, sw = FP.fake_reorder_quantize_w(torch.index_select(ws, 1, i64), ke)
    qx0, _ = FP.fake_reorder_quantize_x(torch.index_select(xs, 1, i64), 0)
    assert _sha(qx.float().numpy()) == gold["fake_x_sha256"]
    assert _sha(qw.float().numpy()) == gold["fake_w_sha256"]
    assert _sha(qx0.float().numpy()) == gold["fake_x_ke0_sha256"]
    sl = np.load(os.path.join(golden_dir, "reference_fake_config1_slice.npz"))
    assert np.array_equal(qx.float().numpy()[:4], sl["fake_x"])


def test_arc_residual_lowers_the_error():
    xs, idx = scaled_activations(64, 1024, seed=3)
    i64 = idx.to(torch.int64)
    xg = torch.index_select(xs, 1, i64).float().numpy()
    w = synth.weights(96, 1024, seed=4)
    ws = (w / synth.global_scale(w)).contiguous()
    wg = torch.index_select(ws, 1, i64).float().numpy()
    ref = xg @ wg.T
    errs = []
    for ke in (0, 64, 256):
        qa, sa = O.quantize_x(xs, idx.numpy(), ke)
        qb, sb = O.quantize_w(ws, idx.numpy(), ke)
        y = O.gemm_fast(qa, sa, qb, sb, 1.0)
        errs.append(np.linalg.norm(y - ref) / np.linalg.norm(ref))
    assert errs[2] < errs[1] < errs[0]


def test_residual_is_rounded_to_bf16_before_requantizing():
    """x = q*s + r exactly for the bf16-rounded r; the appended block is the NVFP4 of that r."""
    kq, ke = 64, 32
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(2, kq, generator=g) * 5).to(torch.bfloat16)
    q, sf = O.quantize_x(x, None, ke)
    deq = O.dequant(q, sf)
    g0 = (kq - ke) // 16
    for j in range(ke // 16):
        main = deq[:, 16 * g0 + 32 * j:16 * g0 + 32 * j + 16]
        src = x[:, 16 * (g0 + j):16 * (g0 + j) + 16].float().numpy()
        r = torch.from_numpy(src - main).to(torch.bfloat16)
        qr, sfr = O.quantize_x(r, None, 0)
        assert np.array_equal(qr, q[:, 8 * g0 + 16 * j + 8:8 * g0 + 16 * j + 16])


def test_adversarial_rows_decode_within_half_a_step():
    x = adversarial_rows(256)
    q, sf = O.quantize_x(x, None, 0)
    deq = O.dequant(q, sf)
    xf = x.float().numpy()
    amax = np.abs(xf).reshape(xf.shape[0], -1, 16).max(-1).repeat(16, axis=1)
    # values inside the representable range of their block (|x| <= 6*448) are within one grid step
    ok = amax <= 6 * 448
    # block scales in the ue4m3 subnormal range move in steps of 2^-9: allow six half-steps on top
    assert (np.abs(deq - xf)[ok] <= amax[ok] / 6 * 1.07 + 6 * 2.0 ** -10).all()
    assert np.isfinite(deq).all()


def test_rmsnorm_oracle_tracks_fp32_rmsnorm():
    kq = 2048
    out = synth.outlier_channels(kq, 20, 1)
    x = synth.activations(16, kq, 2, out)
    gamma = synth.rms_gain(kq, 3)
    idx = synth.reorder_index_from_stats(x.abs().amax(0))
    q, sf = O.quantize_x(x, idx.numpy(), 0, gamma=gamma, eps=1e-5)
    deq = O.dequant(q, sf)
    xf = x.float()
    ref = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * gamma.float())[:, idx.to(torch.int64)].numpy()
    amax = np.abs(ref).reshape(16, -1, 16).max(-1).repeat(16, axis=1)
    assert (np.abs(deq - ref) <= amax / 6 * 1.07 + np.abs(ref) * 2 ** -7).all()
    assert np.linalg.norm(deq - ref) / np.linalg.norm(ref) < 0.2


def test_rmsnorm_sum_order_is_the_references():
    """A row whose naive left-to-right fp32 sum differs from the reference's thread/tree order."""
    kq = 2048
    x = torch.zeros(1, kq)
    x[0, 0] = 4096.0
    x[0, 8:] = 0.0443                    # many tiny squares that a sequential sum would absorb differently
    x = x.to(torch.bfloat16)
    gamma = torch.ones(kq, dtype=torch.bfloat16)
    q, sf = O.quantize_x(x, None, 0, gamma=gamma, eps=1e-5)
    # reference order: thread t sums chunk t then chunk t+128 (8 values each), then the tree
    v = x.float().numpy()[0].astype(np.float32)
    part = np.zeros(128, np.float32)
    for t in range(128):
        acc = np.float32(0)
        for i in list(range(8 * t, 8 * t + 8)) + list(range(8 * (128 + t), 8 * (128 + t) + 8)):
            acc = np.float32(np.float32(v[i] * v[i]) + acc)
        part[t] = acc
    s = part.copy()
    for t in range(64):
        s[t] = s[t] + s[t + 64]
    for t in range(32):
        s[t] = s[t] + s[t + 32]
    for sh in (16, 8, 4, 2, 1):
        for t in range(sh):
            s[t] = s[t] + s[t + sh]
    rstd = np.float32(O.lib().arcq_rsqrt_rn(float(np.float32(s[0] / np.float32(kq)) + np.float32(1e-5))))
    xn = torch.from_numpy((v * rstd).astype(np.float32)).to(torch.bfloat16).reshape(1, kq)
    q2, sf2 = O.quantize_x(xn, None, 0)
    assert np.array_equal(q, q2)
    assert np.array_equal(sf, sf2)


def test_oracle_rejects_shapes_the_layout_cannot_express():
    x = torch.zeros(2, 40, dtype=torch.bfloat16)
    for bad in ((x, 0, 16), (torch.zeros(2, 64, dtype=torch.bfloat16), 8, 16), (torch.zeros(2, 48, dtype=torch.bfloat16), 16, 32)):
        try:
            O.quantize_x(bad[0], None, bad[1], mode=bad[2])
        except ValueError:
            continue
        raise AssertionError("shape accepted")

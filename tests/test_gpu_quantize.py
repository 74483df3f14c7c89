"""Parity of the CUDA quantizer with the CPU oracle, through the C ABI (ctypes): packed e2m1 codes
and ue4m3 scale bytes must be bit-exact."""
import numpy as np
import pytest
import torch

from arcquant_b200 import synth
from tests.helpers import (adversarial_rows, sampled_rows_match_oracle, scaled_activations, steady_state_rows,
                           valid_sf)

pytestmark = pytest.mark.gpu


def _ops():
    from arcquant_b200 import ops
    return ops


def _oracle():
    from oracle import oracle as O
    return O


def _check(kind, x, idx, ke, mode, gamma=None, eps=0.0):
    ops, O = _ops(), _oracle()
    dev = torch.device("cuda:0")
    xd = x.to(dev)
    idxd = None if idx is None else idx.to(dev)
    if kind == "x":
        q, sf = ops.reorder_quantize_x(xd, idxd, ke, mode=mode)
        qo, sfo = O.quantize_x(x, None if idx is None else idx.numpy(), ke, mode=mode)
    elif kind == "w":
        q, sf = ops.reorder_quantize_w(xd, idxd, ke, mode=mode)
        qo, sfo = O.quantize_w(x, None if idx is None else idx.numpy(), ke, mode=mode)
    else:
        q, sf = ops.rmsnorm_quantize_x(xd, gamma.to(dev), eps, idxd, ke)
        qo, sfo = O.quantize_x(x, None if idx is None else idx.numpy(), ke, mode=16, gamma=gamma, eps=eps)
    torch.cuda.synchronize()
    rows, kq = x.shape
    qg = q.cpu().numpy()
    assert qg.shape == qo.shape
    bad = np.argwhere(qg != qo)
    assert bad.size == 0, f"{len(bad)} code bytes differ, first at {bad[:5].tolist()}: gpu {qg[tuple(bad[0])]:#x} oracle {qo[tuple(bad[0])]:#x}"
    sg, so = valid_sf(sf, rows, kq + ke), valid_sf(sfo, rows, kq + ke)
    bad = np.argwhere(sg != so)
    assert bad.size == 0, f"{len(bad)} scale bytes differ, first {bad[:5].tolist()}"
    assert sf.numel() >= O.sf_bytes_reference(rows, kq + ke)


@pytest.mark.parametrize("tokens", [1, 16, 128, 1024])
@pytest.mark.parametrize("ke", [0, 64, 128, 256])
def test_reorder_quantize_x_hidden4096(tokens, ke):
    xs, idx = scaled_activations(tokens, 4096, seed=100 + tokens + ke)
    _check("x", xs, idx, ke, 16)


@pytest.mark.parametrize("kq,ke,mode,tokens", [
    (2048, 128, 16, 33), (3072, 64, 16, 7), (5120, 128, 16, 5), (8192, 256, 16, 9), (11008, 128, 16, 4),
    (13824, 64, 16, 3), (14336, 128, 16, 130), (3584, 64, 32, 19), (18944, 128, 32, 5), (512, 512, 16, 6),
    (1792, 16, 16, 11), (64, 0, 16, 257)])
def test_reorder_quantize_x_other_widths(kq, ke, mode, tokens):
    xs, idx = scaled_activations(tokens, kq, seed=kq + ke)
    _check("x", xs, idx, ke, mode)


@pytest.mark.parametrize("kq", [27648, 28672])
def test_pre_gathered_wide_rows_mode32(kq):
    xs, _ = scaled_activations(3, kq, seed=kq)
    _check("x", xs, None, 128, 32)          # identity order: the caller gathered beforehand
    w = synth.weights(4, kq, seed=1)
    _check("w", (w / synth.global_scale(w)).contiguous(), None, 128, 32)


def test_rounding_boundaries_and_signed_zeros():
    x = adversarial_rows(4096)
    idx = torch.randperm(4096, generator=torch.Generator().manual_seed(3)).to(torch.int16)
    _check("x", x, idx, 128, 16)
    _check("x", x, None, 0, 16)
    _check("x", adversarial_rows(3584), None, 64, 32)


@pytest.mark.parametrize("kq,ke,mode", [(1024, 64, 16), (4096, 128, 16), (3584, 64, 32), (1792, 64, 16)])
def test_every_block_maximum(kq, ke, mode):
    """Every finite bf16 magnitude (all 32640 bit patterns) as the maximum of some block: covers every
    block scale the format has, the subnormal and the saturated ones included, in main and residual
    slots."""
    g = torch.Generator().manual_seed(kq)
    groups = kq // 16
    rows = (0x7f80 + groups - 1) // groups
    bits = (torch.arange(rows * groups, dtype=torch.int32) % 0x7f80).reshape(rows, groups)
    amax = (bits.to(torch.int16)).view(torch.bfloat16).float()                       # [rows, groups]
    frac = torch.rand(rows, groups, 16, generator=g)
    frac[..., 0] = 1.0
    perm = torch.argsort(torch.rand(rows, groups, 16, generator=g), dim=-1)          # position of the maximum
    frac = torch.gather(frac, -1, perm)
    sign = torch.where(torch.rand(rows, groups, 16, generator=g) < 0.5, -1.0, 1.0)
    x = (amax[..., None] * frac).to(torch.bfloat16).float() * sign
    x = x.reshape(rows, kq).to(torch.bfloat16).contiguous()
    _check("x", x, None, ke, mode)
    idx = torch.randperm(kq, generator=g).to(torch.int16)
    _check("x", x, idx, ke, mode)


@pytest.mark.parametrize("kq,ke", [(4096, 128), (14336, 128), (11008, 64), (2048, 64), (7168, 64), (1024, 64),
                                   (3584, 64), (512, 64), (1792, 64)])
def test_fused_division_by_the_tensor_scale(kq, ke):
    """reorder_quantize_x(x, scale=s) must give the bytes of reorder_quantize_x(x / s): every bf16 bit
    pattern (zeros of both signs, subnormals, infinities excluded) against a spread of divisors.
    (11008, 1792 and 512 are widths the fused kernel does not cover: the operator divides first.  The
    widths with 64 residual channels are the row-parallel shards of a Llama-3-8B layer over 2, 4 and 8
    ranks.)"""
    ops = _ops()
    g = torch.Generator().manual_seed(kq)
    bits = torch.arange(65536, dtype=torch.int32)
    bits = bits[(bits & 0x7f80) != 0x7f80]                                   # finite values only
    n = (bits.numel() // kq + 1) * kq
    vals = bits[torch.randint(0, bits.numel(), (n,), generator=g)]
    vals[:bits.numel()] = bits
    x = vals.to(torch.int16).view(torch.bfloat16).reshape(-1, kq).contiguous().cuda()
    idx = torch.randperm(kq, generator=g).to(torch.int16).cuda()
    scales = [1.0, 3.0, 0.3721, 1.9999999, 7.0e-4, 2.688e3, 1.0000001, 5.960464e-8, 1.5e9, 0.99999994, 1e-25, 1e25,
              1e-35, 3e35]
    scales += [float(v) for v in torch.rand(12, generator=g) * 4 + 1e-3]
    for sv in scales:
        sc = torch.tensor(sv, dtype=torch.float32, device="cuda")
        q, sf = ops.reorder_quantize_x(x, idx, ke, scale=sc)
        q2, sf2 = ops.reorder_quantize_x(x / sc, idx, ke)
        assert torch.equal(q, q2), f"codes differ for divisor {sv}"
        a, b = valid_sf(sf, x.shape[0], kq + ke), valid_sf(sf2, x.shape[0], kq + ke)
        assert (a == b).all(), f"scales differ for divisor {sv}"


@pytest.mark.parametrize("kq", [2048, 3072, 3584, 4096, 5120, 8192])
@pytest.mark.parametrize("tokens", [1, 130])
def test_rmsnorm_quantize_x(kq, tokens):
    out = synth.outlier_channels(kq, kq // 100, 5)
    x = synth.activations(tokens, kq, 17 + kq, out)
    gamma = synth.rms_gain(kq, 3)
    idx = synth.reorder_index_from_stats(synth.activations(256, kq, 9, out).abs().amax(0))
    _check("rms", x, idx, 128, 16, gamma=gamma, eps=1e-5)
    if kq == 4096:
        for ke in (0, 64, 256):
            _check("rms", x, idx, ke, 16, gamma=gamma, eps=1e-5)


def test_rmsnorm_rows_with_extreme_norms():
    kq = 4096
    x = adversarial_rows(kq)
    gamma = synth.rms_gain(kq, 4)
    _check("rms", x, None, 128, 16, gamma=gamma, eps=1e-6)


@pytest.mark.parametrize("kq,ke,mode,n", [(4096, 128, 16, 300), (14336, 128, 16, 40), (3584, 64, 32, 64), (4096, 0, 16, 17)])
def test_reorder_quantize_w(kq, ke, mode, n):
    w = synth.weights(n, kq, seed=kq + n)
    ws = (w / synth.global_scale(w)).contiguous()
    idx = torch.randperm(kq, generator=torch.Generator().manual_seed(kq)).to(torch.int16)
    _check("w", ws, idx, ke, mode)


def test_full_size_is_row_independent_and_matches_oracle_on_samples():
    """32768 tokens x 4096: too large for the scalar oracle as a whole, so (a) quantizing the halves
    separately must give the same bytes as quantizing everything (rows are independent), (b) a
    spread of rows is checked against the oracle, (c) a checksum over everything is stable across
    two runs."""
    ops, O = _ops(), _oracle()
    tokens, kq, ke = 32768, 4096, 128
    dev = torch.device("cuda:0")
    out = synth.outlier_channels(kq, 41, 1)
    x = synth.activations(tokens, kq, 2, out, device=dev)
    idx = synth.reorder_index_from_stats(x[:4096].abs().amax(0)).to(dev)
    q, sf = ops.reorder_quantize_x(x, idx, ke)
    q2, sf2 = ops.reorder_quantize_x(x, idx, ke)
    assert torch.equal(q, q2)
    qa, sfa = ops.reorder_quantize_x(x[:16384].contiguous(), idx, ke)
    qb, sfb = ops.reorder_quantize_x(x[16384:].contiguous(), idx, ke)
    assert torch.equal(q[:16384], qa) and torch.equal(q[16384:], qb)
    span = O.sf_bytes_span(16384, kq + ke)
    assert torch.equal(sf[:span], sfa[:span]) and torch.equal(sf[span:2 * span], sfb[:span])
    rows = torch.cat([torch.arange(0, 8), torch.arange(16380, 16388), torch.arange(tokens - 8, tokens),
                      torch.randint(0, tokens, (40,), generator=torch.Generator().manual_seed(0))])
    xs = x[rows.to(dev)].cpu()
    qo, sfo = O.quantize_x(xs, idx.cpu().numpy(), ke)
    assert np.array_equal(q[rows.to(dev)].cpu().numpy(), qo)
    ncols = (kq + ke) // 16
    sfh = sf.cpu().numpy()
    for j, r in enumerate(rows.tolist()):
        for c in (0, 1, 131, 247, 248, 249, 263):
            assert sfh[O.sf_offset(r, c, ncols)] == sfo[O.sf_offset(j, c, ncols)]


# ---- steady state of the persistent kernels: many row pairs per CTA, rings wrapping ----------------
# The launches below are too large for the scalar oracle as a whole; rows are independent, so the
# oracle runs on a sample chosen to hit the first, ring-wrapping, middle and last pairs of several
# CTAs (see tests.helpers.steady_state_rows).


def _big_inputs(tokens, kq, seed):
    dev = torch.device("cuda:0")
    out = synth.outlier_channels(kq, max(1, kq // 100), seed)
    x = synth.activations(tokens, kq, seed + 1, out, device=dev)
    idx = synth.reorder_index_from_stats(x[:2048].abs().amax(0))
    return x, idx


@pytest.mark.parametrize("tokens", [1024, 8192, 32768])
@pytest.mark.parametrize("ke", [0, 64, 128, 256])
def test_rmsnorm_quantize_x_steady_state(tokens, ke):
    """Fused RMSNorm at the token counts of the kernel-alone benchmark grid (hidden 4096): every CTA
    takes up to 111 row pairs, both producer teams alternate, raw and gather rings wrap many times."""
    ops, O = _ops(), _oracle()
    kq = 4096
    x, idx = _big_inputs(tokens, kq, 40 + ke)
    gamma = synth.rms_gain(kq, 3)
    q, sf = ops.rmsnorm_quantize_x(x, gamma.cuda(), 1e-5, idx.cuda(), ke)
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    rows = steady_state_rows(tokens)
    qo, sfo = O.quantize_x(x[rows.cuda()].cpu(), idx.numpy(), ke, gamma=gamma, eps=1e-5)
    sampled_rows_match_oracle(q, sf, rows, qo, sfo, kq + ke)


@pytest.mark.parametrize("kq", [2048, 3072, 3584, 5120, 8192])
def test_rmsnorm_quantize_x_steady_state_other_widths(kq):
    ops, O = _ops(), _oracle()
    tokens, ke = 16384, 128
    x, idx = _big_inputs(tokens, kq, kq)
    gamma = synth.rms_gain(kq, 5)
    q, sf = ops.rmsnorm_quantize_x(x, gamma.cuda(), 1e-5, idx.cuda(), ke)
    rows = steady_state_rows(tokens)
    qo, sfo = O.quantize_x(x[rows.cuda()].cpu(), idx.numpy(), ke, gamma=gamma, eps=1e-5)
    sampled_rows_match_oracle(q, sf, rows, qo, sfo, kq + ke)


@pytest.mark.parametrize("kq,tokens", [(14336, 16384), (8192, 16384), (14336, 16383), (1024, 40000), (7168, 8192),
                                       (3584, 8192), (1792, 8192), (512, 8192)])
def test_reorder_quantize_x_steady_state_wide_and_shard_widths(kq, tokens):
    """Plain operator at the down projection's width (half-pair raw ring), at an odd row count, and at
    the row-parallel shard widths of 2, 4 and 8 ranks."""
    ops, O = _ops(), _oracle()
    ke = 128 if kq >= 4096 else 64
    x, idx = _big_inputs(tokens, kq, kq + 1)
    mode = O.reference_mode(kq)
    q, sf = ops.reorder_quantize_x(x, idx.cuda(), ke, mode=mode)
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    rows = steady_state_rows(tokens, ring=3 if kq > 8192 else 8)
    qo, sfo = O.quantize_x(x[rows.cuda()].cpu(), idx.numpy(), ke, mode=mode)
    sampled_rows_match_oracle(q, sf, rows, qo, sfo, kq + ke)


@pytest.mark.parametrize("kq,tokens", [(4096, 16384), (14336, 16384), (4096, 32767), (7168, 8192), (2048, 8192),
                                       (3584, 8192), (1024, 8192), (1792, 8192), (512, 8192)])
def test_fused_division_steady_state(kq, tokens):
    """`scale=` (division by the per-tensor scale fused into the quantizer) at layer sizes, against the
    oracle fed torch's own CUDA quotient x / scale - the reference callers' pre-scaling
    (model/qLlamaLayer.py:73-77 of ARCQuant)."""
    ops, O = _ops(), _oracle()
    ke = 128 if kq >= 4096 else 64
    x, idx = _big_inputs(tokens, kq, kq + 2)
    mode = O.reference_mode(kq)
    scale = ops.absmax(x) / 2688.0
    q, sf = ops.reorder_quantize_x(x, idx.cuda(), ke, mode=mode, scale=scale)
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    rows = steady_state_rows(tokens, ring=3 if kq > 8192 else 8)
    xs = (x[rows.cuda()] / scale).cpu()
    qo, sfo = O.quantize_x(xs, idx.numpy(), ke, mode=mode)
    sampled_rows_match_oracle(q, sf, rows, qo, sfo, kq + ke)


def test_reference_script_distribution_seed_45510():
    """The input distribution of the reference's own manual check (kernels/main.py:8-33 of ARCQuant),
    restated: seed 45510, 128 x 4096 uniform magnitudes in [0, 3) with random signs, the last 384
    channels in [3, 6), the last 128 in [8, 16), the last 16 in [32, 64); identity channel order;
    residual widths 0, 256, ..., 4096; activations and weights divided by max|.| / 2688 first.  (The
    reference draws on the GPU, so the values differ; the distribution and the sweep are the same.)"""
    ops, O = _ops(), _oracle()
    g = torch.Generator().manual_seed(45510)
    m, n, kq = 128, 64, 4096
    sign = torch.randint(0, 2, (m, kq), generator=g).float() * 2 - 1
    x = torch.rand(m, kq, generator=g) * 3
    x[:, -384:] = torch.rand(m, 384, generator=g) * 3 + 3
    x[:, -128:] = torch.rand(m, 128, generator=g) * 8 + 8
    x[:, -16:] = torch.rand(m, 16, generator=g) * 32 + 32
    x = (x * sign).to(torch.bfloat16)
    w = (torch.rand(n, kq, generator=g) * 3).to(torch.bfloat16)
    idx = torch.arange(kq, dtype=torch.int16)
    xs = (x / (x.abs().max().float() / 2688.0)).contiguous()
    ws = (w / (w.abs().max().float() / 2688.0)).contiguous()
    for ke in range(0, kq + 1, kq // 16):
        _check("x", xs, idx, ke, 16)
        _check("w", ws, idx, ke, 16)


def test_absmax():
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    for n in (1, 7, 8, 4096, 1 << 20, (1 << 20) + 5):
        x = (torch.randn(n, generator=g) * 3).to(torch.bfloat16).cuda()
        assert float(ops.absmax(x)) == float(x.abs().max().float())


def test_runs_on_the_current_stream_and_device_memory_only():
    ops = _ops()
    xs, idx = scaled_activations(64, 4096, seed=1)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        xd, idxd = xs.cuda(non_blocking=True), idx.cuda(non_blocking=True)
        q, sf = ops.reorder_quantize_x(xd, idxd, 128)
    s.synchronize()
    O = _oracle()
    qo, _ = O.quantize_x(xs, idx.numpy(), 128)
    assert np.array_equal(q.cpu().numpy(), qo)


@pytest.mark.parametrize("rows,kq,ke,nd", [(4096, 4096, 128, 4), (256, 4096, 128, 8), (2048, 2048, 64, 2), (1024, 8192, 256, 3)])
def test_fused_operator_storing_its_output_several_times(rows, kq, ke, nd):
    """`rmsnorm_quantize_x_multi`: the same bytes at every destination (here local buffers standing for the
    peers' gathered buffers, each at its own offset inside a larger guarded allocation), equal to the
    single-destination operator, which the other tests hold to the oracle."""
    from arcquant_b200 import ops

    dev = "cuda:0"
    x = synth.activations(rows, kq, rows + 1, synth.outlier_channels(kq, kq // 100, 2), device=dev)
    gain = (1.0 + 0.1 * torch.randn(kq, generator=torch.Generator().manual_seed(5))).to(torch.bfloat16).to(dev)
    idx = synth.reorder_index_from_stats(x[:256].abs().amax(0)).to(dev)
    q_ref, sf_ref = ops.rmsnorm_quantize_x(x, gain, 1e-5, idx, ke)
    k_eff = kq + ke
    tile = ((k_eff // 16 + 3) // 4) * 512
    span = (rows // 128) * tile
    qbuf = torch.full((nd, 3 * rows, k_eff // 2), 0x5A, dtype=torch.uint8, device=dev)
    sfbuf = torch.full((nd, 3 * span), 0x5A, dtype=torch.uint8, device=dev)
    ops.rmsnorm_quantize_x_multi(x, gain, 1e-5, idx, ke, [qbuf[d, rows:].data_ptr() for d in range(nd)],
                                 [sfbuf[d, span:].data_ptr() for d in range(nd)])
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    for d in range(nd):
        assert torch.equal(qbuf[d, rows:2 * rows], q_ref), d
        assert torch.equal(sfbuf[d, span:2 * span], sf_ref[:span]), d
        assert bool((qbuf[d, :rows] == 0x5A).all()) and bool((qbuf[d, 2 * rows:] == 0x5A).all())
        assert bool((sfbuf[d, :span] == 0x5A).all()) and bool((sfbuf[d, 2 * span:] == 0x5A).all())

"""Parity of the tcgen05 block-scaled NVFP4 GEMM with the oracle's dequantised fp32 matmul.

The kernel's output type is bf16 (as the reference's).  Rounding an exact result to bf16 alone puts
a relative Frobenius distance of ~1.6e-3 between it and the fp32 value (uniform error of half a
7-bit-mantissa ulp), so the 1e-3 tolerance is applied where it is meaningful: between the kernel's
output and the oracle's result rounded to the same output type - what remains is only the fp32
accumulation order, a handful of one-ulp flips.  The raw distance to the unrounded fp32 oracle is
bounded separately by the rounding floor."""
import numpy as np
import pytest
import torch

from arcquant_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 1e-3


def _ops():
    from arcquant_b200 import ops
    return ops


def _oracle():
    from oracle import oracle as O
    return O


def _operands(m, n, kq, ke, seed):
    """Packed operands made by the ORACLE from seeded N(0,1) activations / N(0,0.02) weights."""
    O = _oracle()
    out = synth.outlier_channels(kq, max(1, kq // 100), seed)
    x = synth.activations(m, kq, seed + 1, out)
    w = synth.weights(n, kq, seed + 2)
    sx, sw = synth.global_scale(x), synth.global_scale(w)
    idx = synth.reorder_index_from_stats(synth.activations(128, kq, seed + 3, out).abs().amax(0)).numpy()
    a, sfa = O.quantize_x((x / sx).contiguous(), idx, ke)
    b, sfb = O.quantize_w((w / sw).contiguous(), idx, ke)
    return a, sfa, b, sfb, float(sx * sw)


def _run(a, sfa, b, sfb, alpha):
    ops = _ops()
    dev = "cuda:0"
    t = [torch.from_numpy(v).to(dev) for v in (a, b, sfa, sfb)]
    c = ops.matmul(t[0], t[1], t[2], t[3], alpha)
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    return c.float().cpu().numpy()


BF16_FLOOR = 2.2e-3     # relative Frobenius distance that bf16 rounding of the output alone may cause


def _relerr(c, ref):
    return float(np.linalg.norm(c - ref) / max(np.linalg.norm(ref), 1e-30))


def _to_bf16(ref):
    return torch.from_numpy(np.ascontiguousarray(ref)).to(torch.bfloat16).float().numpy()


def _assert_close(c, ref):
    """c: kernel output (bf16 values as fp32); ref: fp32 oracle."""
    refb = _to_bf16(ref)
    assert _relerr(c, refb) <= TOL, ("vs oracle rounded to bf16", _relerr(c, refb))
    assert (c == refb).mean() >= 0.99            # all but accumulation-order flips are bit-equal
    assert _relerr(c, ref) <= BF16_FLOOR, ("vs fp32 oracle", _relerr(c, ref))


def test_one_hot_operands_land_where_they_should():
    """A single non-zero code in A and in B with unit scales: exactly one output element is set.
    Catches nibble order, swizzle, K-step and scale-atom placement errors by position."""
    O = _oracle()
    m, n, k = 128, 256, 512
    ncols = k // 16
    for (am, ak, bn, bk) in [(0, 0, 0, 0), (5, 1, 9, 1), (127, 511, 255, 511), (64, 70, 130, 70), (33, 200, 7, 200),
                             (99, 321, 200, 321)]:
        a = np.zeros((m, k // 2), np.uint8); b = np.zeros((n, k // 2), np.uint8)
        sfa = np.zeros(O.sf_alloc_bytes(m, k), np.uint8); sfb = np.zeros(O.sf_alloc_bytes(n, k), np.uint8)
        a[am, ak // 2] = 0x2 << (4 * (ak & 1))          # +1.0
        b[bn, bk // 2] = 0x4 << (4 * (bk & 1))          # +2.0
        sfa[O.sf_offset(am, ak // 16, ncols)] = 0x38    # 1.0
        sfb[O.sf_offset(bn, bk // 16, ncols)] = 0x40    # 2.0
        c = _run(a, sfa, b, sfb, 1.0)
        want = np.zeros((m, n), np.float32); want[am, bn] = 4.0
        assert np.array_equal(c, want), (am, ak, bn, bk, np.argwhere(c != 0)[:4].tolist())


def test_exact_small_integers():
    """Codes in {0, +-1, +-2} with scales in {1, 2} and K=64: every partial sum is a small integer,
    so the bf16 result is exact."""
    O = _oracle()
    rng = np.random.default_rng(0)
    m, n, k = 128, 128, 64
    lut = np.array([0x0, 0x2, 0xA, 0x4, 0xC], np.uint8)
    ca = lut[rng.integers(0, 5, (m, k))]; cb = lut[rng.integers(0, 5, (n, k))]
    a = (ca[:, 0::2] | (ca[:, 1::2] << 4)).astype(np.uint8); b = (cb[:, 0::2] | (cb[:, 1::2] << 4)).astype(np.uint8)
    sfa = np.zeros(O.sf_alloc_bytes(m, k), np.uint8); sfb = np.zeros(O.sf_alloc_bytes(n, k), np.uint8)
    for r in range(128):
        for c in range(4):
            sfa[O.sf_offset(r, c, 4)] = 0x38 if (r + c) % 2 else 0x40
            sfb[O.sf_offset(r, c, 4)] = 0x40 if (r * c) % 3 else 0x38
    ref = O.gemm(a, sfa, b, sfb, 1.0)
    c = _run(a, sfa, b, sfb, 1.0)
    assert np.array_equal(c, ref)


@pytest.mark.parametrize("m,n,kq,ke", [
    (1, 128, 64, 0), (16, 256, 256, 64), (128, 256, 1024, 0), (130, 264, 448, 64), (257, 512, 4096, 128),
    (128, 6144, 4096, 128), (64, 4096, 14336, 128), (300, 1000, 1984, 64), (16, 28672, 4096, 128)])
def test_matches_dequantised_fp32_matmul(m, n, kq, ke):
    O = _oracle()
    a, sfa, b, sfb, alpha = _operands(m, n, kq, ke, seed=m + n)
    ref = O.gemm_fast(a, sfa, b, sfb, alpha)
    c = _run(a, sfa, b, sfb, alpha)
    _assert_close(c, ref)


def test_tail_k_stage_and_garbage_in_scale_padding():
    """K_eff = 4224 is 16.5 stages of 256: the last stage is half.  Scale bytes outside the valid
    region are poisoned with NaN codes and must never reach an output."""
    O = _oracle()
    m, n, kq, ke = 100, 136, 4096, 128
    a, sfa, b, sfb, alpha = _operands(m, n, kq, ke, seed=5)
    ref = O.gemm_fast(a, sfa, b, sfb, alpha)
    for arr, rows in ((sfa, m), (sfb, n)):
        keep = np.zeros(arr.size, bool); keep[O.sf_valid_offsets(rows, kq + ke)] = True
        arr[~keep] = 0x7F
    c = _run(a, sfa, b, sfb, alpha)
    assert np.isfinite(c).all()
    _assert_close(c, ref)


def test_device_resident_alpha():
    ops, O = _ops(), _oracle()
    a, sfa, b, sfb, alpha = _operands(64, 256, 512, 64, seed=11)
    t = [torch.from_numpy(v).cuda() for v in (a, b, sfa, sfb)]
    sa = torch.tensor(alpha ** 0.5, dtype=torch.float32, device="cuda")
    c1 = ops.matmul_dev_alpha(t[0], t[1], t[2], t[3], sa, sa).float().cpu().numpy()
    ref = O.gemm_fast(a, sfa, b, sfb, float(np.float32(alpha ** 0.5)) ** 2)
    _assert_close(c1, ref)


@pytest.mark.parametrize("m,n,kq", [(4096, 4096, 4096), (16384, 6144, 4096), (4096, 4096, 14336)])
def test_large_shapes_by_row_independence_and_samples(m, n, kq):
    """Full BASELINE shapes: the scalar oracle checks a sample of output rows; the rest is covered
    by row independence (the GEMM of a row subset equals the subset of the GEMM)."""
    ops, O = _ops(), _oracle()
    ke = 128
    dev = "cuda:0"
    out = synth.outlier_channels(kq, kq // 100, 1)
    x = synth.activations(m, kq, 2, out, device=dev)
    w = synth.weights(n, kq, 3, device=dev)
    idx = synth.reorder_index_from_stats(x[:2048].abs().amax(0)).to(dev)
    sx, sw = ops.absmax(x) / 2688.0, ops.absmax(w) / 2688.0
    a, sfa = ops.reorder_quantize_x((x / sx).to(torch.bfloat16), idx, ke)
    b, sfb = ops.reorder_quantize_w((w / sw).to(torch.bfloat16), idx, ke)
    alpha = float(sx * sw)
    c = ops.matmul(a, b, sfa, sfb, alpha)
    assert ops.gemm_poll_error() == 0
    rows = torch.cat([torch.arange(0, 4), torch.arange(m - 4, m), torch.randint(0, m, (24,), generator=torch.Generator().manual_seed(1))])
    asub = a[rows.to(dev)].contiguous()
    # scales of the sampled rows, re-laid out for a 32-row operand
    ncols = (kq + ke) // 16
    sfh = sfa.cpu().numpy()
    sfsub = np.zeros(O.sf_alloc_bytes(len(rows), kq + ke), np.uint8)
    cols = np.arange(ncols)
    for j, r in enumerate(rows.tolist()):
        src = ((r // 128) * ((ncols + 3) // 4) + cols // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + cols % 4
        dst = (cols // 4) * 512 + (j % 32) * 16 + ((j // 32) % 4) * 4 + cols % 4
        sfsub[dst] = sfh[src]
    csub = ops.matmul(asub, b, torch.from_numpy(sfsub).to(dev), sfb, alpha)
    # (a skinny problem may be split over K: same products, fp32 partial sums added in another order,
    # so a few outputs can land on the neighbouring bf16 value)
    ref_rows = c[rows.to(dev)]
    same = (csub == ref_rows).float().mean().item()
    rel = ((csub.float() - ref_rows.float()).norm() / ref_rows.float().norm()).item()
    assert same > 0.995 and rel < 1e-3, (same, rel)
    ref = O.gemm_fast(asub.cpu().numpy(), sfsub, b.cpu().numpy(), sfb.cpu().numpy(), alpha)
    _assert_close(csub.float().cpu().numpy(), ref)
    # and against the unquantised product the ARC error stays in the expected band
    y = (x[rows.to(dev)].float() @ w.float().T).cpu().numpy()
    assert _relerr(csub.float().cpu().numpy(), y) < 0.2


@pytest.mark.parametrize("m,n,kq,ke", [(1, 4096, 4096, 128), (16, 4096, 4096, 128), (128, 4096, 14336, 128), (100, 1000, 1984, 64),
                                        (256, 2048, 1024, 64)])
def test_split_k_for_skinny_problems(m, n, kq, ke):
    """Few output tiles: K is cut over otherwise idle SMs, fp32 partials in caller-provided scratch,
    summed in a fixed order.  Same answer as the unsplit kernel up to fp32 summation order, and
    bit-stable; without scratch (third call) the problem runs unsplit."""
    import ctypes

    from arcquant_b200 import _lib

    O = _oracle()
    a, sfa, b, sfb, alpha = _operands(m, n, kq, ke, seed=m + n + 1)
    ref = O.gemm_fast(a, sfa, b, sfb, alpha)
    L = _lib.load()
    t = [torch.from_numpy(v).cuda() for v in (a, b, sfa, sfb)]
    k_eff = kq + ke
    ws_bytes = int(L.arcq_matmul_workspace_bytes(m, n, k_eff))
    assert ws_bytes > 0 and ws_bytes % (m * n * 4) == 0          # these shapes are split
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
    outs = []
    for wsp, wsb in ((ws.data_ptr(), ws_bytes), (ws.data_ptr(), ws_bytes), (None, 0)):
        c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        rc = L.arcq_matmul_nvfp4_ws(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), m, n, k_eff,
                                    alpha, None, None, c.data_ptr(), wsp, wsb, None)
        assert rc == 0
        torch.cuda.synchronize()
        outs.append(c.float().cpu().numpy())
    assert _ops().gemm_poll_error() == 0
    assert np.array_equal(outs[0], outs[1])                       # deterministic
    for c in outs:
        _assert_close(c, ref)
    # too small a workspace silently falls back to the unsplit kernel
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    assert L.arcq_matmul_nvfp4_ws(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), m, n, k_eff,
                                  alpha, None, None, c.data_ptr(), ws.data_ptr(), 16, None) == 0
    torch.cuda.synchronize()
    assert np.array_equal(c.float().cpu().numpy(), outs[2])


@pytest.mark.parametrize("m,n", [(1000, 4104), (4100, 4104), (1000, 28672), (16383, 4104), (300, 9992), (4100, 28672)])
def test_cta_pair_kernel_on_ragged_tiles(m, n):
    """Shapes that select the CTA-pair kernel (256 x 256 tiles) with M and/or N that are not multiples of
    the tile: the last tile row has a half-empty A box and scale tile, the last tile column clips its
    bulk stores.  Sampled rows x sampled columns (first, last, tile borders, random) against the oracle."""
    import ctypes

    from arcquant_b200 import _lib
    from tests.helpers import sf_take_rows

    ops, O = _ops(), _oracle()
    kq, ke = 4096, 128
    k_eff = kq + ke
    kind = ctypes.c_int(-1)
    assert _lib.load().arcq_matmul_plan(m, n, k_eff, ctypes.byref(kind), None, None) == 0
    assert kind.value == _lib.GEMM_KIND_PAIR
    dev = "cuda:0"
    out = synth.outlier_channels(kq, kq // 100, 1)
    x = synth.activations(m, kq, m + 2, out, device=dev)
    w = synth.weights(n, kq, n + 3, device=dev)
    idx = synth.reorder_index_from_stats(x[:1000].abs().amax(0)).to(dev)
    sx, sw = ops.absmax(x) / 2688.0, ops.absmax(w) / 2688.0
    a, sfa = ops.reorder_quantize_x((x / sx).to(torch.bfloat16), idx, ke)
    b, sfb = ops.reorder_quantize_w((w / sw).to(torch.bfloat16), idx, ke)
    alpha = float(sx * sw)
    guard = torch.full((m + 8, n), 7.0, dtype=torch.bfloat16, device=dev)      # rows beyond M must stay untouched
    c = guard[:m]
    rc = _lib.load().arcq_matmul_nvfp4(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, k_eff, alpha,
                                       c.data_ptr(), None)
    assert rc == 0
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    assert bool((guard[m:] == 7.0).all())

    def sample(size, seed):
        edges = [0, 1, 2, 3, size - 4, size - 3, size - 2, size - 1]
        for t in range(256, size, 256):
            edges += [t - 1, t]
        edges += [(size // 256) * 256 + d for d in (0, 1, 127, 128) if (size // 256) * 256 + d < size]
        g = torch.Generator().manual_seed(seed)
        pick = sorted(set(e for e in edges if 0 <= e < size))
        if len(pick) > 96:
            pick = sorted(set(pick[:8] + pick[-24:] + [pick[i] for i in torch.randint(0, len(pick), (64,), generator=g).tolist()]))
        pick = sorted(set(pick + torch.randint(0, size, (48,), generator=g).tolist()))
        return np.asarray(pick, dtype=np.int64)

    rows, cols = sample(m, 1), sample(n, 2)
    rt, ct = torch.from_numpy(rows).to(dev), torch.from_numpy(cols).to(dev)
    ref = O.gemm_fast(a[rt].cpu().numpy(), sf_take_rows(sfa, rows, k_eff), b[ct].cpu().numpy(),
                      sf_take_rows(sfb, cols, k_eff), alpha)
    got = c[rt][:, ct].float().cpu().numpy()
    _assert_close(got, ref)


@pytest.mark.parametrize("m,n,nd", [(1024, 2048, 4), (2048, 4096, 8), (768, 2056, 8), (1024, 1024, 1), (4096, 4096, 2)])
def test_scattered_output_rows_land_in_their_destinations(m, n, nd):
    """`matmul_scatter`: rows [d M/nd, (d+1) M/nd) of the result go to destination d (here: separate local
    buffers standing for the peers' receive slots).  The bytes are those of the plain GEMM on the CTA-pair
    kernel (same tiles, same accumulation order - only the address of each bulk store changes), which the
    other tests of this file hold to the oracle; rows_per_dest 96 makes destinations change inside a 256-row
    tile, and memory around every destination must stay untouched."""
    ops = _ops()
    kq, ke = 1024, 64
    dev = "cuda:0"
    out = synth.outlier_channels(kq, kq // 100, 1)
    x = synth.activations(m, kq, m + 2, out, device=dev)
    w = synth.weights(n, kq, n + 3, device=dev)
    idx = synth.reorder_index_from_stats(x[:512].abs().amax(0)).to(dev)
    sx, sw = ops.absmax(x) / 2688.0, ops.absmax(w) / 2688.0
    a, sfa = ops.reorder_quantize_x((x / sx).to(torch.bfloat16), idx, ke)
    b, sfb = ops.reorder_quantize_w((w / sw).to(torch.bfloat16), idx, ke)
    rows = m // nd
    guard = torch.full((nd, rows + 16, n), 7.0, dtype=torch.bfloat16, device=dev)
    dests = [guard[d, 8:].data_ptr() for d in range(nd)]
    ops.matmul_scatter(a, b, sfa, sfb, sx, sw, dests)
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    # the reference bytes: the same kernel with one destination (the plain launcher may pick the single-CTA
    # kernel for the small shapes, whose accumulation order differs in the last bit)
    whole = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    ops.matmul_scatter(a, b, sfa, sfb, sx, sw, [whole.data_ptr()])
    plain = ops.matmul_dev_alpha(a, b, sfa, sfb, sx, sw)
    torch.cuda.synchronize()
    assert torch.equal(guard[:, 8:8 + rows].reshape(m, n), whole)
    assert bool((guard[:, :8] == 7.0).all()) and bool((guard[:, 8 + rows:] == 7.0).all())
    err = float((whole.float() - plain.float()).norm() / plain.float().norm())
    assert err < TOL, err
    assert float((whole == plain).float().mean()) > 0.99


def test_scattered_output_against_the_oracle():
    """One scattered launch held to the oracle directly (sampled rows of every destination)."""
    from tests.helpers import sf_take_rows

    ops, O = _ops(), _oracle()
    m, n, kq, ke, nd = 2048, 2304, 2048, 128, 8
    k_eff = kq + ke
    dev = "cuda:0"
    out = synth.outlier_channels(kq, kq // 100, 5)
    x = synth.activations(m, kq, 11, out, device=dev)
    w = synth.weights(n, kq, 12, device=dev)
    idx = synth.reorder_index_from_stats(x[:512].abs().amax(0)).to(dev)
    sx, sw = ops.absmax(x) / 2688.0, ops.absmax(w) / 2688.0
    a, sfa = ops.reorder_quantize_x((x / sx).to(torch.bfloat16), idx, ke)
    b, sfb = ops.reorder_quantize_w((w / sw).to(torch.bfloat16), idx, ke)
    slots = torch.zeros((nd, m // nd, n), dtype=torch.bfloat16, device=dev)
    ops.matmul_scatter(a, b, sfa, sfb, sx, sw, [slots[d].data_ptr() for d in range(nd)])
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    g = torch.Generator().manual_seed(3)
    rows = np.asarray(sorted(set([0, 255, 256, 257, m - 1] + torch.randint(0, m, (40,), generator=g).tolist())), dtype=np.int64)
    rt = torch.from_numpy(rows).to(dev)
    ref = O.gemm_fast(a[rt].cpu().numpy(), sf_take_rows(sfa, rows, k_eff), b.cpu().numpy(), sfb.cpu().numpy(),
                      float(sx * sw))
    got = slots.reshape(m, n)[rt].float().cpu().numpy()
    _assert_close(got, ref)


@pytest.mark.parametrize("m,n,kq", [(1024, 1024, 1024), (4100, 4104, 1024), (2048, 4096, 4096), (300, 9992, 512)])
def test_residual_added_in_the_epilogue_equals_gemm_then_addition(m, n, kq):
    """`matmul_residual`: bf16(R + bf16(GEMM)) from the epilogue - bit for bit the GEMM of the same kernel followed
    by torch's bf16 addition; ragged shapes clip the residual boxes like the output boxes; rows beyond M stay
    untouched."""
    ops = _ops()
    ke = 64
    dev = "cuda:0"
    out = synth.outlier_channels(kq, max(1, kq // 100), 1)
    x = synth.activations(m, kq, m + 2, out, device=dev)
    w = synth.weights(n, kq, n + 3, device=dev)
    idx = synth.reorder_index_from_stats(x[:256].abs().amax(0)).to(dev)
    sx, sw = ops.absmax(x) / 2688.0, ops.absmax(w) / 2688.0
    a, sfa = ops.reorder_quantize_x((x / sx).to(torch.bfloat16), idx, ke)
    b, sfb = ops.reorder_quantize_w((w / sw).to(torch.bfloat16), idx, ke)
    res = (0.05 * torch.randn((m, n), generator=torch.Generator().manual_seed(9))).to(torch.bfloat16).to(dev)
    whole = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    ops.matmul_scatter(a, b, sfa, sfb, sx, sw, [whole.data_ptr()]) if m % 32 == 0 else None
    if m % 32:
        # (the scattered launcher wants whole 32-row boxes; the plain launcher picks the pair kernel for these shapes)
        whole = ops.matmul_dev_alpha(a, b, sfa, sfb, sx, sw)
    guard = torch.full((m + 8, n), 7.0, dtype=torch.bfloat16, device=dev)
    got = ops.matmul_residual(a, b, sfa, sfb, sx, sw, res, out=guard[:m])
    torch.cuda.synchronize()
    assert ops.gemm_poll_error() == 0
    assert torch.equal(got, res + whole)
    assert bool((guard[m:] == 7.0).all())

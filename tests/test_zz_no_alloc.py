"""The allocation-free GEMM entry point, `arcq_matmul_nvfp4_static`.

Some users of this library may not allocate device memory at the point where they need the GEMM: a
serving plugin whose enqueue hook must not touch the allocator, a process that has already given
all device memory to another framework's pool, a latency-critical decode loop.  For them the split-K
GEMM keeps its fp32 partial sums in a 2 MiB block that is part of the library image.  This test
drives that entry point through the C ABI and holds it to the output of the existing
caller-scratch entry point (`arcq_matmul_nvfp4_ws`): same kernels, same fixed summation order, so the
bf16 results must be identical - on two calls in a row, because the block is shared and keeps the
previous call's contents.  (The file name sorts last so that a run that stops at the first failure
has already run every other test.)"""
import numpy as np
import pytest
import torch

from arcquant_b200 import synth

pytestmark = pytest.mark.gpu


def _packed(m, n, kq, ke, seed):
    """Packed operands made by the library's own quantizers from seeded inputs."""
    from arcquant_b200 import ops

    x = synth.activations(m, kq, seed, synth.outlier_channels(kq, kq // 100, seed)).cuda()
    w = synth.weights(n, kq, seed + 1).cuda()
    idx = torch.randperm(kq, generator=torch.Generator().manual_seed(seed)).to(torch.int16).cuda()
    sx, sw = ops.absmax(x) / 2688.0, ops.absmax(w) / 2688.0
    a, sfa = ops.reorder_quantize_x((x / sx).to(torch.bfloat16), idx, ke)
    b, sfb = ops.reorder_quantize_w((w / sw).to(torch.bfloat16), idx, ke)
    return a, sfa, b, sfb, float(sx * sw)


@pytest.mark.parametrize("m,n,kq", [(16, 4096, 4096), (16, 4096, 14336), (1, 1024, 4096)])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(m, n, kq):
    from arcquant_b200 import _lib, ops

    L = _lib.load()
    ke = 128
    k_eff = kq + ke
    need = int(L.arcq_matmul_workspace_bytes(m, n, k_eff))
    assert 0 < need <= _lib.STATIC_SCRATCH_BYTES              # split, and within the built-in block
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    for call, seed in enumerate((11, 12)):                     # second call: new data over the old scratch
        a, sfa, b, sfb, alpha = _packed(m, n, kq, ke, seed)
        want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = L.arcq_matmul_nvfp4_ws(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, k_eff, alpha,
                                    None, None, want.data_ptr(), ws.data_ptr(), need, None)
        assert rc == 0
        rc = L.arcq_matmul_nvfp4_static(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, k_eff,
                                        alpha, None, None, got.data_ptr(), None)
        assert rc == 0, L.arcq_status_string(rc)
        torch.cuda.synchronize()
        assert ops.gemm_poll_error() == 0
        # identical kernels and summation order: the tolerance the GEMM tests use (1e-3 relative
        # Frobenius in the output type) is met with equality
        w_, g_ = want.float().cpu().numpy(), got.float().cpu().numpy()
        assert np.isfinite(g_).all()
        assert np.linalg.norm(g_ - w_) <= 1e-3 * np.linalg.norm(w_)
        assert np.array_equal(g_, w_), f"call {call}"
        # and directly against the CPU oracle's dequantised fp32 matmul, rounded to the output type
        from oracle import oracle as O
        ref = O.gemm_fast(a.cpu().numpy(), sfa.cpu().numpy(), b.cpu().numpy(), sfb.cpu().numpy(), alpha)
        refb = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
        assert np.linalg.norm(g_ - refb) <= 1e-3 * np.linalg.norm(refb), f"call {call} against the oracle"
    # the entry point allocates nothing: free device memory is the same before and after warmed-up calls
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert L.arcq_matmul_nvfp4_static(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, k_eff,
                                          alpha, None, None, got.data_ptr(), None) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, (free0, free1)


def test_shapes_beyond_the_block_are_refused_and_unsplit_shapes_need_none():
    from arcquant_b200 import _lib

    L = _lib.load()
    m, n, kq, ke = 128, 4096, 14336, 128
    assert int(L.arcq_matmul_workspace_bytes(m, n, kq + ke)) > _lib.STATIC_SCRATCH_BYTES
    a, sfa, b, sfb, alpha = _packed(m, n, kq, ke, 3)
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    rc = L.arcq_matmul_nvfp4_static(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kq + ke, alpha,
                                    None, None, out.data_ptr(), None)
    assert rc == _lib.ERR_SCRATCH_LIMIT
    assert b"scratch" in L.arcq_status_string(rc)
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0                       # refused before anything ran
    # a shape that is not split runs through the same entry point without scratch
    m, n, kq = 512, 4096, 4096
    assert int(L.arcq_matmul_workspace_bytes(m, n, kq + ke)) == 0
    a, sfa, b, sfb, alpha = _packed(m, n, kq, ke, 4)
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    got = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    assert L.arcq_matmul_nvfp4(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kq + ke, alpha,
                               want.data_ptr(), None) == 0
    assert L.arcq_matmul_nvfp4_static(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kq + ke, alpha,
                                      None, None, got.data_ptr(), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(want, got)

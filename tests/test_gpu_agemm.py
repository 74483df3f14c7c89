"""The reference's call pattern through the `agemm` module (model/qLinearLayer.py:25-28,64-81 and
model/qLlamaLayer.py:73-77 of ARCQuant): config 1 of the benchmark contract, end to end."""
import os
import sys

import numpy as np
import pytest
import torch

from arcquant_b200 import synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _agemm():
    sys.path.insert(0, os.path.join(ROOT, "arcquant_b200"))
    import agemm
    return agemm


def test_config1_single_linear_matches_oracle_and_fp32():
    from oracle import oracle as O

    agemm = _agemm()
    x, w, idx, ke = synth.config1()
    dev = "cuda:0"
    xd, wd, idxd = x.to(dev), w.to(dev), idx.to(dev)
    # the callers' pre-scaling (bf16 tensor / 0-dim fp32 CUDA tensor)
    sx = torch.max(xd.abs()).float() / (448.0 * 6.0)
    sw = torch.max(wd.abs()).float() / (448.0 * 6.0)
    xs, ws = xd / sx, wd / sw
    assert xs.dtype == torch.bfloat16
    A, SFA = agemm.reorder_quantize_x(xs, idxd, ke)
    B, SFB = agemm.reorder_quantize_w(ws, idxd, ke)
    Y = agemm.matmul(A, B, SFA, SFB, float(sx * sw))
    torch.cuda.synchronize()
    assert Y.shape == (512, 4096) and Y.dtype == torch.bfloat16
    assert A.shape == (512, 2112) and SFA.numel() == 168960 and SFA.dtype == torch.uint8
    # bit-exact codes/scales against the oracle fed the very same pre-scaled bf16 inputs
    qa, sfa = O.quantize_x(xs.cpu(), idx.numpy(), ke)
    qb, sfb = O.quantize_w(ws.cpu(), idx.numpy(), ke)
    assert np.array_equal(A.cpu().numpy(), qa) and np.array_equal(B.cpu().numpy(), qb)
    va, vb = O.sf_valid_offsets(512, 4224), O.sf_valid_offsets(4096, 4224)
    assert np.array_equal(SFA.cpu().numpy()[va], sfa[va]) and np.array_equal(SFB.cpu().numpy()[vb], sfb[vb])
    ref = O.gemm_fast(qa, sfa, qb, sfb, float(sx * sw))
    y = Y.float().cpu().numpy()
    # output type is bf16: compare with the oracle rounded to bf16 (see tests/test_gpu_gemm.py)
    refb = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
    assert np.linalg.norm(y - refb) / np.linalg.norm(refb) <= 1e-3
    assert np.linalg.norm(y - ref) / np.linalg.norm(ref) <= 2.2e-3
    # and the quantization error itself is where ARC puts it (about 0.1 on this input)
    full = (x.float() @ w.float().T).numpy()
    err = np.linalg.norm(y - full) / np.linalg.norm(full)
    assert 0.02 < err < 0.13


def test_fused_rmsnorm_operator():
    from oracle import oracle as O

    agemm = _agemm()
    kq = 4096
    out = synth.outlier_channels(kq, 41, 1)
    x = synth.activations(48, kq, 2, out)
    gamma = synth.rms_gain(kq, 3)
    idx = synth.reorder_index_from_stats(x.abs().amax(0))
    A, SFA = agemm.rmsnorm_quantize_x(x.cuda(), gamma.cuda(), 1e-5, idx.cuda(), 128)
    qa, sfa = O.quantize_x(x, idx.numpy(), 128, gamma=gamma, eps=1e-5)
    assert np.array_equal(A.cpu().numpy(), qa)
    v = O.sf_valid_offsets(48, kq + 128)
    assert np.array_equal(SFA.cpu().numpy()[v], sfa[v])


def test_error_behaviour_mirrors_the_reference():
    agemm = _agemm()
    idx = torch.arange(4096, dtype=torch.int16, device="cuda")
    with pytest.raises(RuntimeError):          # wrong dtype: data_ptr<BFloat16>() throws
        agemm.reorder_quantize_x(torch.zeros(4, 4096, dtype=torch.float16, device="cuda"), idx, 128)
    with pytest.raises(RuntimeError):          # a width the kernels do not serve
        agemm.reorder_quantize_x(torch.zeros(4, 40, dtype=torch.bfloat16, device="cuda"),
                                 torch.arange(40, dtype=torch.int16, device="cuda"), 0)
    with pytest.raises(RuntimeError):
        agemm.rmsnorm_quantize_x(torch.zeros(4, 14336, dtype=torch.bfloat16, device="cuda"),
                                 torch.ones(14336, dtype=torch.bfloat16, device="cuda"), 1e-5,
                                 torch.arange(14336, dtype=torch.int16, device="cuda"), 128)
    # inputs are borrowed, never mutated
    x = torch.randn(8, 4096, device="cuda").to(torch.bfloat16)
    keep = x.clone()
    agemm.reorder_quantize_x(x, idx, 128)
    assert torch.equal(x, keep)


def test_host_pipeline_matches_single_call():
    """Chunked upload / kernel / download over three streams gives the bytes of one call on the batch."""
    from arcquant_b200 import ops
    from arcquant_b200.host_pipeline import HostQuantizePipeline

    tokens, kq, ke = 1000, 4096, 128          # not a multiple of the chunk: ragged last chunk, odd tile
    out = synth.outlier_channels(kq, 40, 2)
    x = synth.activations(tokens, kq, 21, out)
    gamma = synth.rms_gain(kq, 5)
    idx = synth.reorder_index_from_stats(synth.activations(64, kq, 3, out).abs().amax(0))
    hx = x.pin_memory()
    pipe = HostQuantizePipeline(tokens, kq, ke, "cuda:0", chunk_rows=256)
    hq = torch.empty((tokens, (kq + ke) // 2), dtype=torch.uint8).pin_memory()
    hsf = torch.zeros((pipe.sf_bytes(),), dtype=torch.uint8).pin_memory()
    nvalid = ((tokens + 127) // 128) * (((kq + ke) // 16 + 3) // 4) * 512
    for g in (None, gamma.cuda()):
        pipe.run(hx, idx.cuda(), hq, hsf, gamma=g, eps=1e-5)
        if g is None:
            q, sf = ops.reorder_quantize_x(x.cuda(), idx.cuda(), ke)
        else:
            q, sf = ops.rmsnorm_quantize_x(x.cuda(), g, 1e-5, idx.cuda(), ke)
        assert torch.equal(hq, q.cpu())
        # rows beyond `tokens` in the last tile are never written by either path: compare valid bytes
        from tests.helpers import valid_sf
        assert (valid_sf(hsf[:nvalid], tokens, kq + ke) == valid_sf(sf[:nvalid], tokens, kq + ke)).all()

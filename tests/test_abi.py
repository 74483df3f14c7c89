"""The drop-in boundary without a GPU: the C ABI exports what include/arcq.h declares, refuses to
compute without a CUDA device, and the `agemm` module offers the reference's operator names."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "arcq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(arcq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from arcquant_b200 import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), n
    assert sorted(_lib.SIGNATURES) == names          # the ctypes table mirrors the header


def test_host_side_helpers():
    from arcquant_b200 import _lib

    L = _lib.load()
    assert L.arcq_sf_bytes(512, 4224) == 168960
    assert L.arcq_sf_bytes(128, 4224) == 2 * 128 * 264
    assert L.arcq_sf_bytes(1, 4160) >= 65 * 512
    assert [L.arcq_reference_mode(k) for k in (4096, 3584, 14336, 28672, 18944, 27648)] == [16, 32, 16, 32, 32, 32]
    assert L.arcq_status_string(0) == b"ok"


def test_argument_validation_precedes_any_cuda_call():
    from arcquant_b200 import _lib

    L = _lib.load()
    p = 1 << 12
    assert L.arcq_reorder_quantize_x(p, None, 4, 40, 0, 16, p, p, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_reorder_quantize_x(p, None, 4, 64, 8, 16, p, p, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_reorder_quantize_x(p, None, 4, 64, 16, 32, p, p, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_reorder_quantize_x(None, None, 4, 64, 0, 16, p, p, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_reorder_quantize_x(p + 2, None, 4, 64, 0, 16, p, p, None) == _lib.ERR_ALIGNMENT
    assert L.arcq_rmsnorm_quantize_x(p, p, 1e-5, None, 4, 14336, 0, p, p, None) == _lib.ERR_UNSUPPORTED_K
    assert L.arcq_matmul_nvfp4(p, p, p, p, 4, 64, 96, 1.0, p, None) == _lib.ERR_BAD_SHAPE      # K % 64
    assert L.arcq_matmul_nvfp4(p, p, p, p, 4, 60, 128, 1.0, p, None) == _lib.ERR_BAD_SHAPE     # N % 8
    assert L.arcq_matmul_nvfp4(p, p, p, p, 0, 64, 128, 1.0, p, None) == _lib.OK                # empty M
    assert L.arcq_reorder_quantize_x(p, None, 0, 64, 0, 16, p, p, None) == _lib.OK             # empty input
    assert L.arcq_reorder_quantize_x_scaled(p, None, None, 4, 64, 0, 16, p, p, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_reorder_quantize_x_scaled(p, p, None, 4, 72, 0, 16, p, p, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_rope_bf16(p, p, p, 4, 512, 2, 120, 8, None) == _lib.ERR_BAD_SHAPE            # head_dim % 16
    assert L.arcq_rope_bf16(p, p, p, 4, 512, 5, 128, 8, None) == _lib.ERR_BAD_SHAPE            # heads beyond the row
    assert L.arcq_rope_bf16(p, None, p, 4, 512, 2, 128, 8, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_rope_bf16(p, p, p, 0, 512, 2, 128, 8, None) == _lib.OK                       # no tokens
    assert L.arcq_silu_mul_bf16(p, p, 4, 100, None, None) == _lib.ERR_BAD_SHAPE                # F % 8
    assert L.arcq_silu_mul_bf16(None, p, 4, 128, None, None) == _lib.ERR_NULL_POINTER


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_cpu_fallback():
    from arcquant_b200 import _lib, ops

    L = _lib.load()
    p = 1 << 12
    assert L.arcq_reorder_quantize_x(p, None, 4, 64, 0, 16, p, p, None) == _lib.ERR_CUDA
    with pytest.raises(RuntimeError):
        ops.reorder_quantize_x(torch.zeros(4, 64, dtype=torch.bfloat16), None, 0)


def test_agemm_module_surface():
    import importlib
    import sys

    sys.path.insert(0, os.path.join(ROOT, "arcquant_b200"))
    agemm = importlib.import_module("agemm")
    for name in ("matmul", "reorder_quantize_x", "reorder_quantize_w", "rmsnorm_quantize_x"):
        assert callable(getattr(agemm, name))
    with pytest.raises(RuntimeError):
        agemm.reorder_quantize_x(torch.zeros(4, 64, dtype=torch.bfloat16), torch.arange(64, dtype=torch.int16), 0)


def test_agemm_rejects_host_tensors_and_short_buffers_before_any_launch():
    """Every tensor a kernel would dereference is checked by the extension itself: a CPU scalar, a
    short index or a short scale buffer raises here instead of reaching a kernel as a bad pointer."""
    import importlib
    import sys

    sys.path.insert(0, os.path.join(ROOT, "arcquant_b200"))
    agemm = importlib.import_module("agemm")
    x = torch.zeros(4, 64, dtype=torch.bfloat16)
    idx = torch.arange(64, dtype=torch.int16)
    u8 = torch.zeros(4, 32, dtype=torch.uint8)
    sf = torch.zeros(512, dtype=torch.uint8)
    s = torch.tensor(1.0)
    for call in (lambda: agemm.reorder_quantize_x_scaled(x, s, idx, 0),
                 lambda: agemm.matmul_dev_alpha(u8, u8, sf, sf, s, None),
                 lambda: agemm.matmul(u8, u8, sf, sf, 1.0),
                 lambda: agemm.rmsnorm_quantize_x(x, x[0], 1e-5, idx, 0),
                 lambda: agemm.absmax(x)):
        with pytest.raises(RuntimeError, match="CUDA tensor"):
            call()


@pytest.mark.gpu
def test_agemm_argument_checks_on_device_tensors():
    import importlib
    import sys

    sys.path.insert(0, os.path.join(ROOT, "arcquant_b200"))
    agemm = importlib.import_module("agemm")
    dev = "cuda"
    x = torch.zeros(4, 64, dtype=torch.bfloat16, device=dev)
    idx = torch.arange(64, dtype=torch.int16, device=dev)
    s = torch.tensor(1.0, device=dev)
    with pytest.raises(RuntimeError, match="CUDA tensor"):            # a host amax passed as the scale
        agemm.reorder_quantize_x_scaled(x, torch.tensor(1.0), idx, 0)
    with pytest.raises(RuntimeError, match="KQ entries"):             # a short index
        agemm.reorder_quantize_x_scaled(x, s, idx[:32].contiguous(), 0)
    with pytest.raises(RuntimeError, match="KQ entries"):
        agemm.reorder_quantize_x(x, idx[:32].contiguous(), 0)
    with pytest.raises(RuntimeError, match="expected"):               # index of the wrong type
        agemm.reorder_quantize_x(x, idx.int(), 0)
    a = torch.zeros(4, 32, dtype=torch.uint8, device=dev)
    b = torch.zeros(8, 32, dtype=torch.uint8, device=dev)
    sf = torch.zeros(512, dtype=torch.uint8, device=dev)
    with pytest.raises(RuntimeError, match="smaller than the scale layout"):
        agemm.matmul(a, b, sf[:256].contiguous(), sf, 1.0)
    with pytest.raises(RuntimeError, match="disagree on K"):
        agemm.matmul(a, torch.zeros(8, 64, dtype=torch.uint8, device=dev), sf, sf, 1.0)
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        agemm.matmul_dev_alpha(a, b, sf, sf, torch.tensor(1.0), None)
    with pytest.raises(RuntimeError, match="one fp32 value"):
        agemm.matmul_dev_alpha(a, b, sf, sf, torch.ones(2, device=dev), None)
    torch.cuda.synchronize()                                          # nothing was launched, nothing faulted
    assert agemm.matmul(a, b, sf, sf, 1.0).shape == (4, 8)


def test_peer_and_scatter_entry_points_validate_before_any_cuda_call():
    """The entry points of the tensor- / expert-parallel forms refuse bad shapes and null pointers on the host."""
    import ctypes as C

    from arcquant_b200 import _lib, ops

    L = _lib.load()
    p = 1 << 12
    two = (C.c_void_p * 2)(p, p)
    hole = (C.c_void_p * 2)(p, None)
    # GEMM with scattered output: 1..8 destinations, rows split evenly in multiples of 32, no null destination
    assert L.arcq_matmul_nvfp4_scatter(p, p, p, p, 128, 64, 64, p, None, None, 2, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_matmul_nvfp4_scatter(p, p, p, p, 128, 64, 64, p, None, two, 9, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_matmul_nvfp4_scatter(p, p, p, p, 96, 64, 64, p, None, two, 2, None) == _lib.ERR_BAD_SHAPE      # 48 rows each
    assert L.arcq_matmul_nvfp4_scatter(p, p, p, p, 128, 64, 64, p, None, hole, 2, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_matmul_nvfp4_scatter(p, p, p, p, 128, 64, 64, None, None, two, 2, None) == _lib.ERR_NULL_POINTER   # alpha_a
    assert L.arcq_matmul_nvfp4_residual(p, p, p, p, 128, 64, 64, p, None, None, p, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_matmul_nvfp4_residual(p, p, p, p, 128, 64, 64, p, None, p + 2, p, None) == _lib.ERR_ALIGNMENT
    # sum of partial results
    assert L.arcq_sum_partials_bf16(two, 0, 1024, None, p, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_sum_partials_bf16(two, 2, 1020, None, p, None) == _lib.ERR_BAD_SHAPE                 # elems % 8
    assert L.arcq_sum_partials_bf16(hole, 2, 1024, None, p, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_sum_partials_bf16(two, 2, 0, None, p, None) == _lib.OK
    # quantizer with several destinations
    assert L.arcq_rmsnorm_quantize_x_multi(p, p, 1e-5, p, 128, 4096, 128, two, two, 0, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_rmsnorm_quantize_x_multi(p, p, 1e-5, p, 128, 4096, 128, two, hole, 2, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_rmsnorm_quantize_x_multi(p, p, 1e-5, p, 128, 1000, 0, two, two, 2, None) != _lib.OK   # width
    # barrier and expert-parallel dispatch
    assert L.arcq_peer_barrier(two, 2, 2, p, None) == _lib.ERR_BAD_SHAPE                               # rank outside the group
    assert L.arcq_peer_barrier(two, 0, 9, p, None) == _lib.ERR_BAD_SHAPE
    assert L.arcq_peer_barrier(hole, 0, 2, p, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_peer_barrier(two, 0, 2, None, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_ep_send_layout(p, 16, 2, 9, 128, 0, p, two, p, None) == _lib.ERR_BAD_SHAPE           # more than 8 ranks
    assert L.arcq_ep_send_layout(p, 16, 2, 2, 128, 2, p, two, p, None) == _lib.ERR_BAD_SHAPE           # rank outside
    assert L.arcq_ep_send_layout(p, 16, 2, 2, 128, 0, p, hole, p, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_ep_rows(p, None, 2, 16, None, 32, 100, 128, 2, 0, two, None) == _lib.ERR_BAD_SHAPE   # row bytes % 16
    assert L.arcq_ep_rows(p, None, 0, 16, None, 32, 128, 128, 2, 0, two, None) == _lib.ERR_BAD_SHAPE   # div
    assert L.arcq_ep_rows(p, None, 2, 16, None, 0, 128, 128, 2, 0, two, None) == _lib.OK               # nothing to move
    assert L.arcq_peer_export(None, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_peer_open(None, None) == _lib.ERR_NULL_POINTER
    assert L.arcq_peer_set_wait_limit_ms(L.arcq_peer_set_wait_limit_ms(1234)) == 1234
    # the torch-facing wrappers refuse host tensors
    u8 = torch.zeros(64, 32, dtype=torch.uint8)
    sf = torch.zeros(512, dtype=torch.uint8)
    s = torch.tensor(1.0)
    for call in (lambda: ops.matmul_scatter(u8, u8, sf, sf, s, None, [p]),
                 lambda: ops.matmul_residual(u8, u8, sf, sf, s, None, torch.zeros(64, 64, dtype=torch.bfloat16)),
                 lambda: ops.sum_partials([p], 64, torch.zeros(64, dtype=torch.bfloat16)),
                 lambda: ops.rmsnorm_quantize_x_multi(torch.zeros(128, 4096, dtype=torch.bfloat16),
                                                      torch.zeros(4096, dtype=torch.bfloat16), 1e-5,
                                                      torch.zeros(4096, dtype=torch.int16), 128, [p], [p])):
        with pytest.raises(RuntimeError, match="CUDA tensor"):
            call()

"""ctypes front end of the CPU oracle (``arcq_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Only the test-suite, the smoke check and the CPU
baseline leg of the benchmark may import this module; the shipped package
never does.  Every function here forwards to the C restatement of the
reference kernels' arithmetic and works on numpy arrays (bf16 tensors travel
as ``uint16`` bit patterns).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libarcq_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C oracle next to its source (gcc, a second or two)."""
    src = os.path.join(_HERE, "arcq_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "-B"])
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        p = C.c_void_p
        L.arcq_e2m1_decode.restype = C.c_float
        L.arcq_e2m1_decode.argtypes = [C.c_uint8]
        L.arcq_e2m1_encode.restype = C.c_uint8
        L.arcq_e2m1_encode.argtypes = [C.c_float]
        L.arcq_ue4m3_decode.restype = C.c_float
        L.arcq_ue4m3_decode.argtypes = [C.c_uint8]
        L.arcq_ue4m3_encode.restype = C.c_uint8
        L.arcq_ue4m3_encode.argtypes = [C.c_float]
        L.arcq_rsqrt_rn.restype = C.c_float
        L.arcq_rsqrt_rn.argtypes = [C.c_float]
        L.arcq_f32_to_bf16.restype = C.c_uint16
        L.arcq_f32_to_bf16.argtypes = [C.c_float]
        L.arcq_sf_offset.restype = C.c_int64
        L.arcq_sf_offset.argtypes = [C.c_int64] * 3
        L.arcq_sf_bytes_reference.restype = C.c_int64
        L.arcq_sf_bytes_reference.argtypes = [C.c_int64] * 2
        L.arcq_sf_bytes_span.restype = C.c_int64
        L.arcq_sf_bytes_span.argtypes = [C.c_int64] * 2
        L.arcq_oracle_quantize_x.restype = C.c_int
        L.arcq_oracle_quantize_x.argtypes = [p, C.c_int64, C.c_int, p, C.c_int, C.c_int, p, C.c_float, p, p]
        L.arcq_oracle_quantize_w.restype = C.c_int
        L.arcq_oracle_quantize_w.argtypes = [p, C.c_int64, C.c_int, p, C.c_int, C.c_int, p, p]
        L.arcq_oracle_fake_values.restype = C.c_int
        L.arcq_oracle_fake_values.argtypes = [p, C.c_int64, C.c_int, p, C.c_int, p]
        L.arcq_oracle_dequant.restype = None
        L.arcq_oracle_dequant.argtypes = [p, p, C.c_int64, C.c_int, p]
        L.arcq_oracle_gemm.restype = None
        L.arcq_oracle_gemm.argtypes = [p, p, p, p, C.c_int64, C.c_int64, C.c_int, C.c_float, p]
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def to_bits(t) -> np.ndarray:
    """torch bf16 tensor (CPU) or uint16 ndarray -> contiguous uint16 ndarray."""
    if isinstance(t, np.ndarray):
        assert t.dtype == np.uint16
        return np.ascontiguousarray(t)
    import torch

    assert t.dtype == torch.bfloat16
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def sf_bytes_reference(rows: int, k_eff: int) -> int:
    return int(lib().arcq_sf_bytes_reference(rows, k_eff))


def sf_bytes_span(rows: int, k_eff: int) -> int:
    return int(lib().arcq_sf_bytes_span(rows, k_eff))


def sf_alloc_bytes(rows: int, k_eff: int) -> int:
    return max(sf_bytes_reference(rows, k_eff), sf_bytes_span(rows, k_eff))


def sf_offset(r: int, c: int, ncols: int) -> int:
    return int(lib().arcq_sf_offset(r, c, ncols))


def sf_valid_offsets(rows: int, k_eff: int) -> np.ndarray:
    """Sorted byte offsets of every scale the quantizers write for ``rows`` rows."""
    ncols = k_eff // 16
    natoms = (ncols + 3) // 4
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(ncols, dtype=np.int64)[None, :]
    off = ((r // 128) * natoms + c // 4) * 512 + (r % 32) * 16 + ((r // 32) % 4) * 4 + (c % 4)
    return np.sort(off.reshape(-1))


def reference_mode(kq: int) -> int:
    """Which reference kernel family serves this KQ (kernels/src/bindings.cpp:141-160)."""
    return 32 if kq in (3584, 18944, 27648, 28672) else 16


def quantize_x(x, idx, ke: int, mode: int = 16, gamma=None, eps: float = 0.0, fill: int = 0):
    """Oracle for reorder_quantize_x / rmsnorm_quantize_x.

    Returns (QX uint8 [M, K_eff/2], SFX uint8 [alloc]) with never-written scale
    bytes set to ``fill``."""
    xb = to_bits(x)
    m, kq = xb.shape
    idxa = None if idx is None else np.ascontiguousarray(np.asarray(idx, dtype=np.int16))
    g = None if gamma is None else to_bits(gamma)
    k_eff = kq + ke
    q = np.zeros((m, k_eff // 2), dtype=np.uint8)
    sf = np.full(sf_alloc_bytes(m, k_eff), fill, dtype=np.uint8)
    rc = lib().arcq_oracle_quantize_x(_ptr(xb), m, kq, _ptr(idxa), ke, mode, _ptr(g), float(eps), _ptr(q), _ptr(sf))
    if rc != 0:
        raise ValueError(f"oracle rejected shape KQ={kq} KE={ke} mode={mode}")
    return q, sf


def quantize_w(w, idx, ke: int, mode: int = 16, fill: int = 0):
    wb = to_bits(w)
    n, kq = wb.shape
    idxa = None if idx is None else np.ascontiguousarray(np.asarray(idx, dtype=np.int16))
    k_eff = kq + ke
    q = np.zeros((n, k_eff // 2), dtype=np.uint8)
    sf = np.full(sf_alloc_bytes(n, k_eff), fill, dtype=np.uint8)
    rc = lib().arcq_oracle_quantize_w(_ptr(wb), n, kq, _ptr(idxa), ke, mode, _ptr(q), _ptr(sf))
    if rc != 0:
        raise ValueError(f"oracle rejected shape KQ={kq} KE={ke} mode={mode}")
    return q, sf


def fake_values(x, idx, ke: int) -> np.ndarray:
    """The oracle's structure run with the fake path's arithmetic knobs: fp32
    values [M, KQ+KE], main block then the appended residual block."""
    xb = to_bits(x)
    m, kq = xb.shape
    idxa = None if idx is None else np.ascontiguousarray(np.asarray(idx, dtype=np.int16))
    out = np.empty((m, kq + ke), dtype=np.float32)
    rc = lib().arcq_oracle_fake_values(_ptr(xb), m, kq, _ptr(idxa), ke, _ptr(out))
    if rc != 0:
        raise ValueError("oracle rejected shape")
    return out


def dequant(q: np.ndarray, sf: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    sf = np.ascontiguousarray(sf, dtype=np.uint8)
    rows, kb = q.shape
    out = np.empty((rows, kb * 2), dtype=np.float32)
    lib().arcq_oracle_dequant(_ptr(q), _ptr(sf), rows, kb * 2, _ptr(out))
    return out


def gemm(a, sfa, b, sfb, alpha: float) -> np.ndarray:
    """fp32 reference of the block-scaled GEMM (double accumulation, small shapes)."""
    a = np.ascontiguousarray(a, dtype=np.uint8)
    b = np.ascontiguousarray(b, dtype=np.uint8)
    sfa = np.ascontiguousarray(sfa, dtype=np.uint8)
    sfb = np.ascontiguousarray(sfb, dtype=np.uint8)
    m, kb = a.shape
    n = b.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    lib().arcq_oracle_gemm(_ptr(a), _ptr(sfa), _ptr(b), _ptr(sfb), m, n, kb * 2, float(alpha), _ptr(out))
    return out


def gemm_fast(a, sfa, b, sfb, alpha: float) -> np.ndarray:
    """Same reference for larger shapes: dequantise in C, multiply with BLAS in
    fp64 so that the check adds no accumulation-order noise of its own."""
    da = dequant(a, sfa).astype(np.float64)
    db = dequant(b, sfb).astype(np.float64)
    return (float(alpha) * (da @ db.T)).astype(np.float32)

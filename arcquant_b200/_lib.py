"""ctypes binding of libarcq.so (the C ABI declared in include/arcq.h).

There is no fallback: if the shared library has not been built, importing this
module raises, and so does every operator of the package.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libarcq.so")

OK = 0
ERR_BAD_SHAPE = 1
ERR_UNSUPPORTED_K = 2
ERR_NULL_POINTER = 3
ERR_CUDA = 4
ERR_ALIGNMENT = 5
ERR_TIMEOUT = 6
ERR_SCRATCH_LIMIT = 7
STATIC_SCRATCH_BYTES = 2 << 20

GEMM_KIND_SINGLE, GEMM_KIND_SPLIT_K, GEMM_KIND_PAIR = 0, 1, 2

MODE_16 = 16
MODE_32 = 32

# name -> (restype, argtypes); mirrors include/arcq.h one to one
_vp, _i64, _i32, _f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
SIGNATURES = {
    "arcq_status_string": (C.c_char_p, [_i32]),
    "arcq_last_cuda_error": (_i32, []),
    "arcq_version": (_i32, []),
    "arcq_set_sm_limit": (_i32, [_i32]),
    "arcq_sf_bytes": (C.c_size_t, [_i64, _i64]),
    "arcq_reference_mode": (_i32, [_i32]),
    "arcq_reorder_quantize_x": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "arcq_reorder_quantize_x_scaled": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "arcq_rmsnorm_quantize_x": (_i32, [_vp, _vp, _f32, _vp, _i64, _i32, _i32, _vp, _vp, _vp]),
    "arcq_reorder_quantize_w": (_i32, [_vp, _vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "arcq_matmul_nvfp4": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _vp, _vp]),
    "arcq_matmul_nvfp4_dev_alpha": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp]),
    "arcq_matmul_workspace_bytes": (C.c_size_t, [_i64, _i64, _i64]),
    "arcq_matmul_plan": (_i32, [_i64, _i64, _i64, _vp, _vp, _vp]),
    "arcq_matmul_nvfp4_ws": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "arcq_matmul_nvfp4_static": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _vp, _vp, _vp, _vp]),
    "arcq_gemm_poll_error": (_i32, []),
    "arcq_absmax_bf16": (_i32, [_vp, _i64, _vp, _i32, _vp]),
    "arcq_rope_bf16": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _vp]),
    "arcq_silu_mul_bf16": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp]),
    "arcq_calib_stats_bf16": (_i32, [_vp, _i64, _i32, _vp, _vp, _vp]),
    "arcq_moe_layout": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp]),
    "arcq_silu_mul_grouped_bf16": (_i32, [_vp, _vp, _i64, _i32, _vp, _vp, _i32, _vp, _vp]),
    "arcq_absmax_grouped_bf16": (_i32, [_vp, _vp, _vp, _i32, _i32, _vp, _vp]),
    "arcq_reorder_quantize_x_grouped": (_i32, [_vp, _vp, _vp, _vp, _vp, _i32, _i64, _i32, _i32, _i32, _vp, _vp, _vp]),
    "arcq_matmul_nvfp4_grouped": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _vp, _vp, _vp, _vp]),
    "arcq_matmul_nvfp4_swiglu": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "arcq_matmul_nvfp4_grouped_swiglu": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _vp]),
    "arcq_moe_combine_bf16": (_i32, [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "arcq_matmul_nvfp4_residual": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp]),
    "arcq_matmul_nvfp4_scatter": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _vp]),
    "arcq_sum_partials_bf16": (_i32, [_vp, _i32, _i64, _vp, _vp, _vp]),
    "arcq_rmsnorm_quantize_x_multi": (_i32, [_vp, _vp, _f32, _vp, _i64, _i32, _i32, _vp, _vp, _i32, _vp]),
    "arcq_ep_send_layout": (_i32, [_vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp]),
    "arcq_ep_rows": (_i32, [_vp, _vp, _i32, _i32, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _vp]),
    "arcq_peer_barrier": (_i32, [_vp, _i32, _i32, _vp, _vp]),
    "arcq_peer_poll_error": (_i32, []),
    "arcq_peer_set_wait_limit_ms": (_i32, [_i32]),
    "arcq_peer_alloc": (_i32, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "arcq_peer_free": (_i32, [_vp]),
    "arcq_peer_export": (_i32, [_vp, C.c_char_p]),
    "arcq_peer_open": (_i32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "arcq_peer_close": (_i32, [_vp]),
}
PEER_HANDLE_BYTES = 64

_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m arcquant_b200.build` "
                "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


class ArcqError(RuntimeError):
    def __init__(self, status: int, where: str):
        lib = load()
        text = lib.arcq_status_string(status).decode()
        extra = f" (cudaError {lib.arcq_last_cuda_error()})" if status == ERR_CUDA else ""
        super().__init__(f"{where}: {text}{extra}")
        self.status = status


CALLS = 0   # launching calls into the library that came back through `check` (what a caller may count)


def check(status: int, where: str) -> None:
    global CALLS
    CALLS += 1
    if status != OK:
        raise ArcqError(status, where)

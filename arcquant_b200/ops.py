"""Torch-facing operators over the C ABI, with the reference extension's
signatures (kernels/src/bindings.cpp:99-254 of ARCQuant): they allocate their
outputs, borrow their inputs and run on torch's current CUDA stream.

These are thin: shape bookkeeping in Python, every byte of work in libarcq.so.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


_EXT = None


def _ext():
    """The `agemm` extension module if it has been built (its calls cost about a third of a ctypes
    call on the host), else False.  Both reach the same C ABI."""
    global _EXT
    if _EXT is None:
        import importlib.util
        import os
        import sysconfig

        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "agemm" + sysconfig.get_config_var("EXT_SUFFIX"))
        try:
            import sys

            mod = sys.modules.get("agemm")
            if mod is None or os.path.abspath(getattr(mod, "__file__", "")) != path:
                if not os.path.exists(path):
                    raise ImportError(path)
                spec = importlib.util.spec_from_file_location("agemm", path)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                sys.modules.setdefault("agemm", mod)
            _EXT = mod if hasattr(mod, "silu_mul") else False
        except Exception:
            _EXT = False
    return _EXT


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def set_sm_limit(sms: int) -> int:
    """Later launches use at most `sms` SMs (0 = all), so that collectives on other streams find room to
    run beside them; returns the previous limit."""
    return int(_lib.load().arcq_set_sm_limit(int(sms)))


def sf_bytes(rows: int, k_eff: int) -> int:
    return int(_lib.load().arcq_sf_bytes(rows, k_eff))


def reference_mode(kq: int) -> int:
    return int(_lib.load().arcq_reference_mode(kq))


def _quantize(kind: str, x, gamma, eps, reorder_index, ke: int, mode, out=None, scale=None):
    lib = _lib.load()
    _require(x, torch.bfloat16, "input")
    if x.dim() != 2:
        raise RuntimeError("input must be 2-D [rows, KQ]")
    rows, kq = x.shape
    if mode is None:
        mode = reference_mode(kq)
    idx_ptr = None
    if reorder_index is not None:
        _require(reorder_index, torch.int16, "reorder_index")
        if reorder_index.numel() != kq:
            raise RuntimeError("reorder_index must have KQ entries")
        idx_ptr = reorder_index.data_ptr()
    k_eff = kq + ke
    if out is None:
        q = torch.empty((rows, k_eff // 2), dtype=torch.uint8, device=x.device)
        sf = torch.empty((sf_bytes(rows, k_eff),), dtype=torch.uint8, device=x.device)
    else:   # caller-provided outputs (e.g. slices of larger buffers)
        q, sf = out
        _require(q, torch.uint8, "out codes")
        _require(sf, torch.uint8, "out scales")
        span = ((rows + 127) // 128) * ((k_eff // 16 + 3) // 4) * 512
        if q.numel() < rows * (k_eff // 2) or sf.numel() < span:
            raise RuntimeError("output buffers too small")
    with torch.cuda.device(x.device):
        if kind == "x" and scale is not None:
            _require(scale, torch.float32, "scale")
            rc = lib.arcq_reorder_quantize_x_scaled(x.data_ptr(), scale.data_ptr(), idx_ptr, rows, kq, ke, mode,
                                                    q.data_ptr(), sf.data_ptr(), _stream())
            if rc == _lib.ERR_UNSUPPORTED_K:   # width not covered by the fused path: divide first
                xs = x / scale
                rc = lib.arcq_reorder_quantize_x(xs.data_ptr(), idx_ptr, rows, kq, ke, mode, q.data_ptr(),
                                                 sf.data_ptr(), _stream())
        elif kind == "x":
            rc = lib.arcq_reorder_quantize_x(x.data_ptr(), idx_ptr, rows, kq, ke, mode, q.data_ptr(),
                                             sf.data_ptr(), _stream())
        elif kind == "w":
            rc = lib.arcq_reorder_quantize_w(x.data_ptr(), idx_ptr, rows, kq, ke, mode, q.data_ptr(),
                                             sf.data_ptr(), _stream())
        else:
            _require(gamma, torch.bfloat16, "weight")
            rc = lib.arcq_rmsnorm_quantize_x(x.data_ptr(), gamma.data_ptr(), float(eps), idx_ptr, rows, kq, ke,
                                             q.data_ptr(), sf.data_ptr(), _stream())
    _lib.check(rc, f"{kind}-quantize KQ={kq} KE={ke}")
    return q, sf


def reorder_quantize_x(x, reorder_index, ke: int, mode=None, out=None, scale=None):
    """(QX u8 [M,(KQ+KE)/2], SFX u8 [sf_bytes]) = ARC-NVFP4 of bf16 x [M,KQ].
    scale (0-dim fp32 CUDA tensor): quantize ``x / scale`` instead, the division fused into the kernel."""
    ext = _ext()
    if ext and out is None and scale is not None and reorder_index is not None:
        return ext.reorder_quantize_x_scaled(x, scale, reorder_index, ke, -1 if mode is None else mode)
    return _quantize("x", x, None, 0.0, reorder_index, ke, mode, out, scale)


def reorder_quantize_w(w, reorder_index, ke: int, mode=None):
    """Offline weight packer: residual slots duplicate the critical columns."""
    return _quantize("w", w, None, 0.0, reorder_index, ke, mode)


def rmsnorm_quantize_x(x, weight, eps: float, reorder_index, ke: int, out=None):
    """RMSNorm(x)*weight fused in front of reorder_quantize_x."""
    ext = _ext()
    if ext and out is None and reorder_index is not None:
        return ext.rmsnorm_quantize_x(x, weight, float(eps), reorder_index, ke)
    return _quantize("rms", x, weight, eps, reorder_index, ke, _lib.MODE_16, out)


def _matmul(a, b, sfa, sfb, alpha: float, alpha_a, alpha_b) -> torch.Tensor:
    lib = _lib.load()
    for t, n in ((a, "A"), (b, "B"), (sfa, "SFA"), (sfb, "SFB")):
        _require(t, torch.uint8, n)
    m, kb = a.shape
    n = b.shape[0]
    if b.shape[1] != kb:
        raise RuntimeError("A and B disagree on K")
    c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        # skinny problems split K over idle SMs; the fp32 partial sums need scratch
        ws_bytes = int(lib.arcq_matmul_workspace_bytes(m, n, kb * 2))
        ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=a.device) if ws_bytes else None
        rc = lib.arcq_matmul_nvfp4_ws(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kb * 2,
                                      float(alpha), None if alpha_a is None else alpha_a.data_ptr(),
                                      None if alpha_b is None else alpha_b.data_ptr(), c.data_ptr(),
                                      None if ws is None else ws.data_ptr(), ws_bytes, _stream())
    _lib.check(rc, f"matmul M={m} N={n} K={kb * 2}")
    return c


def matmul(a, b, sfa, sfb, scale) -> torch.Tensor:
    """bf16 [M,N] = scale * (A.SFA)(B.SFB)^T.  ``scale`` may be a Python float or
    a 0-dim tensor; a CUDA 0-dim fp32 tensor is consumed on the device (no
    host synchronisation)."""
    if isinstance(scale, torch.Tensor) and scale.is_cuda and scale.dtype == torch.float32:
        return _matmul(a, b, sfa, sfb, 1.0, scale, None)
    return _matmul(a, b, sfa, sfb, float(scale), None, None)


def matmul_dev_alpha(a, b, sfa, sfb, alpha_a: torch.Tensor, alpha_b: torch.Tensor | None = None) -> torch.Tensor:
    """matmul with alpha = alpha_a * alpha_b, both fp32 scalars in device memory."""
    ext = _ext()
    if ext:
        return ext.matmul_dev_alpha(a, b, sfa, sfb, alpha_a, alpha_b)
    return _matmul(a, b, sfa, sfb, 1.0, alpha_a, alpha_b)


def absmax(x: torch.Tensor) -> torch.Tensor:
    """0-dim fp32 CUDA tensor max|x| of a bf16 tensor, one pass."""
    ext = _ext()
    if ext and x.is_contiguous():
        return ext.absmax(x)
    lib = _lib.load()
    _require(x, torch.bfloat16, "input")
    out = torch.empty((), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.arcq_absmax_bf16(x.data_ptr(), x.numel(), out.data_ptr(), 0, _stream())
    _lib.check(rc, "absmax")
    return out


def rope_inplace(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, heads: int, head_dim: int) -> torch.Tensor:
    """Rotate-half rotary embedding in place on the first `heads` heads of every row of x [tokens, row]
    (bf16); cos / sin fp32 [seq, head_dim], row = token % seq.  Bit-equal to the eager
    ``(x.float() * cos + rotate_half(x.float()) * sin).to(bf16)``."""
    ext = _ext()
    if ext:
        return ext.rope_inplace(x, cos, sin, heads, head_dim)
    lib = _lib.load()
    _require(x, torch.bfloat16, "x")
    _require(cos, torch.float32, "cos")
    _require(sin, torch.float32, "sin")
    if x.dim() != 2 or cos.shape != sin.shape or cos.dim() != 2 or cos.shape[1] != head_dim:
        raise RuntimeError("x must be [tokens, row]; cos / sin [seq, head_dim]")
    with torch.cuda.device(x.device):
        rc = lib.arcq_rope_bf16(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), x.shape[0], x.shape[1], heads, head_dim,
                                cos.shape[0], _stream())
    _lib.check(rc, "rope")
    return x


def silu_mul(gate_up: torch.Tensor, with_amax: bool = True):
    """(out bf16 [tokens, F], amax 0-dim fp32 or None) for gate_up [tokens, 2F] = [gate | up]:
    out = silu(gate) * up as eager bf16 torch computes it, max|out| in the same pass."""
    ext = _ext()
    if ext and with_amax:
        return ext.silu_mul(gate_up)
    lib = _lib.load()
    _require(gate_up, torch.bfloat16, "gate_up")
    if gate_up.dim() != 2 or gate_up.shape[1] % 16:
        raise RuntimeError("gate_up must be [tokens, 2F] with F a multiple of 8")
    tokens, f2 = gate_up.shape
    out = torch.empty((tokens, f2 // 2), dtype=torch.bfloat16, device=gate_up.device)
    amax = torch.empty((), dtype=torch.float32, device=gate_up.device) if with_amax else None
    with torch.cuda.device(gate_up.device):
        rc = lib.arcq_silu_mul_bf16(gate_up.data_ptr(), out.data_ptr(), tokens, f2 // 2,
                                    None if amax is None else amax.data_ptr(), _stream())
    _lib.check(rc, "silu_mul")
    return out, amax


def calib_stats(x: torch.Tensor, chan_absmax: torch.Tensor, above: torch.Tensor | None = None) -> None:
    """Accumulates the calibration statistics of x [..., K] (bf16, CUDA) in one pass: per-channel running
    max|x| into chan_absmax (fp32 [K]) and, if given, the count of elements above an eighth of their row's
    maximum into `above` (int64 scalar tensor)."""
    lib = _lib.load()
    x2 = x.reshape(-1, x.shape[-1])
    _require(x2, torch.bfloat16, "input")
    _require(chan_absmax, torch.float32, "chan_absmax")
    if chan_absmax.numel() != x2.shape[1]:
        raise RuntimeError("chan_absmax must have one entry per channel")
    if above is not None:
        _require(above, torch.int64, "above")
    with torch.cuda.device(x.device):
        rc = lib.arcq_calib_stats_bf16(x2.data_ptr(), x2.shape[0], x2.shape[1], chan_absmax.data_ptr(),
                                       None if above is None else above.data_ptr(), _stream())
    _lib.check(rc, "calib_stats")


def moe_layout(slot_group: torch.Tensor, ngroups: int, tile: int, rows_bound: int, div: int = 1):
    """Padded layout of routed rows in one launch: (dest int32 [n], row_map int32 [rows_bound], groups int32
    [2*ngroups], tile_group int32 [rows_bound/tile]); see `arcq_moe_layout` in arcq.h."""
    lib = _lib.load()
    _require(slot_group, torch.int64, "slot_group")
    n, dev = slot_group.numel(), slot_group.device
    dest = torch.empty((n,), dtype=torch.int32, device=dev)
    row_map = torch.empty((rows_bound,), dtype=torch.int32, device=dev)
    groups = torch.empty((2 * ngroups,), dtype=torch.int32, device=dev)
    tile_group = torch.empty((rows_bound // tile,), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.arcq_moe_layout(slot_group.data_ptr(), n, ngroups, tile, rows_bound, div, dest.data_ptr(),
                                 row_map.data_ptr(), groups.data_ptr(), tile_group.data_ptr(), _stream())
    _lib.check(rc, "moe_layout")
    return dest, row_map, groups, tile_group


def silu_mul_grouped(gate_up: torch.Tensor, tile_group: torch.Tensor, groups: torch.Tensor, ngroups: int):
    """(out bf16 [rows, F], amax fp32 [ngroups]) for grouped rows of gate_up [rows, 2F]: empty 256-row tiles
    are skipped, amax[e] = max|out| over the rows of run e."""
    lib = _lib.load()
    _require(gate_up, torch.bfloat16, "gate_up")
    _require(tile_group, torch.int32, "tile_group")
    _require(groups, torch.int32, "groups")
    rows, f2 = gate_up.shape
    out = torch.empty((rows, f2 // 2), dtype=torch.bfloat16, device=gate_up.device)
    amax = torch.empty((ngroups,), dtype=torch.float32, device=gate_up.device)
    with torch.cuda.device(gate_up.device):
        rc = lib.arcq_silu_mul_grouped_bf16(gate_up.data_ptr(), out.data_ptr(), rows, f2 // 2, tile_group.data_ptr(),
                                            groups.data_ptr(), ngroups, amax.data_ptr(), _stream())
    _lib.check(rc, "silu_mul_grouped")
    return out, amax


def absmax_grouped(x: torch.Tensor, row_map, groups: torch.Tensor, ngroups: int) -> torch.Tensor:
    """fp32 [ngroups]: max|x| over the rows of each run (see `reorder_quantize_x_grouped`)."""
    lib = _lib.load()
    _require(x, torch.bfloat16, "input")
    _require(groups, torch.int32, "groups")
    if row_map is not None:
        _require(row_map, torch.int32, "row_map")
    if groups.numel() != 2 * ngroups:
        raise RuntimeError("groups must hold 2 * ngroups entries")
    out = torch.empty((ngroups,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.arcq_absmax_grouped_bf16(x.data_ptr(), None if row_map is None else row_map.data_ptr(), groups.data_ptr(),
                                          ngroups, x.shape[-1], out.data_ptr(), _stream())
    _lib.check(rc, "absmax_grouped")
    return out


def reorder_quantize_x_grouped(x: torch.Tensor, row_map, scales: torch.Tensor, reorder_indices: torch.Tensor,
                               groups: torch.Tensor, rows_bound: int, ke: int, mode: int = 16):
    """ARC-NVFP4 of grouped rows in one launch.  The output has `rows_bound` rows in runs: run e starts at
    row groups[e] (a multiple of 256), holds groups[E + e] rows, is divided by scales[e] and uses the channel
    order reorder_indices[e]; output row r reads input row row_map[r] (or r).  Everything that describes
    the split lives on the device.  Rows outside the runs are left unwritten."""
    lib = _lib.load()
    _require(x, torch.bfloat16, "input")
    _require(scales, torch.float32, "scales")
    _require(reorder_indices, torch.int16, "reorder_indices")
    _require(groups, torch.int32, "groups")
    ngroups, kq = reorder_indices.shape
    if x.shape[-1] != kq or scales.numel() != ngroups or groups.numel() != 2 * ngroups:
        raise RuntimeError("scales / reorder_indices / groups disagree on the number of runs or on KQ")
    if row_map is not None:
        _require(row_map, torch.int32, "row_map")
        if row_map.numel() < rows_bound:
            raise RuntimeError("row_map must cover rows_bound rows")
    elif x.shape[0] < rows_bound:
        raise RuntimeError("input has fewer rows than rows_bound")
    k_eff = kq + ke
    q = torch.empty((rows_bound, k_eff // 2), dtype=torch.uint8, device=x.device)
    sf = torch.empty((sf_bytes(rows_bound, k_eff),), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.arcq_reorder_quantize_x_grouped(x.data_ptr(), None if row_map is None else row_map.data_ptr(),
                                                 scales.data_ptr(), reorder_indices.data_ptr(), groups.data_ptr(),
                                                 ngroups, rows_bound, kq, ke, mode, q.data_ptr(), sf.data_ptr(), _stream())
    _lib.check(rc, f"grouped x-quantize KQ={kq} KE={ke}")
    return q, sf


def matmul_grouped(a, b, sfa, sfb, tile_group: torch.Tensor, ngroups: int, n: int, alpha_a: torch.Tensor,
                   alpha_b: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [rows, n]: every 256-row tile m of A times the weight matrix tile_group[m] of the `ngroups`
    matrices stacked in b [ngroups * n, K_eff/2] (negative = tile skipped), scaled by
    alpha_a[g] * alpha_b[g]."""
    lib = _lib.load()
    for t, name in ((a, "A"), (b, "B"), (sfa, "SFA"), (sfb, "SFB")):
        _require(t, torch.uint8, name)
    _require(tile_group, torch.int32, "tile_group")
    _require(alpha_a, torch.float32, "alpha_a")
    if alpha_b is not None:
        _require(alpha_b, torch.float32, "alpha_b")
    m, kb = a.shape
    if b.shape != (ngroups * n, kb) or tile_group.numel() < (m + 255) // 256 or alpha_a.numel() != ngroups:
        raise RuntimeError("operand shapes disagree")
    atoms = (kb * 2 // 16 + 3) // 4
    if sfa.numel() < ((m + 127) // 128) * atoms * 512 or sfb.numel() < ((ngroups * n + 127) // 128) * atoms * 512:
        raise RuntimeError("scale buffers are smaller than the scale layout of their operands")
    c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    with torch.cuda.device(a.device):
        rc = lib.arcq_matmul_nvfp4_grouped(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kb * 2,
                                           tile_group.data_ptr(), ngroups, alpha_a.data_ptr(),
                                           None if alpha_b is None else alpha_b.data_ptr(), c.data_ptr(), _stream())
    _lib.check(rc, f"grouped matmul M={m} N={n} K={kb * 2} groups={ngroups}")
    return c


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[2F, K] weight whose rows alternate blocks of `block` gate channels and the same up channels: the row
    order `matmul_swiglu` expects of its B operand."""
    f, k = w_gate.shape
    if w_up.shape != (f, k) or f % block:
        raise RuntimeError("gate and up must have the same shape, with a multiple of 128 output channels")
    return torch.stack([w_gate.reshape(f // block, block, k), w_up.reshape(f // block, block, k)], dim=1).reshape(2 * f, k)


def matmul_swiglu(a, b, sfa, sfb, alpha_a: torch.Tensor, alpha_b: torch.Tensor | None = None):
    """(act bf16 [M, N/2], amax 0-dim fp32): gate/up GEMM over an interleaved weight (`interleave_gate_up`) with
    silu(gate) * up and its max|.| taken in the epilogue."""
    lib = _lib.load()
    for t, name in ((a, "A"), (b, "B"), (sfa, "SFA"), (sfb, "SFB")):
        _require(t, torch.uint8, name)
    _require(alpha_a, torch.float32, "alpha_a")
    if alpha_b is not None:
        _require(alpha_b, torch.float32, "alpha_b")
    m, kb = a.shape
    n = b.shape[0]
    if b.shape[1] != kb or n % 256:
        raise RuntimeError("A and B disagree on K, or N is not a multiple of 256")
    atoms = (kb * 2 // 16 + 3) // 4
    if sfa.numel() < ((m + 127) // 128) * atoms * 512 or sfb.numel() < (n // 128) * atoms * 512:
        raise RuntimeError("scale buffers are smaller than the scale layout of their operands")
    c = torch.empty((m, n // 2), dtype=torch.bfloat16, device=a.device)
    amax = torch.empty((), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        rc = lib.arcq_matmul_nvfp4_swiglu(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kb * 2,
                                          alpha_a.data_ptr(), None if alpha_b is None else alpha_b.data_ptr(),
                                          c.data_ptr(), amax.data_ptr(), _stream())
    _lib.check(rc, f"swiglu matmul M={m} N={n} K={kb * 2}")
    return c, amax


def matmul_grouped_swiglu(a, b, sfa, sfb, tile_group: torch.Tensor, groups: torch.Tensor, ngroups: int, n: int,
                          alpha_a: torch.Tensor, alpha_b: torch.Tensor | None = None):
    """`matmul_grouped` with the SwiGLU epilogue: (act bf16 [rows, n/2], amax fp32 [ngroups])."""
    lib = _lib.load()
    for t, name in ((a, "A"), (b, "B"), (sfa, "SFA"), (sfb, "SFB")):
        _require(t, torch.uint8, name)
    _require(tile_group, torch.int32, "tile_group")
    _require(groups, torch.int32, "groups")
    _require(alpha_a, torch.float32, "alpha_a")
    if alpha_b is not None:
        _require(alpha_b, torch.float32, "alpha_b")
    m, kb = a.shape
    if b.shape != (ngroups * n, kb) or tile_group.numel() < (m + 255) // 256 or alpha_a.numel() != ngroups or n % 256:
        raise RuntimeError("operand shapes disagree")
    atoms = (kb * 2 // 16 + 3) // 4
    if sfa.numel() < ((m + 127) // 128) * atoms * 512 or sfb.numel() < ((ngroups * n + 127) // 128) * atoms * 512:
        raise RuntimeError("scale buffers are smaller than the scale layout of their operands")
    c = torch.empty((m, n // 2), dtype=torch.bfloat16, device=a.device)
    amax = torch.empty((ngroups,), dtype=torch.float32, device=a.device)
    with torch.cuda.device(a.device):
        rc = lib.arcq_matmul_nvfp4_grouped_swiglu(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kb * 2,
                                                  tile_group.data_ptr(), groups.data_ptr(), ngroups, alpha_a.data_ptr(),
                                                  None if alpha_b is None else alpha_b.data_ptr(), c.data_ptr(),
                                                  amax.data_ptr(), _stream())
    _lib.check(rc, f"grouped swiglu matmul M={m} N={n} K={kb * 2} groups={ngroups}")
    return c, amax


def moe_combine(y: torch.Tensor, pos: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """out [T, H] = sum_j bf16(y[pos[t, j]] * weights[t, j]) in bf16: the routed copies of every token,
    weighted and added (pos int32 [T, k], weights bf16 [T, k])."""
    lib = _lib.load()
    _require(y, torch.bfloat16, "y")
    _require(pos, torch.int32, "pos")
    _require(weights, torch.bfloat16, "weights")
    tokens, k = pos.shape
    out = torch.empty((tokens, y.shape[1]), dtype=torch.bfloat16, device=y.device)
    with torch.cuda.device(y.device):
        rc = lib.arcq_moe_combine_bf16(y.data_ptr(), pos.data_ptr(), weights.data_ptr(), out.data_ptr(), tokens,
                                       y.shape[1], k, _stream())
    _lib.check(rc, "moe_combine")
    return out


def gemm_poll_error() -> int:
    return int(_lib.load().arcq_gemm_poll_error())


def matmul_scatter(a, b, sfa, sfb, alpha_a: torch.Tensor, alpha_b: torch.Tensor | None, dests) -> None:
    """GEMM of `matmul_dev_alpha` whose result rows leave for len(dests) buffers of M / len(dests) rows each:
    dests are device addresses (ints) of bf16 [M / len(dests), N] blocks - receive slots in the peers' memory
    (see `peer.PeerSlots`) or local memory."""
    lib = _lib.load()
    for t, name in ((a, "A"), (b, "B"), (sfa, "SFA"), (sfb, "SFB")):
        _require(t, torch.uint8, name)
    _require(alpha_a, torch.float32, "alpha_a")
    if alpha_b is not None:
        _require(alpha_b, torch.float32, "alpha_b")
    m, kb = a.shape
    n = b.shape[0]
    nd = len(dests)
    if b.shape[1] != kb:
        raise RuntimeError("A and B disagree on K")
    if nd < 1 or nd > 8 or m % nd or (m // nd) % 32:
        raise RuntimeError("rows must split evenly over 1..8 destinations, in multiples of 32")
    atoms = (kb * 2 // 16 + 3) // 4
    if sfa.numel() < ((m + 127) // 128) * atoms * 512 or sfb.numel() < ((n + 127) // 128) * atoms * 512:
        raise RuntimeError("scale buffers are smaller than the scale layout of their operands")
    arr = (C.c_void_p * nd)(*[int(d) for d in dests])
    with torch.cuda.device(a.device):
        rc = lib.arcq_matmul_nvfp4_scatter(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kb * 2,
                                           alpha_a.data_ptr(), None if alpha_b is None else alpha_b.data_ptr(),
                                           arr, nd, _stream())
    _lib.check(rc, f"scatter matmul M={m} N={n} K={kb * 2} dests={nd}")


def sum_partials(srcs, elems: int, out: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """out = residual + bf16(sum of the bf16 blocks at the device addresses `srcs`, fp32, in that order)."""
    lib = _lib.load()
    _require(out, torch.bfloat16, "out")
    if residual is not None:
        _require(residual, torch.bfloat16, "residual")
        if residual.numel() != elems:
            raise RuntimeError("residual and sources disagree on the element count")
    if out.numel() != elems or elems % 8:
        raise RuntimeError("out must hold `elems` elements, a multiple of 8")
    n = len(srcs)
    arr = (C.c_void_p * n)(*[int(p) for p in srcs])
    with torch.cuda.device(out.device):
        rc = lib.arcq_sum_partials_bf16(arr, n, elems, None if residual is None else residual.data_ptr(),
                                        out.data_ptr(), _stream())
    _lib.check(rc, f"sum of {n} partials, {elems} elements")
    return out


def rmsnorm_quantize_x_multi(x, weight, eps: float, reorder_index, ke: int, q_dests, sf_dests) -> None:
    """`rmsnorm_quantize_x` into destination 0 and a copy of the result to the others: q_dests[d] / sf_dests[d]
    are device addresses (ints) of where these rows' codes and scale tiles start in destination d (this rank's or
    a peer's memory)."""
    lib = _lib.load()
    _require(x, torch.bfloat16, "input")
    _require(weight, torch.bfloat16, "weight")
    _require(reorder_index, torch.int16, "reorder_index")
    rows, kq = x.shape
    n = len(q_dests)
    if weight.numel() != kq or reorder_index.numel() != kq or len(sf_dests) != n:
        raise RuntimeError("gain / channel order must have one entry per channel; one scale address per code address")
    qa = (C.c_void_p * n)(*[int(p) for p in q_dests])
    sa = (C.c_void_p * n)(*[int(p) for p in sf_dests])
    with torch.cuda.device(x.device):
        rc = lib.arcq_rmsnorm_quantize_x_multi(x.data_ptr(), weight.data_ptr(), float(eps), reorder_index.data_ptr(),
                                               rows, kq, ke, qa, sa, n, _stream())
    _lib.check(rc, f"rmsnorm_quantize_x to {n} destinations, rows={rows} KQ={kq} KE={ke}")


def peer_barrier(flag_blocks, rank: int, counter: torch.Tensor) -> None:
    """Device-side barrier of a tensor-parallel group on the current stream (see `peer.PeerBarrier`)."""
    lib = _lib.load()
    n = len(flag_blocks)
    arr = (C.c_void_p * n)(*[int(p) for p in flag_blocks])
    with torch.cuda.device(counter.device):
        rc = lib.arcq_peer_barrier(arr, int(rank), n, counter.data_ptr(), _stream())
    _lib.check(rc, "peer barrier")


def peer_poll_error() -> int:
    """ARCQ_ERR_TIMEOUT if a peer barrier gave up waiting since the last poll (synchronises the device)."""
    return int(_lib.load().arcq_peer_poll_error())


def matmul_residual(a, b, sfa, sfb, alpha_a: torch.Tensor, alpha_b: torch.Tensor | None, residual: torch.Tensor,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 [M, N] = residual + bf16(alpha_a * alpha_b * (A.SFA)(B.SFB)^T), the addition done in the GEMM's epilogue
    (same bits as `matmul_dev_alpha` followed by a bf16 addition)."""
    lib = _lib.load()
    for t, name in ((a, "A"), (b, "B"), (sfa, "SFA"), (sfb, "SFB")):
        _require(t, torch.uint8, name)
    _require(alpha_a, torch.float32, "alpha_a")
    if alpha_b is not None:
        _require(alpha_b, torch.float32, "alpha_b")
    _require(residual, torch.bfloat16, "residual")
    m, kb = a.shape
    n = b.shape[0]
    if b.shape[1] != kb or tuple(residual.shape) != (m, n):
        raise RuntimeError("A and B disagree on K, or the residual is not [M, N]")
    atoms = (kb * 2 // 16 + 3) // 4
    if sfa.numel() < ((m + 127) // 128) * atoms * 512 or sfb.numel() < ((n + 127) // 128) * atoms * 512:
        raise RuntimeError("scale buffers are smaller than the scale layout of their operands")
    c = torch.empty((m, n), dtype=torch.bfloat16, device=a.device) if out is None else out
    _require(c, torch.bfloat16, "out")
    with torch.cuda.device(a.device):
        rc = lib.arcq_matmul_nvfp4_residual(a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), m, n, kb * 2,
                                            alpha_a.data_ptr(), None if alpha_b is None else alpha_b.data_ptr(),
                                            residual.data_ptr(), c.data_ptr(), _stream())
    _lib.check(rc, f"matmul with residual M={m} N={n} K={kb * 2}")
    return c


def ep_send_layout(ids: torch.Tensor, e_local: int, ep: int, cap: int, rank: int, slot_tables, overflow: torch.Tensor):
    """int32 [n]: place of every routed copy in the receive buffers of the experts' ranks (see
    `arcq_ep_send_layout` in arcq.h); slot_tables: device addresses (ints) of every rank's slot table."""
    lib = _lib.load()
    _require(ids, torch.int64, "ids")
    _require(overflow, torch.int32, "overflow")
    n = ids.numel()
    slot = torch.empty((n,), dtype=torch.int32, device=ids.device)
    arr = (C.c_void_p * ep)(*[int(p) for p in slot_tables])
    with torch.cuda.device(ids.device):
        rc = lib.arcq_ep_send_layout(ids.data_ptr(), n, e_local, ep, cap, rank, slot.data_ptr(), arr, overflow.data_ptr(),
                                     _stream())
    _lib.check(rc, "ep_send_layout")
    return slot


def ep_rows(src: torch.Tensor, item_src, div: int, src_limit: int, item_slot, n: int, cap: int, ep: int, rank: int,
            dsts) -> None:
    """Rows of `src` [*, H] bf16 into the peers' buffers (see `arcq_ep_rows` in arcq.h); dsts: device addresses."""
    lib = _lib.load()
    _require(src, torch.bfloat16, "src")
    for t, name in ((item_src, "item_src"), (item_slot, "item_slot")):
        if t is not None:
            _require(t, torch.int32, name)
    arr = (C.c_void_p * ep)(*[int(p) for p in dsts])
    with torch.cuda.device(src.device):
        rc = lib.arcq_ep_rows(src.data_ptr(), None if item_src is None else item_src.data_ptr(), div, src_limit,
                              None if item_slot is None else item_slot.data_ptr(), n, src.shape[1] * 2, cap, ep, rank,
                              arr, _stream())
    _lib.check(rc, "ep_rows")


def peer_set_wait_limit_ms(ms: int) -> int:
    """Bound of the wait inside later `peer_barrier` launches (default 10 000 ms); returns the previous one."""
    return int(_lib.load().arcq_peer_set_wait_limit_ms(int(ms)))

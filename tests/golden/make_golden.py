"""Generates the fixtures in this directory.  Run from the repository root:

    python tests/golden/make_golden.py [--reference /path/to/ARCQuant]

Three kinds of fixtures:

1. Known-answer tables for the number formats, computed HERE with exact
   rational arithmetic straight from the format definitions (independent of
   the C oracle): e2m1 (values 0,.5,1,1.5,2,3,4,6 with sign; round to nearest,
   ties to the even mantissa bit, saturating) and ue4m3 (bias 7, 3 mantissa
   bits, subnormal step 2^-9, max 448).
2. The scale-factor layout, enumerated as nested loops over the 512-byte atom
   (row tiles, K atoms, 32 rows, 4 row quads, 4 columns) rather than by the
   closed formula the oracle and the kernels use.
3. Outputs of the reference's own CPU-runnable fake-quant path
   (model/quantize.py of ARCQuant), produced by importing it from a checkout
   given with --reference; stored as SHA-256 digests plus a small slice.  The
   test-suite compares the oracle (run with the fake path's arithmetic knobs)
   and oracle/fake_port.py against them.  Without --reference this part is
   left as it is on disk.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import struct
import sys
import types
from fractions import Fraction

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

E2M1 = [Fraction(0), Fraction(1, 2), Fraction(1), Fraction(3, 2), Fraction(2), Fraction(3), Fraction(4), Fraction(6)]


def f32(x: float) -> float:
    return struct.unpack("f", struct.pack("f", x))[0]


def e2m1_encode_exact(x: float) -> int:
    sign = 8 if (struct.unpack("I", struct.pack("f", x))[0] >> 31) else 0
    a = abs(Fraction(x))
    best, best_d = None, None
    for code, v in enumerate(E2M1):
        d = abs(a - v)
        if best is None or d < best_d or (d == best_d and (code & 1) == 0):
            best, best_d = code, d
    return sign | best


def ue4m3_value(code: int) -> Fraction:
    e, m = (code >> 3) & 15, code & 7
    if e == 0:
        return Fraction(m, 512)
    return (1 + Fraction(m, 8)) * Fraction(2) ** (e - 7)


def ue4m3_encode_exact(x: float) -> int:
    a = Fraction(x)
    if a >= 448:
        return 0x7E
    best, best_d = None, None
    for code in range(0x7F):
        d = abs(a - ue4m3_value(code))
        if best is None or d < best_d or (d == best_d and (code & 1) == 0):
            best, best_d = code, d
    return best


def make_kats():
    vals = []
    for k in range(-512, 513):
        vals.append(k / 64.0)
    ties = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    for t in ties:
        for s in (1.0, -1.0):
            vals += [s * t, s * float(np.nextafter(np.float32(t), np.float32(10))),
                     s * float(np.nextafter(np.float32(t), np.float32(0)))]
    vals += [0.0, -0.0, 1e-30, -1e-30, 6.0, -6.0, 100.0, -100.0]
    e2m1 = [[struct.unpack("I", struct.pack("f", v))[0], e2m1_encode_exact(f32(v))] for v in vals]

    ue = []
    codes = list(range(0x7F))
    for c in codes:
        v = float(ue4m3_value(c))
        ue.append(v)
        if c + 1 < 0x7F:
            mid = float((ue4m3_value(c) + ue4m3_value(c + 1)) / 2)  # exactly representable in fp32
            ue += [mid, float(np.nextafter(np.float32(mid), np.float32(1e9))),
                   float(np.nextafter(np.float32(mid), np.float32(0)))]
    ue += [447.9, 448.0, 0.001953125, 0.0029296875]
    ue = [v for v in ue if v > 0]
    ue4m3 = [[struct.unpack("I", struct.pack("f", v))[0], ue4m3_encode_exact(f32(v))] for v in ue]
    decode = [[c, struct.unpack("I", struct.pack("f", float(ue4m3_value(c))))[0]] for c in codes]
    with open(os.path.join(HERE, "kat_formats.json"), "w") as f:
        json.dump({"e2m1_encode": e2m1, "ue4m3_encode": ue4m3, "ue4m3_decode": decode,
                   "note": "[fp32 bit pattern, expected code]; decode: [code, fp32 bit pattern]"}, f)


def enumerate_sf(rows: int, k_eff: int) -> np.ndarray:
    """offset[row, col] by walking the layout in memory order."""
    ncols = k_eff // 16
    natoms = (ncols + 3) // 4
    ntiles = (rows + 127) // 128
    table = -np.ones((ntiles * 128, natoms * 4), dtype=np.int64)
    off = 0
    for rt in range(ntiles):
        for ka in range(natoms):
            for r32 in range(32):
                for quad in range(4):
                    for c in range(4):
                        table[rt * 128 + quad * 32 + r32, ka * 4 + c] = off
                        off += 1
    return table[:rows, :ncols]


def make_sf():
    out = {}
    for rows, k_eff in ((1, 4224), (129, 4224), (512, 14464), (300, 4160)):
        t = enumerate_sf(rows, k_eff)
        spots = [[int(r), int(c), int(t[r, c])] for r, c in
                 ((0, 0), (rows - 1, k_eff // 16 - 1), (rows // 2, 5), (min(rows - 1, 33), 7), (min(rows - 1, 127), 3))]
        out[f"{rows}x{k_eff}"] = {"sha256": hashlib.sha256(t.astype("<i8").tobytes()).hexdigest(), "spots": spots}
    with open(os.path.join(HERE, "sf_layout.json"), "w") as f:
        json.dump(out, f, indent=1)


def make_reference(ref_root: str):
    import torch

    sys.modules["agemm"] = types.ModuleType("agemm")  # model/quantize.py imports the CUDA extension at line 8
    sys.path.insert(0, os.path.join(ref_root, "model"))
    import quantize as RQ  # the reference's fake path

    from arcquant_b200 import synth

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    x, w, idx, ke = synth.config1()
    i64 = idx.to(torch.int64)
    rows = 64                      # a slice of config 1 keeps the fixture small and the run short
    xs = (x[:rows] / synth.global_scale(x)).contiguous()      # bf16, as the reference's caller forms it on CPU
    ws = (w[:rows] / synth.global_scale(w)).contiguous()
    xg = torch.index_select(xs, 1, i64).float()
    wg = torch.index_select(ws, 1, i64).float()
    ar = torch.arange(4096)
    out = {}
    # block quantizer alone, then the two ARC entry points
    fq = RQ.quantize_nvfp4_tensor(xg.clone())
    fe = RQ.quantize_nvfp4_tensor((xg - fq)[:, -ke:].contiguous())
    full = torch.cat([fq, fe], dim=1).numpy().astype("<f4")
    out["x_values_sha256"] = hashlib.sha256(full.tobytes()).hexdigest()
    qx, _, sx = RQ.fake_reorder_quantize_x(torch.index_select(xs, 1, i64), ar, ke)
    qw, _, sw = RQ.fake_reorder_quantize_w(torch.index_select(ws, 1, i64), ar, ke)
    qx0, _, _ = RQ.fake_reorder_quantize_x(torch.index_select(xs, 1, i64), ar, 0)
    out["fake_x_sha256"] = hashlib.sha256(qx.float().numpy().astype("<f4").tobytes()).hexdigest()
    out["fake_w_sha256"] = hashlib.sha256(qw.float().numpy().astype("<f4").tobytes()).hexdigest()
    out["fake_x_ke0_sha256"] = hashlib.sha256(qx0.float().numpy().astype("<f4").tobytes()).hexdigest()
    out["fake_x_scale"] = float(sx)
    out["fake_w_scale"] = float(sw)
    out["rows"] = rows
    out["ke"] = ke
    with open(os.path.join(HERE, "reference_fake_config1.json"), "w") as f:
        json.dump(out, f, indent=1)
    np.savez_compressed(os.path.join(HERE, "reference_fake_config1_slice.npz"),
                        x_values=full[:4], fake_x=qx.float().numpy()[:4], fake_w=qw.float().numpy()[:4])


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None)
    a = ap.parse_args()
    make_kats()
    make_sf()
    if a.reference:
        make_reference(a.reference)
    print("fixtures written to", HERE)

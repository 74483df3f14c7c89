"""Generates kat_formats_cutlass.json: the known-answer tables of the e2m1 and ue4m3 conversions as
answered by NVIDIA CUTLASS's own converters, the templates the reference's kernels call
(kernels/src/reorder.cu:98-104 of ARCQuant).  Run from the repository root:

    python tests/golden/make_kat_cutlass.py

It host-compiles tests/golden/kat_cutlass.cu with nvcc against a CUTLASS header tree (by default the copy
vendored inside the installed `flashinfer` package; the reference's own CUTLASS is an un-pinned, un-vendored
git submodule, so there is no pinned version to take instead) and feeds it the same inputs as
make_golden.py's exact-arithmetic tables plus every e2m1 decision boundary and its fp32 neighbours at a
spread of binades.  Test infrastructure only: nothing of CUTLASS is built into the library.
"""
from __future__ import annotations

import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def cutlass_include() -> str:
    env = os.environ.get("CUTLASS_INCLUDE")
    if env:
        return env
    import flashinfer
    return os.path.join(os.path.dirname(flashinfer.__file__), "data", "cutlass", "include")


def bits(x: float) -> int:
    return struct.unpack("I", struct.pack("f", x))[0]


def main():
    kat = json.load(open(os.path.join(HERE, "kat_formats.json")))
    e2m1_in = [b for b, _ in kat["e2m1_encode"]]
    ue_in = [b for b, _ in kat["ue4m3_encode"]]
    # every multiple of 1/32 up to 8 with its two fp32 neighbours, both signs: all decision boundaries of e2m1
    for k in range(0, 257):
        v = np.float32(k / 32.0)
        for w in (v, np.nextafter(v, np.float32(100)), np.nextafter(v, np.float32(-100))):
            e2m1_in += [bits(float(w)), bits(float(-w))]
    rng = np.random.default_rng(0)
    e2m1_in += [bits(float(v)) for v in rng.standard_normal(4000).astype(np.float32) * 3]
    ue_in += [bits(float(v)) for v in np.exp(rng.uniform(np.log(1e-3), np.log(500.0), 4000)).astype(np.float32)]
    e2m1_in, ue_in = sorted(set(e2m1_in)), sorted(set(ue_in))
    lines = [f"e2m1 {b:x}" for b in e2m1_in] + [f"ue4m3 {b:x}" for b in ue_in] + [f"dec {c:x}" for c in range(0x7F)]
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "kat_cutlass")
        subprocess.check_call(["nvcc", "-std=c++17", "-O1", "-I" + cutlass_include(), os.path.join(HERE, "kat_cutlass.cu"),
                               "-o", exe])
        p = subprocess.run([exe], input="\n".join(lines) + "\n", capture_output=True, text=True, check=True)
    out = [int(v) for v in p.stdout.split()]
    assert len(out) == len(lines)
    n1, n2 = len(e2m1_in), len(ue_in)
    res = {"source": "cutlass::NumericConverter<float_e2m1_t | float_ue4m3_t, float, round_to_nearest>, host code path, "
                     + p.stderr.strip() + " (header tree vendored in the flashinfer package)",
           "e2m1_encode": [[b, c] for b, c in zip(e2m1_in, out[:n1])],
           "ue4m3_encode": [[b, c] for b, c in zip(ue_in, out[n1:n1 + n2])],
           "ue4m3_decode": [[c, b] for c, b in zip(range(0x7F), out[n1 + n2:])],
           "note": "[fp32 bit pattern, code]; decode: [code, fp32 bit pattern]"}
    with open(os.path.join(HERE, "kat_formats_cutlass.json"), "w") as f:
        json.dump(res, f)
    print(f"{n1} e2m1, {n2} ue4m3 inputs; {res['source']}")


if __name__ == "__main__":
    sys.exit(main())

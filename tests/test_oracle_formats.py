"""The oracle's number formats against known-answer tables computed with exact rational
arithmetic from the format definitions (tests/golden/make_golden.py)."""
import json
import os
import struct

import numpy as np

from oracle import oracle as O


def _f(bits):
    return struct.unpack("f", struct.pack("I", bits))[0]


def test_e2m1_known_answers(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "kat_formats.json")))
    L = O.lib()
    assert len(kat["e2m1_encode"]) > 1000
    for bits, code in kat["e2m1_encode"]:
        assert L.arcq_e2m1_encode(_f(bits)) == code, (_f(bits), code)


def test_e2m1_tie_points_and_signed_zero():
    L = O.lib()
    ties = {0.25: 0.0, 0.75: 1.0, 1.25: 1.0, 1.75: 2.0, 2.5: 2.0, 3.5: 4.0, 5.0: 4.0}
    for x, want in ties.items():
        assert L.arcq_e2m1_decode(L.arcq_e2m1_encode(x)) == want
        assert L.arcq_e2m1_decode(L.arcq_e2m1_encode(-x)) == -want
    assert L.arcq_e2m1_encode(-0.0) == 0x8
    assert L.arcq_e2m1_encode(-0.1) == 0x8          # underflow keeps the sign
    assert L.arcq_e2m1_encode(1e9) == 0x7 and L.arcq_e2m1_encode(-1e9) == 0xF


def test_ue4m3_known_answers(golden_dir):
    kat = json.load(open(os.path.join(golden_dir, "kat_formats.json")))
    L = O.lib()
    for bits, code in kat["ue4m3_encode"]:
        assert L.arcq_ue4m3_encode(_f(bits)) == code, (_f(bits), code)
    for code, bits in kat["ue4m3_decode"]:
        assert L.arcq_ue4m3_decode(code) == _f(bits)


def test_ue4m3_limits():
    L = O.lib()
    assert L.arcq_ue4m3_encode(0.001953125) == 1        # 2^-9, smallest subnormal
    assert L.arcq_ue4m3_encode(448.0) == 0x7E and L.arcq_ue4m3_encode(1e6) == 0x7E
    assert L.arcq_ue4m3_decode(0x7E) == 448.0


def test_reciprocal_is_the_correctly_rounded_one():
    """The kernels compute fp32(1.0 / double(S)); for every scale code that equals the IEEE fp32
    reciprocal, which is what the CUDA path evaluates with rcp.rn."""
    L = O.lib()
    for code in range(1, 0x7F):
        s = np.float32(L.arcq_ue4m3_decode(code))
        assert np.float32(1.0 / np.float64(s)) == np.float32(1.0) / s


def test_rsqrt_rn_is_nearest():
    from decimal import Decimal, getcontext

    getcontext().prec = 60
    L = O.lib()
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.uniform(1e-6, 1e4, 3000), rng.uniform(0.5, 2.0, 3000), [1.0, 4.0, 0.25, 1e-5]])
    for v in vals.astype(np.float32):
        r = np.float32(L.arcq_rsqrt_rn(float(v)))
        exact = Decimal(1) / Decimal(float(v)).sqrt()
        err = abs(Decimal(float(r)) - exact)
        for nb in (np.nextafter(r, np.float32(np.inf)), np.nextafter(r, np.float32(0))):
            assert err <= abs(Decimal(float(nb)) - exact)


def test_formats_against_the_dependency_itself(golden_dir):
    """The same conversions as answered by CUTLASS's own host-side converters - the templates the
    reference's kernels call (kernels/src/reorder.cu:98-104 of ARCQuant: NumericConverter<float_e2m1_t |
    float_ue4m3_t, float, round_to_nearest>) - tabulated by tests/golden/make_kat_cutlass.py.  The oracle
    is held to them on the domain the kernels feed the converters: |x| <= 6 for e2m1 (the kernels clamp
    first, reorder.cu:153-164) and [2^-9, 448] for the block scale (reorder.cu:138)."""
    kat = json.load(open(os.path.join(golden_dir, "kat_formats_cutlass.json")))
    L = O.lib()
    n = 0
    for bits, code in kat["e2m1_encode"]:
        x = _f(bits)
        if abs(x) <= 6.0:
            assert L.arcq_e2m1_encode(x) == code, (x, code)
            n += 1
    assert n > 4000
    n = 0
    for bits, code in kat["ue4m3_encode"]:
        x = _f(bits)
        if 0.001953125 <= x <= 448.0:
            assert L.arcq_ue4m3_encode(x) == code, (x, code)
            n += 1
    assert n > 3000
    for code, bits in kat["ue4m3_decode"]:
        assert L.arcq_ue4m3_decode(code) == _f(bits)
    # and the two tables agree with one another wherever both have an entry
    exact = json.load(open(os.path.join(golden_dir, "kat_formats.json")))
    lib = dict(map(tuple, kat["e2m1_encode"]))
    assert all(lib[b] == c for b, c in exact["e2m1_encode"] if abs(_f(b)) <= 6.0)
    lib = dict(map(tuple, kat["ue4m3_encode"]))
    assert all(lib[b] == c for b, c in exact["ue4m3_encode"] if 0.001953125 <= _f(b) <= 448.0)

"""Host-side arithmetic of bench.py: the algorithmic byte and flop counts its roofline fractions rest on."""
import importlib.util
import os

import pytest

_SPEC = importlib.util.spec_from_file_location("arcq_bench", os.path.join(os.path.dirname(__file__), "..", "bench.py"))
bench = importlib.util.module_from_spec(_SPEC)
_SPEC.loader.exec_module(bench)


def test_quantizer_bytes_per_token():
    # 2 bytes per input channel, half a byte per stored code, one scale byte per 16 stored codes
    assert bench.quant_bytes_per_token(4096, 128) == 2 * 4096 + 4224 // 2 + 4224 // 16 == 10568
    assert bench.quant_bytes_per_token(14336, 128) == 2 * 14336 + 14464 // 2 + 14464 // 16
    # the measured DRAM traffic per token stays below the algorithmic bytes (part of the output is still in L2)
    assert 2 * 4096 < bench.TRAFFIC_PER_TOKEN_NCU < 10568


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_layer_roofline_terms(world):
    hbm, tf = 6500.0, 1600.0
    r = bench.layer_roofline(world, hbm, tf, sp=world > 1)
    assert abs(r["sum_ms"] - (r["gemm_ms"] + r["hbm_ms"] + r["attention_ms"] + r["collective_ms"])) < 1e-12
    T = bench.LAYER_BATCH * bench.LAYER_SEQ
    k1 = bench.HIDDEN + bench.KE
    ke_r = bench.KE if world == 1 else 64
    flops = 2.0 * T * ((6144 // world) * k1 + bench.HIDDEN * (4096 // world + ke_r) + (2 * bench.FFN // world) * k1 +
                       bench.HIDDEN * (bench.FFN // world + ke_r))
    assert abs(r["gemm_ms"] - flops / (4 * tf * 1e12) * 1e3) < 1e-9
    if world == 1:
        assert r["collective_ms"] == 0.0
    else:
        f = (world - 1) / world
        want = 2 * f * T * bench.HIDDEN * 2 + 2 * f * T * (k1 * 9 // 16)     # two reduce-scatters, two packed all-gathers
        assert abs(r["collective_ms"] - want / (bench.NVLINK_GBS * 1e9) * 1e3) < 1e-9
    # one rank's share shrinks with the group
    if world > 1:
        assert r["gemm_ms"] < bench.layer_roofline(1, hbm, tf, sp=False)["gemm_ms"]


def test_moe_roofline_terms():
    r1, r4 = bench.moe_roofline(1, 6500.0, 1600.0), bench.moe_roofline(4, 6500.0, 1600.0)
    assert r1["collective_ms"] == 0.0 and r4["collective_ms"] > 0.0
    assert abs(r4["gemm_ms"] * 4 - r1["gemm_ms"]) < 1e-9
    for r in (r1, r4):
        assert abs(r["sum_ms"] - (r["gemm_ms"] + r["hbm_ms"] + r["collective_ms"])) < 1e-12

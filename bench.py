"""Benchmark of the ARC-NVFP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One GPU (the default): the headline line is the fused RMSNorm + channel reorder + NVFP4 quantize + ARC
residual kernel on 32768 tokens x 4096 channels, KE = 128, reported as GB/s of algorithmic bytes
(2*KQ + K_eff/2 + K_eff/16 per token) against the measured HBM copy bandwidth.  A "step" is one pass of
that kernel over one batch already resident in HBM; the batch (268 MB in, 78 MB out) is larger than the
126 MB L2, so no flush is needed between steps.  `e2e` is the same pass with pinned HOST buffers on both
sides (`arcquant_b200/host_pipeline.py`).  `extra` carries the other quantities the contract names: the
block-scaled GEMM at Llama-3-8B projection shapes (with the cuBLASLt NVFP4 GEMM of `torch._scaled_mm`
beside it as a third-party comparator), the token / residual-width grid of the quantizer and the M x
shape grid of the GEMM, the Llama-3-8B-shape decoder layer and the Mixtral-shape MoE block with their
rooflines, and the CPU fake-quant timings of the reference's path for each of them.

Several GPUs (`--gpus N` under torchrun): the headline is the quantity the contract names for them, the
Llama-3-8B-shape decoder layer run tensor-parallel over the N ranks (16384 tokens in total: strong
scaling), in its sequence-parallel form, replayed as a CUDA graph; tokens/s.  Before anything is timed,
the small-configuration layer and MoE block are run through NCCL and compared with the same shards
added up inside one process (`extra.parity`); a disagreement aborts the run.

`--impl reference` times the reference's own CPU path for the same quantity (its torch fake-quant
functions, restated in oracle/fake_port.py and pinned against the reference's outputs) on a bounded
sample of the same workload, on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HIDDEN = 4096
FFN = 14336
KE = 128
TOKENS = 32768
LAYER_BATCH, LAYER_SEQ = 8, 2048
MOE_TOKENS = 4096
EPS = 1e-5
BYTES_PER_TOKEN = 2 * HIDDEN + (HIDDEN + KE) // 2 + (HIDDEN + KE) // 16      # 10568
# dram__bytes_read + dram__bytes_write per token, from the ncu capture of a 16384-token launch of the
# current fused kernel summarised under profiles/: (134.28 + 15.59) MB / 16384 tokens (part of the output
# is still dirty in L2 when the kernel ends, so the write part is below the algorithmic 2376 B/token);
# traffic is proportional to tokens
TRAFFIC_PER_TOKEN_NCU = 9147
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
NVLINK_GBS = 770.0          # measured peer copy, per direction per GPU
GEMM_SHAPES = (("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 28672, 4096), ("down", 4096, 14336))


def quant_bytes_per_token(kq: int, ke: int) -> int:
    return 2 * kq + (kq + ke) // 2 + (kq + ke) // 16


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=f,
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = []
        try:
            for line in open(self.path):
                parts = [s.strip() for s in line.split(",")]
                if len(parts) >= 7:
                    rows.append(parts)
            os.unlink(self.path)
        except Exception:
            pass
        if rows:
            clocks = sorted(float(r[0]) for r in rows if r[0].replace(".", "").isdigit())
            if clocks:
                out["sm_mhz"] = clocks[len(clocks) // 2]
            try:
                out["sm_max_mhz"] = float(rows[0][1])
            except Exception:
                pass
            try:
                out["power_w_max"] = max(float(r[2]) for r in rows)
            except Exception:
                pass
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for i, n in enumerate(names):
                if any(r[3 + i].lower().startswith("active") for r in rows):
                    out["reasons"].append(n)
            out["samples"] = len(rows)
        return out


# ------------------------------------------------------------------------------------------ configurations

def quantize_config(tokens: int, plain: bool, world: int) -> dict:
    return {"workload": f"{'reorder' if plain else 'fused rmsnorm+reorder'}+nvfp4+arc quantize, hidden {HIDDEN}, "
                        f"KE {KE}, {tokens} tokens per GPU", "tokens_per_gpu": tokens, "hidden": HIDDEN,
            "select_num": KE, "l2": "step touches 346 MB > 126 MB L2, no flush needed",
            "parallelism": f"tokens sharded x{world}"}


def layer_config(world: int) -> dict:
    return {"workload": f"llama-3-8b-shape decoder layer (hidden {HIDDEN}, 32/8 heads, FFN {FFN}, seven ARC-NVFP4 "
                        f"linears, select_num {KE}), prefill batch {LAYER_BATCH} x seq {LAYER_SEQ}",
            "global_batch": LAYER_BATCH, "seq_len": LAYER_SEQ, "tokens": LAYER_BATCH * LAYER_SEQ,
            "l2": "activations of one step (134 MB in, 470 MB of gate/up) exceed the 126 MB L2, no flush needed",
            "parallelism": f"tp{world}" + ("+sp (sequence-parallel residual stream)" if world > 1 else "")}


# ------------------------------------------------------------------------------------------ CPU arms

def _cpu_threads():
    import torch

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    return threads


def cpu_quantize(tokens_sample: int, steps: int, warmup: int):
    """Config 2 on the host: fp32 RMSNorm + gather + fake ARC-NVFP4 (model/quantize.py:314-343 restated)."""
    from arcquant_b200 import synth
    from oracle import fake_port as FP

    threads = _cpu_threads()
    out = synth.outlier_channels(HIDDEN, 41, 1)
    x = synth.activations(tokens_sample, HIDDEN, 2, out)
    gamma = synth.rms_gain(HIDDEN, 3)
    idx = synth.reorder_index_from_stats(x.abs().amax(0))
    for _ in range(warmup):
        FP.fake_quantize_activations(x, idx, KE, gamma, EPS)
    t0 = time.perf_counter()
    for _ in range(steps):
        FP.fake_quantize_activations(x, idx, KE, gamma, EPS)
    dt = (time.perf_counter() - t0) / steps
    return tokens_sample * BYTES_PER_TOKEN / dt / 1e9, dt, threads


def _fake_weight(n: int, kq: int, seed: int):
    """Stand-in for a fake-quantized weight [N, KQ+KE] (the reference prepares those once, offline; the
    timed forward only multiplies by them, so seeded values of the right shape and type time the same)."""
    from arcquant_b200 import synth
    return synth.weights(n, kq + KE, seed)


def _fake_linear_prequant(x, w_aug, idx):
    """One linear of the fake path with the weight prepared beforehand: gather, fake ARC-NVFP4 of the
    activation (model/quantize.py:314-343), bf16 F.linear over K + KE (model/qLinearLayer.py:71)."""
    import torch
    import torch.nn.functional as F

    from oracle import fake_port as FP

    qx, _ = FP.fake_reorder_quantize_x(torch.index_select(x, 1, idx.to(torch.int64)), KE)
    return F.linear(qx, w_aug)


def cpu_layer(tokens_sample: int, steps: int = 1):
    """Config 4 on the host, fake-quant path, on a sample of one sequence: seven linears, RoPE-free
    causal attention by torch SDPA (the attention itself is bf16 torch in the reference too)."""
    import torch
    import torch.nn.functional as F

    from arcquant_b200 import synth
    from oracle import fake_port as FP

    threads = _cpu_threads()
    g = torch.Generator().manual_seed(0)
    x = synth.activations(tokens_sample, HIDDEN, 7, synth.outlier_channels(HIDDEN, 41, 1))
    idx_h = torch.randperm(HIDDEN, generator=g)
    idx_f = torch.randperm(FFN, generator=g)
    wqkv, wo = _fake_weight(6144, HIDDEN, 1), _fake_weight(HIDDEN, HIDDEN, 2)
    wgu, wd = _fake_weight(2 * FFN, HIDDEN, 3), _fake_weight(HIDDEN, FFN, 4)
    gamma = synth.rms_gain(HIDDEN, 3)

    def step():
        n = FP.rmsnorm(x, gamma, EPS)
        qkv = _fake_linear_prequant(n, wqkv, idx_h)
        q = qkv[:, :4096].reshape(1, tokens_sample, 32, 128).transpose(1, 2)
        k = qkv[:, 4096:5120].reshape(1, tokens_sample, 8, 128).transpose(1, 2)
        v = qkv[:, 5120:].reshape(1, tokens_sample, 8, 128).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k.repeat_interleave(4, 1), v.repeat_interleave(4, 1), is_causal=True)
        h = x + _fake_linear_prequant(a.transpose(1, 2).reshape(tokens_sample, 4096), wo, idx_h)
        gu = _fake_linear_prequant(FP.rmsnorm(h, gamma, EPS), wgu, idx_h)
        act = F.silu(gu[:, :FFN]) * gu[:, FFN:]
        return h + _fake_linear_prequant(act, wd, idx_f)

    step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return tokens_sample / dt, dt, threads


def cpu_moe(tokens_sample: int):
    """Config 5 on the host: the reference's expert loop (model/qMixtralLayer.py:458-471) with fake-quant
    expert linears, 8 experts, top-2."""
    import torch
    import torch.nn.functional as F

    from arcquant_b200 import synth
    from arcquant_b200.moe_block import route_top_k

    threads = _cpu_threads()
    g = torch.Generator().manual_seed(0)
    x = synth.activations(tokens_sample, HIDDEN, 11, synth.outlier_channels(HIDDEN, 41, 1))
    router = (torch.randn(8, HIDDEN, generator=g) * 0.05).to(torch.bfloat16)
    idx_h, idx_f = torch.randperm(HIDDEN, generator=g), torch.randperm(FFN, generator=g)
    w13, w2 = _fake_weight(2 * FFN, HIDDEN, 5), _fake_weight(HIDDEN, FFN, 6)     # one expert's shapes, reused

    def step():
        ids, w = route_top_k(x, router, 2)
        out = torch.zeros_like(x)
        for e in range(8):
            tok, slot = torch.where(ids == e)
            if tok.numel() == 0:
                continue
            h = _fake_linear_prequant(x[tok], w13, idx_h)
            o = _fake_linear_prequant(F.silu(h[:, :FFN]) * h[:, FFN:], w2, idx_f)
            out.index_add_(0, tok, o * w[tok, slot][:, None])
        return out

    t0 = time.perf_counter()
    step()
    dt = time.perf_counter() - t0
    return tokens_sample / dt, dt, threads


def cpu_baselines():
    """The reference's CPU path for configs 1, 3, 4 and 5, each on a bounded sample."""
    import torch
    import torch.nn.functional as F

    from arcquant_b200 import synth
    from oracle import fake_port as FP

    threads = _cpu_threads()
    res = {}
    # config 1: one linear through the fake path, activation and weight quantization included
    x, w, idx, ke = synth.config1(0)
    t0 = time.perf_counter()
    FP.fake_linear(x, w, idx, ke)
    dt = time.perf_counter() - t0
    res["config1_single_linear"] = {"value": 2.0 * 512 * 4096 * 4224 / dt / 1e12, "unit": "TFLOP/s", "seconds": dt,
                                    "cores": threads, "kind": "port", "sample": "the whole configuration (X 512 x 4096, "
                                    "W 4096 x 4096, KE 128), quantization of X and W included, one run"}
    # config 3: dequantised bf16 F.linear over K + KE (what the fake path multiplies) at M 4096
    m = 4096
    pts = []
    for name, n, kq in GEMM_SHAPES:
        a = synth.activations(m, kq + KE, 1)
        b = _fake_weight(n, kq, 2)
        F.linear(a[:64], b)
        t0 = time.perf_counter()
        F.linear(a, b)
        dt = time.perf_counter() - t0
        pts.append({"shape": name, "M": m, "N": n, "K_eff": kq + KE, "tflops": 2.0 * m * n * (kq + KE) / dt / 1e12,
                    "seconds": dt})
    res["config3_dequantised_linear"] = {"points": pts, "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                         "sample": "M 4096 at each of the four shapes, bf16 torch F.linear over K + 128, one run each"}
    tps, dt, _ = cpu_layer(2048)
    res["config4_llama_layer"] = {"value": tps, "unit": "tokens/s", "seconds": dt, "cores": threads, "kind": "port",
                                  "sample": "one of the eight sequences (2048 of the 16384 tokens); weights prepared beforehand"}
    tps, dt, _ = cpu_moe(1024)
    res["config5_moe_block"] = {"value": tps, "unit": "tokens/s", "seconds": dt, "cores": threads, "kind": "port",
                                "sample": "1024 of the 4096 tokens; expert weights prepared beforehand"}
    return res


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 8))
    warm = 1
    if args.gpus <= 1:
        sample = 8192
        gbs, dt, threads = cpu_quantize(sample, steps, warm)
        line = {"impl": "reference", "metric": "arc_nvfp4_rmsnorm_quantize_bandwidth", "value": gbs, "unit": "GB/s",
                "scaling": "weak", "dtype": "bf16 in, fp32 arithmetic (torch CPU)",
                "config": quantize_config(TOKENS, False, 1),
                "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                 "sample": f"{sample} of {TOKENS} tokens per step; torch fake-quant path of the "
                                           "reference (model/quantize.py) restated in oracle/fake_port.py"}}
    else:
        sample = 2048
        steps = max(1, min(args.steps, 3))
        tps, dt, threads = cpu_layer(sample, steps)
        line = {"impl": "reference", "metric": "llama3_8b_shape_tp_layer_throughput", "value": tps, "unit": "tokens/s",
                "scaling": "strong", "dtype": "bf16 (torch CPU)", "config": layer_config(args.gpus),
                "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port",
                                 "sample": f"one of the eight sequences ({sample} of the 16384 tokens) per step; fake-quant layer "
                                           "(model/quantize.py + model/qLlamaLayer.py call order) on the host, one "
                                           "process: the reference has no multi-GPU or multi-process path"}}
    line.update({"n_gpus": args.gpus, "steps": steps, "warmup": warm, "steps_requested": args.steps,
                 "warmup_requested": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                 "vs_baseline": None, "data": "synthetic",
                 "e2e": {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                 "gpu_launches": 0})
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU helpers

def time_ms(fn, steps: int, warmup: int = 3) -> float:
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def max_over_ranks(ms: float, dev) -> float:
    import torch
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())
    return ms


def make_inputs(dev, tokens, seed):
    import torch

    from arcquant_b200 import synth

    out = synth.outlier_channels(HIDDEN, 41, 1)
    x = synth.activations(tokens, HIDDEN, seed, out, device=dev)
    gamma = synth.rms_gain(HIDDEN, 3).to(dev)
    # channel order from a calibration batch of the same distribution (8 x 2048 tokens here; the
    # order only decides which channels sit where, not how much work there is)
    stat = torch.zeros(HIDDEN, device=dev)
    for s in range(8):
        stat = torch.maximum(stat, synth.activations(2048, HIDDEN, 1000 + s, out, device=dev).abs().amax(0).float())
    idx = synth.reorder_index_from_stats(stat).to(dev)
    return x, gamma, idx


def random_gemm_operands(dev, m, n, k_eff, seed):
    import torch

    from arcquant_b200 import ops

    g = torch.Generator(device=dev).manual_seed(seed)
    a = torch.randint(0, 256, (m, k_eff // 2), dtype=torch.uint8, device=dev, generator=g)
    b = torch.randint(0, 256, (n, k_eff // 2), dtype=torch.uint8, device=dev, generator=g)
    # scales between 2^-3 and 2 (codes 0x20..0x40): finite, realistic magnitudes
    sfa = torch.randint(0x20, 0x41, (ops.sf_bytes(m, k_eff),), dtype=torch.uint8, device=dev, generator=g)
    sfb = torch.randint(0x20, 0x41, (ops.sf_bytes(n, k_eff),), dtype=torch.uint8, device=dev, generator=g)
    return a, b, sfa, sfb


def gemm_point(dev, m, n, kq, tf_peak, hbm_peak, reps=10, comparator=False):
    """One GEMM shape: TFLOP/s and the roofline that bounds it - the tensor pipe (4 x the measured bf16
    rate stands in for the dense NVFP4 peak, which is not among the measured peaks) or, for few rows,
    the bytes of the weight stream."""
    import torch

    from arcquant_b200 import ops

    k_eff = kq + KE
    a, b, sfa, sfb = random_gemm_operands(dev, m, n, k_eff, m + n)
    ms = time_ms(lambda: ops.matmul(a, b, sfa, sfb, 1.0), reps)
    flops = 2.0 * m * n * k_eff
    tf = flops / (ms * 1e-3) / 1e12
    t_tensor = flops / (4 * tf_peak * 1e12)
    nbytes = (m + n) * k_eff * 9 // 16 + 2 * m * n
    t_hbm = nbytes / (hbm_peak * 1e9)
    bound = "tensor" if t_tensor >= t_hbm else "hbm"
    pt = {"M": m, "N": n, "K_eff": k_eff, "ms": ms, "tflops": tf, "useful_tflops": 2.0 * m * n * kq / (ms * 1e-3) / 1e12,
          "bound": bound, "frac": max(t_tensor, t_hbm) / (ms * 1e-3),
          "frac_of_4x_measured_bf16": tf / (4 * tf_peak), "frac_of_nominal_fp4_9000": tf / 9000.0}
    if bound == "hbm":
        pt["gbs"] = nbytes / (ms * 1e-3) / 1e9
    if comparator:
        # third-party line: cuBLASLt's NVFP4 GEMM through torch._scaled_mm on views of the same operands
        try:
            a4, b4 = a.view(torch.float4_e2m1fn_x2), b.view(torch.float4_e2m1fn_x2)
            span = lambda rows: ((rows + 127) // 128) * 128 * (((k_eff // 16) + 3) // 4 * 4)
            sa, sb = sfa[:span(m)].view(torch.float8_e4m3fn), sfb[:span(n)].view(torch.float8_e4m3fn)
            lib = lambda: torch._scaled_mm(a4, b4.t(), sa, sb, out_dtype=torch.bfloat16)
            same = bool(torch.equal(lib(), ops.matmul(a, b, sfa, sfb, 1.0)))
            ms_lib = time_ms(lib, reps)
            pt["cublaslt_scaled_mm"] = {"ms": ms_lib, "tflops": flops / (ms_lib * 1e-3) / 1e12, "ours_over_lib": ms_lib / ms,
                                        "bit_identical_output": same, "role": "third-party comparator, not on any path"}
        except Exception as exc:
            pt["cublaslt_scaled_mm"] = {"unavailable": repr(exc)[:160]}
    return pt


def sweeps(dev, hbm_peak, tf_peak):
    """The kernel-alone grids: quantizer over tokens x residual width (fused RMSNorm, hidden 4096) and the
    GEMM over M x the four projection shapes."""
    import torch

    from arcquant_b200 import ops

    quant = []
    x, gamma, idx = make_inputs(dev, 32768, 5)
    for tokens in (1, 16, 128, 1024, 8192, 32768):
        xs = x[:tokens].contiguous()
        for ke in (0, 64, 128, 256):
            reps = 50 if tokens <= 1024 else 20
            ms = time_ms(lambda: ops.rmsnorm_quantize_x(xs, gamma, EPS, idx, ke), reps)
            nbytes = tokens * quant_bytes_per_token(HIDDEN, ke) + 4 * HIDDEN
            gbs = nbytes / (ms * 1e-3) / 1e9
            quant.append({"tokens": tokens, "select_num": ke, "us": ms * 1e3, "gbs": gbs, "frac": gbs / hbm_peak})
    del x
    gemm = []
    for name, n, kq in GEMM_SHAPES:
        for m in (1, 16, 128, 1024, 4096, 16384):
            pt = gemm_point(dev, m, n, kq, tf_peak, hbm_peak, reps=20 if m <= 1024 else 8)
            pt["shape"] = name
            gemm.append(pt)
    if ops.gemm_poll_error() != 0:
        gemm.append({"error": "a bounded device-side wait expired"})
    return {"quantize_fused_hidden4096": quant, "gemm": gemm,
            "note": "frac: achieved / bound, the bound being HBM bytes for the quantizer and for GEMMs with few rows "
                    "((M+N)*K_eff*9/16 + 2*M*N bytes), else 4 x the measured bf16 rate; few-token quantizer points "
                    "are latency-bound"}


def layer_roofline(world: int, hbm_peak: float, tf_peak: float, sp: bool):
    """Sum of the rooflines of one rank's share of the layer: GEMM flops at 4 x the measured bf16 rate,
    quantizer, max|x|, SiLU-output and rotary-embedding bytes at the measured HBM rate, attention flops at the bf16 rate, collective bytes
    at the measured NVLink rate."""
    T = LAYER_BATCH * LAYER_SEQ
    ke_r = KE if world == 1 else 64
    k1 = HIDDEN + KE
    flops = 2.0 * T * ((6144 // world) * k1 + HIDDEN * (4096 // world + ke_r) + (2 * FFN // world) * k1 +
                       HIDDEN * (FFN // world + ke_r))
    rows_q = T // world if sp else T
    nbytes = 2 * rows_q * quant_bytes_per_token(HIDDEN, KE)                       # two fused RMSNorm sites
    for kq in (4096 // world, FFN // world):                                       # o and down inputs
        nbytes += T * (quant_bytes_per_token(kq, ke_r))
    nbytes += T * 2 * (4096 // world)                                              # max|.| pass over the attention output
    nbytes += T * 2 * (FFN // world)                                               # SiLU * up: written by the GEMM's epilogue
    nbytes += T * 2 * (6144 // world) * 2                                          # rotary embedding in place
    attn_flops = 4.0 * LAYER_BATCH * LAYER_SEQ * LAYER_SEQ * (32 // world) * 128 * 0.5
    comm = 0.0
    if world > 1:
        f = (world - 1) / world
        comm = 2 * f * T * HIDDEN * 2                                              # two reduce-scatters (all-reduce: x2)
        comm = comm + 2 * f * T * (k1 * 9 // 16) if sp else 2 * comm
    t = {"gemm_ms": flops / (4 * tf_peak * 1e12) * 1e3, "hbm_ms": nbytes / (hbm_peak * 1e9) * 1e3,
         "attention_ms": attn_flops / (tf_peak * 1e12) * 1e3, "collective_ms": comm / (NVLINK_GBS * 1e9) * 1e3}
    t["sum_ms"] = sum(t.values())
    return t


NCCL_CTAS = int(os.environ.get("ARCQ_BENCH_NCCL_CTAS", "0"))       # CTAs NCCL may use per collective (0 = its own choice)
SM_RESERVE = int(os.environ.get("ARCQ_BENCH_SM_RESERVE", "0"))     # SMs the compute kernels leave to them


SP_CHUNKS = int(os.environ.get("ARCQ_BENCH_CHUNKS", "2"))          # runs of the pipelined sequence-parallel form


def init_nccl(dist, dev):
    """NCCL process group.  ARCQ_BENCH_NCCL_CTAS / ARCQ_BENCH_SM_RESERVE (tuning runs of the pipelined form):
    bound the CTAs of a collective and tell the compute kernels to leave that many SMs free
    (`ops.set_sm_limit`), so that a collective on NCCL's stream runs beside a persistent kernel."""
    opts = None
    if NCCL_CTAS > 0:
        try:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = NCCL_CTAS
            opts.config.min_ctas = min(NCCL_CTAS, 4)
        except Exception:
            opts = None
    import datetime

    # a collective that a peer never joins ends this run after three minutes, not after NCCL's default ten
    limit = datetime.timedelta(seconds=180)
    if opts is not None:
        dist.init_process_group("nccl", device_id=dev, pg_options=opts, timeout=limit)
    else:
        dist.init_process_group("nccl", device_id=dev, timeout=limit)
    if SM_RESERVE > 0:
        import torch

        from arcquant_b200 import ops
        ops.set_sm_limit(torch.cuda.get_device_properties(dev).multi_processor_count - SM_RESERVE)


def build_layer(dev, world, rank, group=None):
    from arcquant_b200.llama_layer import (LlamaLayerConfig, QLlamaDecoderLayerTP, random_layer_weights,
                                           random_reorder_indices)

    cfg = LlamaLayerConfig()
    return cfg, QLlamaDecoderLayerTP(cfg, random_layer_weights(cfg, 0), random_reorder_indices(cfg, 1), tp_rank=rank,
                                     tp_size=world, group=group, device=dev)


def layer_measure(dev, world, rank, steps, hbm_peak, tf_peak, use_peer=True):
    """The decoder layer: eager and CUDA-graph time of the default form (one GPU: `forward`; several: the
    sequence-parallel form on this rank's token shard), the all-reduce form beside it, the per-phase
    breakdown of an eager step, and the end-to-end leg with pinned host buffers."""
    import torch

    from arcquant_b200 import synth
    from arcquant_b200.graphs import GraphedStep
    from arcquant_b200.llama_layer import PhaseTimer

    cfg, layer = build_layer(dev, world, rank)
    T = LAYER_BATCH * LAYER_SEQ
    x = synth.activations(T, cfg.hidden, 7, synth.outlier_channels(cfg.hidden, 41, 1), device=dev)
    pos = torch.arange(LAYER_SEQ, device=dev)
    x3 = x.reshape(LAYER_BATCH, LAYER_SEQ, cfg.hidden)
    rows = T // world
    sp = world > 1
    xs = x[rank * rows:(rank + 1) * rows].clone() if sp else None      # this rank's run of tokens (static graph input)
    step = (lambda: layer.forward_sequence_parallel(xs, LAYER_BATCH, LAYER_SEQ, pos)) if sp else (lambda: layer(x3, pos))
    res = {"tokens": T, "parallelism": f"tp{world}" + ("+sp" if sp else ""), "scaling": "strong"}
    if sp:
        res["form"] = ("sequence-parallel: residual stream sharded by tokens, RMSNorm + quantize on the shard, all-gather "
                       "of packed codes and block scales, reduce-scatter after the row-parallel GEMMs")
    if sp:
        # first with NCCL's reduce-scatter behind the row-parallel GEMMs, then - the form reported - with the GEMMs'
        # epilogues storing into the owners' memory (falls back to the NCCL form, and says so, if the peers'
        # memory cannot be mapped)
        ms_e = max_over_ranks(time_ms(step, steps), dev)
        g_nccl = GraphedStep(step)
        ms_g = max_over_ranks(time_ms(g_nccl, steps), dev)
        res["nccl_reduce_scatter_form"] = {"eager_ms": ms_e, "ms": ms_g, "tokens_per_s": T / (ms_g * 1e-3)}
        del g_nccl
        try:
            if not use_peer:
                raise RuntimeError("peer-memory form failed its parity check on the small configuration")
            layer.enable_peer_scatter(T)
            res["form"] += ("; no NCCL call in the step: the row-parallel GEMMs store their tiles straight into the owning "
                            "rank's memory over NVLink (arcq_matmul_nvfp4_scatter) and the reduce-scatter ends with one local "
                            "pass that also adds the residual (arcq_sum_partials_bf16); the RMSNorm quantizers store their rows "
                            "into every rank's gathered buffers (arcq_rmsnorm_quantize_x_multi); four barriers through flags "
                            "in peer memory (arcq_peer_barrier)")
        except Exception as exc:
            res["peer_scatter_error"] = repr(exc)[:300]
    res["eager_ms"] = max_over_ranks(time_ms(step, steps), dev)
    graphed = GraphedStep(step)
    res["ms"] = max_over_ranks(time_ms(graphed, steps), dev)
    if sp and layer.peer_barrier is not None:
        from arcquant_b200 import ops
        bad = max_over_ranks(float(ops.peer_poll_error() != 0), dev)
        if bad:         # a barrier ran out of time on some rank: these numbers mean nothing, report the NCCL form
            res["peer_scatter_error"] = "a peer barrier timed out during the timed steps"
            del graphed
            layer.disable_peer_scatter()
            res["form"] = res["form"].split("; no NCCL call")[0]
            res["eager_ms"] = max_over_ranks(time_ms(step, steps), dev)
            graphed = GraphedStep(step)
            res["ms"] = max_over_ranks(time_ms(graphed, steps), dev)
    res["tokens_per_s"] = T / (res["ms"] * 1e-3)
    res["launch"] = "one CUDA graph per step (captured once; collectives inside)"
    # per-phase device time of an eager step (phases run one after another on one stream)
    from arcquant_b200 import _lib as _abi
    calls0 = _abi.CALLS
    layer.timer = PhaseTimer()
    step()
    res["library_calls_per_step"] = _abi.CALLS - calls0      # launching C-ABI calls of one step (each one to three kernels)
    layer.timer.totals()
    for _ in range(3):
        step()
    tot = layer.timer.totals()
    layer.timer = None
    res["eager_phase_ms"] = {k: v / 3 for k, v in tot.items()}
    if sp:
        ph = res["eager_phase_ms"]
        if layer.peer_o is not None:
            res["limiter"] = ("NVLink: each rank's o and down GEMMs send (N-1)/N of their bf16 result [16384, 4096] (134 MB) "
                              "to the owners while they run (their time is in the gemm phase: %.2f ms); collective = the four "
                              "barriers (waiting for the slowest rank included): %.2f ms of the %.2f ms eager step" %
                              (ph.get("gemm", 0.0), ph.get("collective", 0.0), sum(ph.values())))
        else:
            res["limiter"] = ("collectives: two reduce-scatters of the bf16 partial sums [16384, 4096] (134 MB each) and two "
                              "all-gathers of packed codes (39 MB each), %.2f ms of the %.2f ms eager step, not overlapped "
                              "with compute (the per-tensor scales of the o and down inputs order the phases)" %
                              (ph.get("collective", 0.0), sum(ph.values())))
        ms_ar = max_over_ranks(time_ms(lambda: layer(x3, pos), max(3, steps // 2)), dev)
        res["all_reduce_form"] = {"eager_ms": ms_ar, "tokens_per_s": T / (ms_ar * 1e-3)}
        if SP_CHUNKS > 1 and LAYER_BATCH % SP_CHUNKS == 0 and (T // SP_CHUNKS // world) % 128 == 0:
            # the pipelined form (runs of whole sequences, asynchronous collectives under the neighbours' compute)
            own = layer.pipelined_shard_rows(T, world, rank, SP_CHUNKS).to(dev)
            xp = x[own].contiguous()
            ms_pp = max_over_ranks(time_ms(lambda: layer.forward_sequence_parallel_pipelined(
                xp, LAYER_BATCH, LAYER_SEQ, pos, SP_CHUNKS), max(3, steps // 2)), dev)
            res["pipelined_form"] = {"runs": SP_CHUNKS, "eager_ms": ms_pp, "tokens_per_s": T / (ms_pp * 1e-3)}
    rf = layer_roofline(world, hbm_peak, tf_peak, sp)
    res["roofline"] = dict(rf, frac=rf["sum_ms"] / res["ms"], bound="sum of the rooflines of the phases (tensor, hbm, "
                           "nvlink)", achieved_ms=res["ms"])
    # end to end: this rank's rows from pinned host memory, the step, its rows of the result back
    if sp:
        hin = torch.empty((rows, cfg.hidden), dtype=torch.bfloat16).pin_memory()
        hin.copy_(xs.cpu())
        hout = torch.empty_like(hin).pin_memory()
        xin = xs
    else:
        hin = torch.empty((T, cfg.hidden), dtype=torch.bfloat16).pin_memory()
        hin.copy_(x.cpu())
        hout = torch.empty_like(hin).pin_memory()
        xin = x

    def e2e_step():
        xin.copy_(hin, non_blocking=True)
        y = graphed()
        hout.copy_(y.reshape(hout.shape), non_blocking=True)

    e2e_ms = max_over_ranks(time_ms(e2e_step, max(3, steps // 2)), dev)
    res["e2e"] = {"value": T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                  "h2d_bytes_per_step": int(hin.numel() * 2) * world, "d2h_bytes_per_step": int(hout.numel() * 2) * world}
    return res


def tp1_reference(dev, steps):
    """The unsharded decoder layer on this GPU alone (no collectives, nothing that involves other ranks)."""
    import torch

    from arcquant_b200 import synth
    from arcquant_b200.graphs import GraphedStep

    cfg, layer = build_layer(dev, 1, 0)
    T = LAYER_BATCH * LAYER_SEQ
    x3 = synth.activations(T, cfg.hidden, 7, synth.outlier_channels(cfg.hidden, 41, 1), device=dev).reshape(
        LAYER_BATCH, LAYER_SEQ, cfg.hidden)
    pos = torch.arange(LAYER_SEQ, device=dev)
    graphed = GraphedStep(lambda: layer(x3, pos))
    ms = time_ms(graphed, steps)
    return {"ms": ms, "tokens_per_s": T / (ms * 1e-3), "parallelism": "tp1", "tokens": T,
            "note": "rank 0 alone while the other ranks wait; same shapes, same CUDA-graph launch"}


def moe_roofline(world: int, hbm_peak: float, tf_peak: float):
    R = MOE_TOKENS * 2 // world                                                   # routed copies per rank
    k1 = HIDDEN + KE
    flops = 2.0 * R * (2 * FFN * k1 + HIDDEN * (FFN + KE))
    # (max|x| pass and quantizer over the routed rows; SiLU * up written by the GEMM's epilogue; its quantizer)
    nbytes = R * (2 * HIDDEN + quant_bytes_per_token(HIDDEN, KE)) + R * 2 * FFN + R * quant_bytes_per_token(FFN, KE)
    nbytes += (8 // world) * (2 * FFN * k1 + HIDDEN * (FFN + KE)) * 9 // 16        # every local expert's weights once
    comm = 0.0 if world == 1 else 2 * (world - 1) / world * R * HIDDEN * 2
    t = {"gemm_ms": flops / (4 * tf_peak * 1e12) * 1e3, "hbm_ms": nbytes / (hbm_peak * 1e9) * 1e3,
         "collective_ms": comm / (NVLINK_GBS * 1e9) * 1e3}
    t["sum_ms"] = sum(t.values())
    return t


def moe_measure(dev, world, rank, steps, hbm_peak, tf_peak, use_peer=True):
    """Mixtral-8x7B-shape sparse MoE block (hidden 4096, FFN 14336, 8 experts, top-2, ARC-NVFP4 expert
    linears, select_num 128), expert-parallel over `world` ranks; 4096 tokens in total."""
    from arcquant_b200 import synth
    from arcquant_b200.graphs import GraphedStep
    from arcquant_b200.moe_block import MoEConfig, QMixtralMoEBlockEP, random_moe_weights

    cfg = MoEConfig()
    # blocks of twice the even share travel between ranks (the worst case - every copy of a rank to one peer -
    # would move `world` times the even share); an overflow would be flagged and fails the measurement
    block = QMixtralMoEBlockEP(cfg, random_moe_weights(cfg, 0), ep_rank=rank, ep_size=world, device=dev,
                               capacity_factor=2.0 if world > 1 else None)
    x = synth.activations(MOE_TOKENS, cfg.hidden, 11, synth.outlier_channels(cfg.hidden, 41, 1), device=dev)
    lo, hi = rank * MOE_TOKENS // world, (rank + 1) * MOE_TOKENS // world
    xs = x[lo:hi].contiguous()
    step = lambda: block(xs)
    res = {"tokens": MOE_TOKENS, "parallelism": f"ep{world}", "scaling": "strong",
           "organisation": "one grouped launch per projection over all local experts; dispatch layout computed on "
                           "the device" if block.grouped else "per-expert loop"}
    if world > 1:
        # first over NCCL's all-to-all, then - the form reported - with the rows stored into the peers' memory
        ms_e = max_over_ranks(time_ms(step, steps), dev)
        g_nccl = GraphedStep(step)
        ms_g = max_over_ranks(time_ms(g_nccl, steps), dev)
        res["nccl_all_to_all_form"] = {"eager_ms": ms_e, "ms": ms_g, "tokens_per_s": MOE_TOKENS / (ms_g * 1e-3)}
        del g_nccl
        if block.dispatcher.overflowed():
            raise RuntimeError("expert-parallel dispatch dropped copies: capacity factor too small for this routing")
        try:
            if not use_peer:
                raise RuntimeError("peer-memory dispatch failed its parity check on the small configuration")
            block.enable_peer_dispatch(hi - lo, 2.0)
            res["organisation"] += ("; rows travel to the experts' ranks and back as stores into peer memory "
                                    "(arcq_ep_send_layout, arcq_ep_rows, arcq_peer_barrier), no collective in the step")
        except Exception as exc:
            res["peer_dispatch_error"] = repr(exc)[:300]
    res["eager_ms"] = max_over_ranks(time_ms(step, steps), dev)
    try:
        graphed = GraphedStep(step)
        res["ms"] = max_over_ranks(time_ms(graphed, steps), dev)
        res["launch"] = "one CUDA graph per step"
    except Exception as exc:
        res["ms"] = res["eager_ms"]
        res["graph_error"] = repr(exc)[:160]
    if world > 1 and "peer_dispatch_error" not in res:
        from arcquant_b200 import ops
        if max_over_ranks(float(ops.peer_poll_error() != 0), dev):
            res["peer_dispatch_error"] = "a peer barrier timed out during the timed steps"
            block.disable_peer_dispatch()
            res["organisation"] = res["organisation"].split("; rows travel")[0]
            res["eager_ms"], res["ms"] = res["nccl_all_to_all_form"]["eager_ms"], res["nccl_all_to_all_form"]["ms"]
    res["tokens_per_s"] = MOE_TOKENS / (res["ms"] * 1e-3)
    if block.dispatcher.overflowed():
        raise RuntimeError("expert-parallel dispatch dropped copies: capacity factor too small for this routing")
    if world > 1:
        res["dispatch"] = f"blocks of {block.dispatcher.capacity} rows per peer (2 x the even share)"
    rf = moe_roofline(world, hbm_peak, tf_peak)
    res["roofline"] = dict(rf, frac=rf["sum_ms"] / res["ms"], achieved_ms=res["ms"])
    return res


def multi_gpu_parity(dev, world, rank):
    """Small-configuration layer and MoE block through NCCL against the same shards added up inside this
    process (tensor-parallel: all-reduce form and sequence-parallel form; expert-parallel: against one
    rank owning every expert).  Relative Frobenius errors; raises above 1e-2."""
    import torch

    from arcquant_b200 import synth
    from arcquant_b200.llama_layer import (LlamaLayerConfig, QLlamaDecoderLayerTP, random_layer_weights,
                                           random_reorder_indices)
    from arcquant_b200.moe_block import MoEConfig, QMixtralMoEBlockEP, random_moe_weights, route_top_k

    cfg = LlamaLayerConfig(hidden=1024, n_heads=8, n_kv_heads=8, head_dim=128, ffn=4096, select_num=64)
    W, I = random_layer_weights(cfg, 0), random_reorder_indices(cfg, 1)
    B, S = 4, 1024
    T = B * S
    x = synth.activations(T, cfg.hidden, 4, synth.outlier_channels(cfg.hidden, 10, 3), device=dev).reshape(B, S, -1)
    pos = torch.arange(S, device=dev)
    mine = QLlamaDecoderLayerTP(cfg, W, I, tp_rank=rank, tp_size=world, device=dev)
    mine.overlap_rows = 1 << 30                           # the plain all-reduce schedule
    y = mine(x, pos)
    ranks = [mine if r == rank else QLlamaDecoderLayerTP(cfg, W, I, tp_rank=r, tp_size=world, device=dev) for r in range(world)]
    x2 = x.reshape(T, -1)
    h = x2 + sum(r.attn_partial(x2, B, S, pos).float() for r in ranks).to(torch.bfloat16)
    ref = h + sum(r.mlp_partial(h).float() for r in ranks).to(torch.bfloat16)
    rel = lambda a, b: float((a.float() - b.float()).norm() / b.float().norm())
    out = {"tp": rel(y.reshape(T, -1), ref)}
    rows = T // world
    y_sp = mine.forward_sequence_parallel(x2[rank * rows:(rank + 1) * rows].contiguous(), B, S, pos)
    own = mine.pipelined_shard_rows(T, world, rank, 4).to(dev)
    y_pp = mine.forward_sequence_parallel_pipelined(x2[own].contiguous(), B, S, pos, 4)
    out["sp"] = max(rel(y_sp, ref[rank * rows:(rank + 1) * rows]), rel(y_pp, ref[own]))
    from arcquant_b200 import ops
    import torch.distributed as dist

    # the peer-memory forms are judged by themselves: a failure (memory that cannot be mapped, a barrier that
    # timed out, a wrong result) switches them off for the timed part instead of ending the run
    out["sp_peer"] = float("inf")
    try:
        mine.enable_peer_scatter(T)
        y_ps = mine.forward_sequence_parallel(x2[rank * rows:(rank + 1) * rows].contiguous(), B, S, pos)
        torch.cuda.synchronize()
        if ops.peer_poll_error() == 0:
            out["sp_peer"] = rel(y_ps, ref[rank * rows:(rank + 1) * rows])
    except RuntimeError as exc:
        if "peer memory unavailable" not in str(exc):
            raise
    dist.barrier()
    mine.disable_peer_scatter()
    del ranks
    mcfg = MoEConfig(hidden=1024, ffn=2048, n_experts=8, top_k=2, select_num=64)
    MW = random_moe_weights(mcfg, 0)
    xt = synth.activations(1024, mcfg.hidden, 5, synth.outlier_channels(mcfg.hidden, 10, 3), device=dev)
    ids, w = route_top_k(xt, MW["router"].to(dev), mcfg.top_k)
    full = QMixtralMoEBlockEP(mcfg, MW, device=dev)(xt, routing=(ids, w))
    lo, hi = rank * 1024 // world, (rank + 1) * 1024 // world
    part = QMixtralMoEBlockEP(mcfg, MW, ep_rank=rank, ep_size=world, device=dev)(
        xt[lo:hi].contiguous(), routing=(ids[lo:hi].contiguous(), w[lo:hi].contiguous()))
    out["ep"] = rel(part, full[lo:hi])
    peer_block = QMixtralMoEBlockEP(mcfg, MW, ep_rank=rank, ep_size=world, device=dev)
    out["ep_peer"] = float("inf")
    try:
        peer_block.enable_peer_dispatch(hi - lo, None)
        part = peer_block(xt[lo:hi].contiguous(), routing=(ids[lo:hi].contiguous(), w[lo:hi].contiguous()))
        torch.cuda.synchronize()
        if ops.peer_poll_error() == 0:
            out["ep_peer"] = rel(part, full[lo:hi])
    except RuntimeError as exc:
        if "peer memory unavailable" not in str(exc):
            raise
    dist.barrier()
    peer_block.disable_peer_dispatch()
    keys = ("tp", "sp", "ep", "sp_peer", "ep_peer")
    worst = torch.tensor([min(out[k], 1e30) for k in keys], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    out = {k: float(v) for k, v in zip(keys, worst.tolist())}
    if max(out["tp"], out["sp"], out["ep"]) > 1e-2:
        raise RuntimeError(f"multi-GPU parity failed: {out}")
    for k in ("sp_peer", "ep_peer"):           # (None: that form is not used in this run)
        if out[k] > 1e-2:
            out[k] = None
    return out


# ------------------------------------------------------------------------------------------ single workloads

def run_side_workload(args):
    """--workload gemm / layer / moe / sweep: one JSON line for that workload alone (profiling and tuning)."""
    import torch

    from arcquant_b200 import ops

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    if world > 1:
        import torch.distributed as dist
        init_nccl(dist, dev)
    if args.workload in ("layer", "moe"):
        fn = layer_measure if args.workload == "layer" else moe_measure
        res = fn(dev, world, rank, args.steps, hbm_peak, tf_peak)
        if world > 1:
            dist.destroy_process_group()
        if rank == 0:
            metric = "llama3_8b_shape_tp_layer_throughput" if args.workload == "layer" else "mixtral_shape_moe_block_throughput"
            print(json.dumps({"metric": metric, "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
                              "steps": args.steps, "ms_per_step": res["ms"], "scaling": "strong", "detail": res}), flush=True)
        return
    if args.workload == "sweep":
        print(json.dumps({"metric": "kernel_alone_grids", "sweep": sweeps(dev, hbm_peak, tf_peak)}), flush=True)
        return
    m, n, kq = (int(v) for v in args.shape.split(","))
    k_eff = kq + KE
    a, b, sfa, sfb = random_gemm_operands(dev, m, n, k_eff, m + n)
    for _ in range(max(args.warmup, 3)):
        c = ops.matmul(a, b, sfa, sfb, 1.0)
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    if args.steps >= 50:      # long enough for nvidia-smi to sample the clocks under this load
        sampler.start()
        time.sleep(0.25)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        c = ops.matmul(a, b, sfa, sfb, 1.0)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop() if args.steps >= 50 else None
    ms = e0.elapsed_time(e1) / args.steps
    tf = 2.0 * m * n * k_eff / (ms * 1e-3) / 1e12
    err = ops.gemm_poll_error()
    line = {"metric": "arc_nvfp4_gemm_throughput", "value": tf, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "ms_per_step": ms, "device_wait_error": err, "clocks": clocks,
            "config": {"workload": f"block-scaled NVFP4 GEMM M {m} N {n} K_eff {k_eff}"},
            "roofline": {"bound": "tensor", "achieved": tf, "peak": 4 * tf_peak, "unit": "TFLOP/s",
                         "frac": tf / (4 * tf_peak), "peak_kind": f"4 x {peak_kind} bf16 cuBLAS peak",
                         "frac_of_nominal_9000": tf / 9000.0},
            "gpu_launches": args.steps}
    if not args.lean:
        line["comparator"] = gemm_point(dev, m, n, kq, tf_peak, hbm_peak, comparator=True).get("cublaslt_scaled_mm")
    if rank == 0:
        print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ the default run

def quantizer_measure(args, dev, world, rank, local, dist, hbm_peak, peak_kind):
    """The kernel-alone quantizer workload: device-resident timing, roofline, clocks, and (unless --lean)
    the end-to-end leg with pinned host buffers."""
    import torch

    from arcquant_b200 import ops

    sys.path.insert(0, os.path.join(ROOT, "arcquant_b200"))
    import agemm

    tokens = args.tokens
    plain = args.workload == "quantize_plain"
    x, gamma, idx = make_inputs(dev, tokens, seed=2 + rank)

    def step():
        if plain:
            return ops.reorder_quantize_x(x, idx, KE)
        return ops.rmsnorm_quantize_x(x, gamma, EPS, idx, KE)

    for _ in range(max(args.warmup, 3)):
        q, sf = step()
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # keep the device busy long enough for the clock sampler to see it under load
    t_end = time.time() + (0.0 if args.lean else 0.6)
    while time.time() < t_end:
        for _ in range(20):
            step()
        torch.cuda.synchronize()

    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        q, sf = step()
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1), dev) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    value = world * tokens * BYTES_PER_TOKEN / (ms_step * 1e-3) / 1e9
    # Average launch duration of the dominant kernel: every step of the timed region is exactly one
    # launch of it, issued back to back on the current stream, so the region's CUDA-event time divided
    # by the launches is the per-launch duration (any gap between launches only makes it larger).
    algo_bytes = tokens * BYTES_PER_TOKEN + (2 if plain else 4) * HIDDEN
    achieved = algo_bytes / (ms_step * 1e-3) / 1e9
    res = {"metric": "arc_nvfp4_rmsnorm_quantize_bandwidth" if not plain else "arc_nvfp4_reorder_quantize_bandwidth",
           "value": value, "unit": "GB/s", "ms_per_step": ms_step, "clocks": clocks,
           "config": quantize_config(tokens, plain, world),
           "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                        "traffic": TRAFFIC_PER_TOKEN_NCU * tokens,
                        "traffic_source": "ncu capture of a 16384-token launch (profiles/), scaled by tokens",
                        "peak_kind": peak_kind,
                        "kernel": "arcq_quantize_ws_kernel<RMS>" if not plain else "arcq_quantize_ws_kernel<plain>",
                        "launch_ms": ms_step, "algorithmic_bytes_per_launch": algo_bytes}}
    if args.lean:
        return res
    # end to end through the reference-facing operator with host buffers: uploads, kernels and downloads of
    # 4096-token chunks overlap on three streams; every byte still crosses PCIe inside the timed region
    hx = torch.empty((tokens, HIDDEN), dtype=torch.bfloat16).pin_memory()
    hx.copy_(x.cpu())
    hq = torch.empty(q.shape, dtype=torch.uint8).pin_memory()
    hsf = torch.empty(sf.shape, dtype=torch.uint8).pin_memory()
    from arcquant_b200.host_pipeline import HostQuantizePipeline
    pipe = HostQuantizePipeline(tokens, HIDDEN, KE, dev, chunk_rows=4096)

    def e2e_step():
        pipe.run(hx, idx, hq, hsf, gamma=None if plain else gamma, eps=EPS)

    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(2):
        e2e_step()
    # the pipelined result must be what the reference-facing operator returns for the whole batch
    a_ref, s_ref = agemm.reorder_quantize_x(x, idx, KE) if plain else agemm.rmsnorm_quantize_x(x, gamma, EPS, idx, KE)
    nvalid = ((tokens + 127) // 128) * (((HIDDEN + KE) // 16 + 3) // 4) * 512
    sf_same = tokens % 128 != 0 or torch.equal(hsf[:nvalid], s_ref.cpu()[:nvalid])   # (unwritten rows of a ragged tile differ)
    if not (torch.equal(hq, a_ref.cpu()) and sf_same):
        raise RuntimeError("host pipeline and agemm operator disagree")
    del a_ref, s_ref
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = max_over_ranks(e2e_s, dev)
    res["e2e"] = {"value": world * tokens * BYTES_PER_TOKEN / e2e_s / 1e9, "unit": "GB/s",
                  "h2d_bytes_per_step": int(hx.numel() * 2), "d2h_bytes_per_step": int(hq.numel() + hsf.numel()),
                  "ms_per_step": e2e_s * 1e3}
    return res


def run_ours(args):
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        init_nccl(dist, dev)
    hbm_peak, tf_peak, peak_kind = measured_peaks()
    warm = max(args.warmup, 3)

    if args.lean or world == 1:
        qres = quantizer_measure(args, dev, world, rank, local, dist, hbm_peak, peak_kind)
        if args.lean:
            if dist is not None:
                dist.barrier()
                dist.destroy_process_group()
            if rank == 0:
                print(json.dumps({"metric": "arc_nvfp4_quantize_bandwidth", "value": qres["value"], "unit": "GB/s",
                                  "n_gpus": world, "steps": args.steps, "ms_per_step": qres["ms_per_step"], "lean": True,
                                  "config": {"workload": args.workload, "tokens_per_gpu": args.tokens},
                                  "roofline": qres["roofline"], "gpu_launches": args.steps}), flush=True)
            return
        extra = {}
        for name, fn in (("llama_layer", lambda: layer_measure(dev, 1, 0, 10, hbm_peak, tf_peak)),
                         ("moe_block", lambda: moe_measure(dev, 1, 0, 10, hbm_peak, tf_peak)),
                         ("gemm", lambda: [dict(gemm_point(dev, m, n, kq, tf_peak, hbm_peak, comparator=True), shape=nm)
                                           for nm, m, n, kq in (("qkv", 4096, 6144, 4096), ("gate_up", 16384, 28672, 4096),
                                                                ("down", 16384, 4096, 14336))]),
                         ("sweep", lambda: sweeps(dev, hbm_peak, tf_peak)),
                         ("cpu_baselines", cpu_baselines)):
            try:
                extra[name] = fn()
            except Exception as exc:       # the headline must survive a failure of a side measurement - visibly
                extra[name + "_error"] = repr(exc)[:300]
        gbs, dt, threads = cpu_quantize(8192, 5, 1)
        cpu = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
               "sample": "8192 of 32768 tokens per step, 5 steps; reference fake-quant path restated in "
                         "oracle/fake_port.py"}
        line = {"metric": qres["metric"], "value": qres["value"], "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                "warmup": warm, "ms_per_step": qres["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16 in, e2m1 + ue4m3 out, fp32 arithmetic", "data": "synthetic",
                "config": qres["config"], "roofline": qres["roofline"], "cpu_baseline": cpu, "e2e": qres["e2e"],
                "gpu_launches": args.steps, "clocks": qres["clocks"], "extra": extra}
        print(json.dumps(line), flush=True)
        return

    # ---- several GPUs: the tensor-parallel decoder layer is the headline
    parity = multi_gpu_parity(dev, world, rank)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    lres = layer_measure(dev, world, rank, max(args.steps, 10), hbm_peak, tf_peak, use_peer=parity["sp_peer"] is not None)
    clocks = sampler.stop() if rank == 0 else None
    extra = {"parity": parity, "llama_layer": lres}
    if rank == 0:
        # the same layer unsharded on rank 0 alone, the other ranks idle: the one-GPU point of the same quantity
        try:
            extra["tp1_same_run"] = tp1_reference(dev, 10)
        except Exception as exc:
            extra["tp1_same_run_error"] = repr(exc)[:300]
    dist.barrier()
    try:
        extra["moe_block"] = moe_measure(dev, world, rank, 10, hbm_peak, tf_peak, use_peer=parity["ep_peer"] is not None)
    except Exception as exc:
        extra["moe_block_error"] = repr(exc)[:300]
    try:
        largs = argparse.Namespace(**vars(args))
        largs.lean = True
        qres = quantizer_measure(largs, dev, world, rank, local, dist, hbm_peak, peak_kind)
        extra["quantizer_tokens_sharded"] = {"value": qres["value"], "unit": "GB/s", "ms_per_step": qres["ms_per_step"],
                                             "scaling": "weak", "roofline_frac_per_gpu": qres["roofline"]["frac"]}
    except Exception as exc:
        extra["quantizer_error"] = repr(exc)[:300]
    dist.barrier()
    dist.destroy_process_group()
    if rank != 0:
        return
    rf = lres["roofline"]
    line = {"metric": "llama3_8b_shape_tp_layer_throughput", "value": lres["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": world, "steps": max(args.steps, 10), "warmup": warm, "ms_per_step": lres["ms"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "nvfp4 linears (fp32 accumulation), bf16 activations and attention", "data": "synthetic",
            "config": layer_config(world),
            "roofline": {"bound": "sum of phase rooflines: tensor (4 x measured bf16) + hbm + nvlink", "achieved": lres["ms"],
                         "peak": rf["sum_ms"], "unit": "ms per step (lower is better)", "frac": rf["frac"], "traffic": None,
                         "parts_ms": {k: rf[k] for k in ("gemm_ms", "hbm_ms", "attention_ms", "collective_ms")}},
            "cpu_baseline": None, "e2e": lres["e2e"],
            # one CUDA-graph launch per step, holding the step's kernels: counted as the library's launching calls
            "gpu_launches": max(args.steps, 10) * max(1, lres.get("library_calls_per_step", 1)),
            "gpu_launches_note": "graph replays x launching calls into libarcq.so per step (each one to three kernels)",
            "clocks": clocks, "extra": extra}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="quantize",
                    choices=["quantize", "quantize_plain", "gemm", "layer", "moe", "sweep"],
                    help="quantize (default, the headline on one GPU): fused RMSNorm+reorder+NVFP4+ARC; quantize_plain: "
                         "without RMSNorm; gemm: one block-scaled GEMM shape; layer: Llama-3-8B-shape decoder layer; "
                         "moe: Mixtral-shape MoE block; sweep: the token x KE and M x shape grids")
    ap.add_argument("--tokens", type=int, default=TOKENS, help="tokens per GPU for the quantize workloads")
    ap.add_argument("--shape", default="4096,6144,4096", help="M,N,KQ of --workload gemm (K_eff = KQ+128)")
    ap.add_argument("--lean", action="store_true",
                    help="only the timed kernel loop: no e2e arm, no CPU baseline, no side measurements "
                         "(what the ncu captures under profiles/ run)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("gemm", "layer", "moe", "sweep"):
        run_side_workload(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Benchmark of the FP4 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" = one pass of the fused RMSNorm + NVFP4 quantisation (row-wise and column-wise
packed E2M1 operands, E4M3 block scales, FP32 tensor scale, round-to-nearest) over one
synthetic activation batch X bf16 [16384 x 4096] ~N(0,1) with 0.1 % of the channels x20 and
gamma = 1 + 0.1 N(0,1), eps 1e-5.  With N > 1 (torchrun, one rank per GPU) every rank runs
the same per-rank batch on its own GPU (the token dimension is what is sharded; weak
scaling, no collective on this path).  Rank 0 prints ONE JSON line.

`value` counts ALGORITHMIC bytes (every input read once, every output written once:
3.125 B per element + gamma + inv_rms) per second; the producer itself reads X twice.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M_ROWS, K_COLS = 16384, 4096
EPS = 1e-5
METRIC = "fused RMSNorm+NVFP4 quant algorithmic HBM throughput"
UNIT = "GB/s"
WORKLOAD = "config2: fused RMSNorm + NVFP4 quant, X bf16 [16384x4096], row+col operands, RTN"


def algorithmic_bytes(M, K):
    return M * K * 3.125 + 2 * K + 4 * M + 8


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


def make_inputs(seed=20261125):
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M_ROWS, K_COLS, generator=g)
    cols = torch.randperm(K_COLS, generator=g)[: max(1, round(K_COLS * 0.001))]
    x[:, cols] *= 20.0
    gamma = 1.0 + 0.1 * torch.randn(K_COLS, generator=g)
    return x.to(torch.bfloat16), gamma.to(torch.bfloat16)


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [s.strip() for s in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); smax.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # samples taken under load are the upper half of the observed clocks
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline_run(x_bf16, gamma_bf16, target_seconds=12.0, max_reps=20):
    """Times the C restatement (oracle/) on the host cores on the bench workload."""
    import numpy as np
    from oracle import c_oracle
    xb = x_bf16.view(__import__("torch").int16).numpy().view(np.uint16)
    gb = gamma_bf16.view(__import__("torch").int16).numpy().view(np.uint16)
    rows = M_ROWS
    t0 = time.perf_counter()
    c_oracle.fused_norm_quantize(xb[:2048], gb, EPS)  # warm-up + speed probe on 1/8 of the rows
    probe = time.perf_counter() - t0
    est_full = probe * (M_ROWS / 2048)
    if est_full > target_seconds:  # slow host: shrink the sample
        rows = max(128, int(M_ROWS * target_seconds / est_full) // 128 * 128)
    reps = max(1, min(max_reps, int(target_seconds / max(est_full * rows / M_ROWS, 1e-3))))
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        c_oracle.fused_norm_quantize(xb[:rows], gb, EPS)
        times.append(time.perf_counter() - t0)
    best = statistics.median(times)
    return {"value": algorithmic_bytes(rows, K_COLS) / best / 1e9, "unit": UNIT, "cores": c_oracle.num_threads(),
            "kind": "port", "sample": f"{rows} of {M_ROWS} rows x {K_COLS}, {reps} repetitions, median",
            "seconds_per_sample": best}


def run_reference(args):
    """Reference arm: the CPU restatement of the reference's path on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    from oracle import c_oracle
    import torch
    x, gamma = make_inputs()
    xb = x.view(torch.int16).numpy().view(np.uint16)
    gb = gamma.view(torch.int16).numpy().view(np.uint16)
    t0 = time.perf_counter()
    c_oracle.fused_norm_quantize(xb[:1024], gb, EPS)
    probe = (time.perf_counter() - t0) * (M_ROWS / 1024)
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows = M_ROWS if probe <= budget else max(128, int(M_ROWS * budget / probe) // 128 * 128)
    for _ in range(args.warmup):
        c_oracle.fused_norm_quantize(xb[:rows], gb, EPS)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        c_oracle.fused_norm_quantize(xb[:rows], gb, EPS)
    dt = (time.perf_counter() - t0) / args.steps
    val = algorithmic_bytes(rows, K_COLS) / dt / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16->e2m1/e4m3 (fp32 scale math)", "data": "synthetic",
            "config": {"workload": WORKLOAD, "sample_rows": rows},
            "cpu_baseline": {"value": val, "unit": UNIT, "cores": c_oracle.num_threads(), "kind": "port",
                             "sample": f"{rows} of {M_ROWS} rows x {K_COLS} per step"},
            "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "note": "reference CUDA kernels need a GPU; this arm times the CPU restatement of the same path "
                    "(oracle/fp4_oracle.c, pthreads) on the host cores"}
    print(json.dumps(line), flush=True)


def _mod(name):
    return importlib.import_module("mfu-fp4-training_b200." + name)


def split3_only(args):
    """One kernel family alone: the three-stream gradient quantiser of the attention backward (dQ | dK | dV with the
    8B model's widths 4096 / 1024 / 1024, each with its own tensor amax): the grouped amax kernel, the grouped strip
    quantiser and the concatenation of the row-wise scale tensors per call."""
    import torch
    M = int(args.split3_only)
    tkq = _mod("tk_quant_v5")
    peaks, _ = measured_peaks()
    g = torch.Generator(device="cuda").manual_seed(11)
    widths = (4096, 1024, 1024)
    grads = [(1e-3 * torch.randn(M, n, device="cuda", generator=g)).to(torch.bfloat16) for n in widths]
    steps, warm = min(args.steps, 50), max(args.warmup, 3)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(warm):
        tkq.tk_group_quantize_dim1_split3_for_gemm(*grads)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        tkq.tk_group_quantize_dim1_split3_for_gemm(*grads)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # per element: 2 B read by the amax pass, 2 B read again, 0.5 + 0.0625 B written per operand
    by = M * sum(widths) * (4.0 + 2 * 0.5625)
    print(json.dumps({"split3_only": {"M": M, "widths": list(widths), "ms_per_call": ms, "launches_per_call": 3,
                                      "algorithmic_GBps": by / (ms * 1e-3) / 1e9,
                                      "frac_of_measured_hbm": by / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}))


def load_reference_kernels():
    """The reference's own extension modules compiled by oracle/build_ref.sh (oracle/_ref/), or {} when absent.
    Used only to time the reference's kernels beside this library's on one GPU; nothing else touches them."""
    import glob
    import importlib.util
    out = {}
    for name in ("_tk_quant_v5", "_C", "mxfp4_quant_v4", "_C_mx"):
        paths = glob.glob(os.path.join(ROOT, "oracle", "_ref", name + ".*.so")) + glob.glob(os.path.join(ROOT, "oracle", "_ref", name + ".so"))
        if not paths:
            continue
        try:
            spec = importlib.util.spec_from_file_location(name, paths[0])
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            out[name] = mod
        except Exception as e:                       # a module that does not load is reported, not fatal
            out[name + "_error"] = str(e)[:200]
    return out


def _time_loop(torch, fn, iters, warm=3):
    """Mean ms of `iters` back-to-back calls of fn(i) after `warm` untimed ones (CUDA events on the current stream)."""
    for i in range(warm):
        fn(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(warm + i)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _sustained(torch, fn, seconds, iters):
    """Keeps fn running back to back for `seconds` (the part settles under its power limit), then times `iters` calls."""
    t0 = time.perf_counter()
    i = 0
    while time.perf_counter() - t0 < seconds:
        for _ in range(32):
            fn(i)
            i += 1
        torch.cuda.synchronize()
    return _time_loop(torch, fn, iters, warm=0)


def gemm_roofline_leg(torch, peaks, local_rank, world, refs, traffic):
    """The two FFN GEMM shapes of config 3 alone (gate/up: N 28672, K 4096; down: N 4096, K 14336; M 16384), random
    codes and scales, three operand sets in rotation (>= 3 x the 126 MB L2 together with the output), 20 timed
    launches after warm-up ("burst": the part still at its boost clock) and 20 more after ~1.2 s of back-to-back
    launches ("sustained": at the 1000 W limit the SM clock settles near 1.3-1.45 GHz).  Beside them, at N = 1 and
    when present, the reference's own nvfp4_gemm kernel and cuBLASLt's NVFP4 GEMM (torch._scaled_mm) on the same
    operands: the ceiling a library reaches on this box."""
    gemm = _mod("tk_gemm_c")
    dev = torch.device("cuda", local_rank)
    g = torch.Generator(device=dev).manual_seed(23)
    out = {}
    for name, (M, N, K) in (("gate_up", (M_ROWS, 28672, K_COLS)), ("down", (M_ROWS, K_COLS, 14336))):
        sets = []
        for _ in range(3):
            sets.append((torch.randint(0, 256, (M, K // 2), dtype=torch.uint8, device=dev, generator=g),
                         torch.randint(40, 64, (M // 128, K // 64, 512), dtype=torch.uint8, device=dev, generator=g),
                         torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=g),
                         torch.randint(40, 64, (N // 128, K // 64, 512), dtype=torch.uint8, device=dev, generator=g)))
        sg = torch.full((1,), 1e-3, dtype=torch.float32, device=dev)
        d = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        fl = 2.0 * M * N * K

        def ours(i):
            a, a_sc, b, b_sc = sets[i % 3]
            gemm.nvfp4_gemm(a, a_sc, sg, b, b_sc, sg, d)
        arms = {"ours": ours}
        if world == 1 and "_C" in refs:
            def ref_kernel(i):
                a, a_sc, b, b_sc = sets[i % 3]
                refs["_C"].nvfp4_gemm(a.view(torch.float4_e2m1fn_x2), a_sc.view(torch.float8_e4m3fn), sg,
                                      b.view(torch.float4_e2m1fn_x2), b_sc.view(torch.float8_e4m3fn), sg, d)
            arms["reference_kernel"] = ref_kernel
        if world == 1 and hasattr(torch, "_scaled_mm") and hasattr(torch, "float4_e2m1fn_x2"):
            def cublaslt(i):
                a, a_sc, b, b_sc = sets[i % 3]
                torch._scaled_mm(a.view(torch.float4_e2m1fn_x2), b.view(torch.float4_e2m1fn_x2).t(),
                                 a_sc.view(torch.float8_e4m3fn).reshape(-1), b_sc.view(torch.float8_e4m3fn).reshape(-1),
                                 out_dtype=torch.bfloat16)
            arms["cublaslt"] = cublaslt
        res = {}
        for arm, fn in arms.items():
            try:
                burst = _time_loop(torch, fn, 20)
                sampler = ClockSampler(local_rank)
                sampler.start()
                sus = _sustained(torch, fn, 1.2, 20)
                clk = sampler.stop()
            except Exception as e:       # a comparison arm that cannot run here is reported, the bench goes on
                if arm == "ours":
                    raise
                res[arm] = {"unavailable": str(e)[:160]}
                continue
            res[arm] = {"burst_ms": burst, "burst_tflops": fl / burst / 1e9, "sustained_ms": sus,
                        "sustained_tflops": fl / sus / 1e9, "sm_mhz_sustained": clk["sm_mhz"], "reasons": clk["reasons"]}
            time.sleep(1.0)              # let the part recover its boost clock before the next arm's burst figure
        out[name] = {"shape": f"{M}x{N}x{K}", **res}
        del sets, d
        torch.cuda.empty_cache()
    o_ = out["gate_up"]["ours"]
    mhz = o_["sm_mhz_sustained"] or 1965.0
    roof = {"bound": "tensor", "kernel": "fp4_gemm_pair_kernel<nvfp4, plain> (gate/up: M 16384, N 28672, K 4096)",
            "achieved": o_["burst_tflops"], "unit": "TFLOP/s", "peak": 9000.0, "frac": o_["burst_tflops"] / 9000.0,
            "peak_kind": "nominal dense FP4 at 1965 MHz (no measured FP4 peak exists); 4 x measured bf16 burst beside it",
            "frac_of_4x_measured_bf16": o_["burst_tflops"] / (4.0 * peaks["bf16_tflops"]),
            "sustained": {"achieved": o_["sustained_tflops"], "sm_mhz": mhz,
                          "frac_of_nominal_at_sampled_clock": o_["sustained_tflops"] / (9000.0 * mhz / 1965.0),
                          "frac_of_4x_measured_bf16_sustained": o_["sustained_tflops"] / (4.0 * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))},
            "traffic": traffic.get("fp4_gemm_pair_kernel", {}).get("dram_bytes_per_launch_16384x28672x4096"),
            "l2": "three operand sets in rotation; the 940 MB output alone exceeds L2"}
    return out, roof


def config1_leg(torch, dev):
    """Benchmark configuration 1: X bf16 [2048 x 4096] (outlier channels) and W bf16 [4096 x 4096] ~ N(0, 0.02) quantised to
    NVFP4 (1-D blocks, round to nearest, decode-centric as the reference's CPU emulation) and multiplied; beside it the
    numpy oracle's quantise -> dequantise -> float64 product on the host cores, and the relative Frobenius distance of
    the GPU's fp32 epilogue from that product."""
    import numpy as np
    from oracle import fp4_oracle as o
    tkq, gemm = _mod("tk_quant_v5"), _mod("tk_gemm_c")
    M, K, N = 2048, 4096, 4096
    x = o.make_activations(M, K, seed=1)
    w = o.bf16_round((0.02 * np.random.default_rng(2).standard_normal((N, K))).astype(np.float32))
    xd = torch.from_numpy(x).to(torch.bfloat16).to(dev)
    wd = torch.from_numpy(w).to(torch.bfloat16).to(dev)
    qw = tkq.tk_quantize_for_gemm(wd, False, False)
    d16 = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    d32 = torch.empty(M, N, dtype=torch.float32, device=dev)
    st = {}

    def step(i):
        st["qx"] = tkq.tk_quantize_for_gemm(xd, False, False)
        q = st["qx"]
        gemm.nvfp4_gemm(q[0], q[1], q[4], qw[0], qw[1], qw[4], d16)
    ms = _time_loop(torch, step, 20)
    q = st["qx"]
    gemm.nvfp4_gemm(q[0], q[1], q[4], qw[0], qw[1], qw[4], d32)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    rx, rw = o.nvfp4_quantize_for_gemm(x, False, False), o.nvfp4_quantize_for_gemm(w, False, False)
    ref = o.nvfp4_gemm_fp32(rx["row_fp4"], rx["row_sc_logical"], rx["sg"], rw["row_fp4"], rw["row_sc_logical"], rw["sg"])
    cpu_s = time.perf_counter() - t0
    got = d32.cpu().numpy()
    rel = float(np.linalg.norm(got - ref) / np.linalg.norm(ref))
    same_codes = bool(np.array_equal(q[0].view(torch.uint8).cpu().numpy(), rx["row_fp4"]))
    fl = 2.0 * M * N * K
    return {"workload": "config1: NVFP4 quantise X[2048x4096] -> GEMM with quantised W[4096x4096], RTN, decode-centric",
            "gpu_ms_quantise_x_plus_gemm": ms, "gpu_tflops": fl / ms / 1e9,
            "cpu_seconds_quantise_both_plus_qgemm": cpu_s, "cpu_tflops": fl / cpu_s / 1e12, "cpu_kind": "numpy oracle (port)",
            "cpu_cores": os.cpu_count(), "rel_frobenius_fp32_epilogue_vs_oracle": rel, "codes_equal_oracle": same_codes,
            "tolerance": 1e-3}


def ffn_forward_leg(torch, dist, world, local_rank, x_dev, gamma, peaks, iters=20):
    """Llama-3-8B FFN forward in NVFP4 at M=16384 per rank (config 3): fused RMSNorm+quant, grouped
    gate/up GEMM (N=28672, K=4096), SwiGLU producer, down GEMM (N=4096, K=14336), chained on real data.  Weights
    are quantised once outside the timed region.  Returns per-kernel and whole-step figures."""
    tkq, gemm = _mod("tk_quant_v5"), _mod("tk_gemm_c")
    H, K, M = 14336, K_COLS, M_ROWS
    dev = x_dev.device
    g = torch.Generator(device="cpu").manual_seed(7)
    def weight(n, k):
        return (0.02 * torch.randn(n, k, generator=g)).to(torch.bfloat16).to(dev)
    gather = None
    if world == 1:
        q1, q3, q2 = (tkq.tk_quantize_for_gemm(weight(H, K), False, True),
                      tkq.tk_quantize_for_gemm(weight(H, K), False, True),
                      tkq.tk_quantize_for_gemm(weight(K, H), False, True))
        ops = [(q[0].view(torch.uint8), q[1].view(torch.uint8), q[4]) for q in (q1, q3, q2)]
    else:
        # weights are FSDP-sharded along their rows; every rank quantises its shard and the ranks
        # all-gather packed codes + scale tiles (plus one float amax all-reduce per weight)
        fsdp = _mod("fsdp_weights")
        rank = dist.get_rank()
        shards = []
        for n, k in ((H, K), (H, K), (K, H)):
            w = weight(n, k)
            shards.append(w[rank * n // world:(rank + 1) * n // world].contiguous())
            del w
        ops = []
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_rep = 10
        for rep in range(3 + n_rep):
            if rep == 3:
                dist.barrier(); torch.cuda.synchronize(); g0.record()
            ops = fsdp.all_gather_nvfp4_weights(shards, None, False, True, reuse_buffers=True)
        g1.record(); torch.cuda.synchronize()
        ag = torch.tensor([g0.elapsed_time(g1) / n_rep], device=dev)
        dist.all_reduce(ag, op=dist.ReduceOp.MAX)
        nbytes = sum(fsdp.gathered_bytes(n, k, "nvfp4", False) for n, k in ((H, K), (H, K), (K, H)))
        gather = {"ms": ag.item(), "bytes_received_per_rank": nbytes, "bf16_equivalent_bytes": 3 * H * K * 2,
                  "note": "quantise own shards, ONE amax all-reduce and ONE group of all-gathers for the three FFN weights "
                          "(row-wise codes and scale tiles), send / receive buffers kept between steps; mean of 10"}
        ops = [(o_[0], o_[1], o_[4]) for o_ in ops]
    (w1c, w1s, w1g), (w3c, w3s, w3g), (w2c, w2s, w2g) = ops
    b13 = torch.cat([w1c, w3c], 0)
    b13_sc = torch.cat([w1s, w3s], 0)
    b13_sg = torch.cat([w1g.expand(H // 256), w3g.expand(H // 256)]).contiguous()
    h1 = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    h3 = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    y = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    st = {}
    def s_norm_quant():
        st["qx"] = tkq.tk_fused_norm_quantize(x_dev, gamma, EPS, False, True)
    def s_gate_up():
        q = st["qx"]; gemm.nvfp4_grouped_gemm(q[0], q[1], q[4], b13, b13_sc, b13_sg, h1, h3)
    def s_swiglu():
        st["qh"] = tkq.tk_silu_quantize_split_for_gemm(h1, h3)
    def s_down():
        q = st["qh"]; gemm.nvfp4_gemm(q[0], q[1], q[4], w2c, w2s, w2g, y)
    names = ["rmsnorm_quant", "gate_up_gemm", "swiglu_quant", "down_gemm"]
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms, total = _timed_stages(torch, [s_norm_quant, s_gate_up, s_swiglu, s_down], iters=iters)
    clk = sampler.stop()
    if world > 1:
        dist.barrier()
    t = torch.tensor(ms + [total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, total = t[:4].tolist(), t[4].item()
    fl_up, fl_down = 2.0 * M * 2 * H * K, 2.0 * M * K * H
    out = {"workload": "config3: Llama-3-8B FFN forward in NVFP4, M=16384 tokens per GPU", "ms": dict(zip(names, ms)),
           "step_ms": total, "iterations": iters, "clocks": clk,
           "gate_up_gemm_tflops": fl_up * world / (ms[1] * 1e-3) / 1e12,
           "down_gemm_tflops": fl_down * world / (ms[3] * 1e-3) / 1e12,
           "step_tflops": (fl_up + fl_down) * world / (total * 1e-3) / 1e12,
           "swiglu_quant_gbs": M * H * 5.125 * world / (ms[2] * 1e-3) / 1e9,
           "swiglu_quant_frac_of_measured_hbm": M * H * 5.125 / (ms[2] * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    if gather is not None:
        out["weight_all_gather"] = gather
    return out


def _timed_stages(torch, stages, iters=3, warm=3):
    """Runs the stage callables in order `warm + iters` times; returns the median ms per stage and per pass.
    Three untimed passes: the mirrors allocate their outputs, and a stage's previous outputs are still
    referenced while the next pass runs, so the caching allocator needs two passes to own both sets.  Medians:
    with tens of GB cached, one pass in ten can still stall for milliseconds inside the allocator (a cudaMalloc or
    a cudaFree of cached blocks behind a 470 MB request), which is the mirrors' cost, not the kernels'."""
    n = len(stages)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(n + 1)] for _ in range(iters)]
    for i in range(warm + iters):
        for j, fn in enumerate(stages):
            if i >= warm:
                ev[i - warm][j].record()
            fn()
        if i >= warm:
            ev[i - warm][n].record()
    torch.cuda.synchronize()
    ms = [statistics.median(e[j].elapsed_time(e[j + 1]) for e in ev) for j in range(n)]
    return ms, statistics.median(e[0].elapsed_time(e[n]) for e in ev)


def ffn_backward_leg(torch, dist, world, x_dev, gamma, peaks, iters=10):
    """Llama-3-8B FFN backward in NVFP4 at M=16384 per rank (benchmark configuration 4 as it is worded): dgrad GEMMs from
    round-to-nearest operands; wgrad GEMMs from operands with the 16-point Hadamard transform along the token
    dimension on BOTH sides (seeded sign vector) and Philox stochastic rounding (fixed seed / subsequence) of the
    gradient side.  Stages: quantise dY (row operand RTN, column operand transformed + SR; the transform's tensor
    maximum scan is part of the stage); W2 dgrad; W2 wgrad; SiLU-derivative producer (dh1, dh3 and their RTN
    operands); wgrad operands of dh1 and dh3 (transformed + SR); W1/W3 dgrad (two accumulated GEMMs); W1 and W3
    wgrads; RMSNorm backward with the residual gradient.  The transformed column operands of the forward's
    activations (x normalised, h) are made once outside the timed passes and timed on their own beside them."""
    tkq, gemm = _mod("tk_quant_v5"), _mod("tk_gemm_c")
    H, K, M = 14336, K_COLS, M_ROWS
    dev = x_dev.device
    SEED, SUBSEQ = 20261125, 3
    g = torch.Generator(device="cpu").manual_seed(11)
    def rnd(n, k, s):
        return (s * torch.randn(n, k, generator=g)).to(torch.bfloat16).to(dev)
    q1 = tkq.tk_quantize_for_gemm(rnd(H, K, 0.02), True, False)
    q3 = tkq.tk_quantize_for_gemm(rnd(H, K, 0.02), True, False)
    q2 = tkq.tk_quantize_for_gemm(rnd(K, H, 0.02), True, False)
    qx = tkq.tk_fused_norm_quantize(x_dev, gamma, EPS, False, True)
    inv_rms = qx[5]
    h1, h3 = rnd(M, H, 1.0), rnd(M, H, 1.0)
    # forward-side wgrad operands: column operands with the transform along M and the same sign vector, no SR
    xn = (x_dev.float() * inv_rms[:, None] * gamma.float()[None, :]).to(torch.bfloat16)
    hh = (torch.nn.functional.silu(h1.float()) * h3.float()).to(torch.bfloat16)
    fw = {}
    def s_fw_x():
        fw["x"] = tkq.tk_quantize_for_gemm_opt(xn, True, True, False, False, "col", True, SEED, SUBSEQ, 448.0, "both")
    def s_fw_h():
        fw["h"] = tkq.tk_quantize_for_gemm_opt(hh, True, True, False, False, "col", True, SEED, SUBSEQ, 448.0, "both")
    fw_ms, _ = _timed_stages(torch, [s_fw_x, s_fw_h], iters=5)
    del xn, hh
    dy = rnd(M, K, 1e-3)
    dh = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    dw2 = torch.empty(K, H, dtype=torch.bfloat16, device=dev)
    dx = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    dw1 = torch.empty(H, K, dtype=torch.bfloat16, device=dev)
    dw3 = torch.empty(H, K, dtype=torch.bfloat16, device=dev)
    st = {}
    tkq.tk_set_sr_invocation_count(0)
    def grad_operands(t):   # row: RTN; column: Hadamard along M with the sign vector + stochastic rounding
        return tkq.tk_quantize_for_gemm_opt(t, True, False, True, False, "col", True, SEED, SUBSEQ, 448.0, "col")
    def s_quant_dy():
        st["qdy"] = grad_operands(dy)
    def s_w2_dgrad():     # dh [M,H] = dY . W2 : B = W2's column operand [H, K/2]
        q = st["qdy"]; gemm.nvfp4_gemm(q[0], q[1], q[4], q2[2], q2[3], q2[4], dh)
    def s_w2_wgrad():     # dW2 [K,H] = dY^T . h : transformed column operands of both, contraction over M
        q, f = st["qdy"], fw["h"]; gemm.nvfp4_gemm(q[2], q[3], q[5], f[2], f[3], f[5], dw2)
    def s_silu_deriv():   # dh1 = dh * h3 * silu'(h1), dh3 = dh * silu(h1), both bf16 (the activations' backward)
        st["dh13"] = tkq.tk_silu_deriv_split_bf16(dh, h3, h1)
    def s_dh_operands():  # each gradient quantised once: row operand for the dgrad, transformed SR column operand for the wgrad
        st["g1"], st["g3"] = grad_operands(st["dh13"][0]), grad_operands(st["dh13"][1])
    def s_w13_dgrad():    # dx [M,K] = dh1 . W1 + dh3 . W3, fp32 running sum, one rounding
        a, b = st["g1"], st["g3"]
        gemm.nvfp4_batched_accum_gemm([a[0], b[0]], [a[1], b[1]], [a[4], b[4]], [q1[2], q3[2]], [q1[3], q3[3]],
                                      [q1[4], q3[4]], dx)
    def s_w13_wgrad():    # dW1 [H,K] = dh1^T . x, dW3 likewise
        f = fw["x"]
        gemm.nvfp4_gemm(st["g1"][2], st["g1"][3], st["g1"][5], f[2], f[3], f[5], dw1)
        gemm.nvfp4_gemm(st["g3"][2], st["g3"][3], st["g3"][5], f[2], f[3], f[5], dw3)
    dx_in = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    dgamma = torch.empty(K, dtype=torch.float32, device=dev)
    def s_rmsnorm_bwd():  # dx_in = RMSNorm backward of dx + the residual stream's gradient (dY), dgamma through row tiles
        gemm.rmsnorm_bwd_residual_out(dx, x_dev, gamma, inv_rms, dy, dx_in, dgamma)
    names = ["quant_dy_rht_sr", "w2_dgrad_gemm", "w2_wgrad_gemm", "silu_deriv_split_bf16", "dh_operands_rht_sr",
             "w13_dgrad_gemms", "w13_wgrad_gemms", "rmsnorm_bwd_residual"]
    ms, total = _timed_stages(torch, [s_quant_dy, s_w2_dgrad, s_w2_wgrad, s_silu_deriv, s_dh_operands, s_w13_dgrad,
                                      s_w13_wgrad, s_rmsnorm_bwd], iters=iters)
    # the attention side's form of the last step: three dgrad streams summed first (12 B per element)
    d_sum = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    partials = torch.empty((M + 255) // 256, K, dtype=torch.float32, device=dev)
    d3 = [dx, dy, rnd(M, K, 1e-3)]
    def s_sum3():
        gemm.sum3_rmsnorm_bwd_out(d3[0], d3[1], d3[2], x_dev, gamma, inv_rms, d_sum, dx_in, partials, dgamma)
    sum3_ms = _timed_stages(torch, [s_sum3], iters=10)[0][0]
    t = torch.tensor(ms + [total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, total = t[:-1].tolist(), t[-1].item()
    fl = {"w2_dgrad_gemm": 2.0 * M * H * K, "w2_wgrad_gemm": 2.0 * K * H * M, "w13_dgrad_gemms": 4.0 * M * K * H,
          "w13_wgrad_gemms": 4.0 * H * K * M}
    gemm_ms = sum(m for n_, m in zip(names, ms) if n_ in fl)
    return {"workload": "config4: Llama-3-8B FFN backward in NVFP4, M=16384 tokens per GPU; dgrad operands RTN, wgrad "
                        "operands Hadamard-16 along tokens with a seeded sign vector on both sides, gradients' column "
                        "operands with Philox SR (seed 20261125, subsequence 3, launch counter from 0)",
            "ms": dict(zip(names, ms)), "step_ms": total, "iterations": iters,
            "forward_side_wgrad_operands_ms": {"x_normalised_rht_col": fw_ms[0], "h_rht_col": fw_ms[1]},
            "gemm_tflops": {n_: fl[n_] * world / (m * 1e-3) / 1e12 for n_, m in zip(names, ms) if n_ in fl},
            "all_gemms_tflops": sum(fl.values()) * world / (gemm_ms * 1e-3) / 1e12,
            "step_tflops": sum(fl.values()) * world / (total * 1e-3) / 1e12,
            "quant_dy_gbs": M * K * 3.125 * world / (ms[0] * 1e-3) / 1e9,
            "silu_deriv_split_gbs": M * H * 10.0 * world / (ms[3] * 1e-3) / 1e9,
            "dh_operands_gbs": 2 * M * H * 3.125 * world / (ms[4] * 1e-3) / 1e9,
            "rmsnorm_bwd_residual_gbs": M * K * 8.0 * world / (ms[7] * 1e-3) / 1e9,
            "sum3_rmsnorm_bwd": {"ms": sum3_ms, "gbs": M * K * 12.0 / (sum3_ms * 1e-3) / 1e9,
                                 "frac_of_measured_hbm": M * K * 12.0 / (sum3_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]},
            "frac_of_nominal_fp4_all_gemms": sum(fl.values()) / (gemm_ms * 1e-3) / 1e12 / 9000.0,
            "frac_of_4x_measured_bf16_all_gemms": sum(fl.values()) / (gemm_ms * 1e-3) / 1e12 / (4.0 * peaks["bf16_tflops"])}


def attention_side_leg(torch, dist, world, peaks):
    """Attention-side producers and epilogues of a Llama-3-8B layer in NVFP4 at M = 16384 tokens per rank (two
    sequences of 8192): fused QKV projection with the rotary embedding in the GEMM epilogue (Q 4096, K 1024,
    V 1024 columns, heads of 128), quantisation of the attention output from its [B, H, S, 64] layout for the
    output projection, the inverse rotation of dQ / dK and the three-stream gradient quantiser in front of the
    QKV dgrad."""
    tkq, gemm = _mod("tk_quant_v5"), _mod("tk_gemm_c")
    M, K, q_dim, kv_dim, seq, head = M_ROWS, K_COLS, 4096, 1024, 8192, 128
    N = q_dim + 2 * kv_dim
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(17)
    def rnd(n, k, s):
        return (s * torch.randn(n, k, generator=g, device=dev)).to(torch.bfloat16)
    qx = tkq.tk_quantize_for_gemm(rnd(M, K, 1.0), False, True)
    qw = tkq.tk_quantize_for_gemm(rnd(N, K, 0.02), False, True)
    b_sg = qw[4].expand(N // 256).contiguous()
    ang = torch.rand(seq, head // 2, generator=g, device=dev) * 6.2831853
    cs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
    dq = torch.empty(M, q_dim, dtype=torch.bfloat16, device=dev)
    dk = torch.empty(M, kv_dim, dtype=torch.bfloat16, device=dev)
    dv = torch.empty(M, kv_dim, dtype=torch.bfloat16, device=dev)
    attn = rnd(M, K, 1.0).view(M // seq, K // 64, seq, 64)          # [B, H, S, 64]
    gq, gk, gv = rnd(M, q_dim, 1e-3), rnd(M, kv_dim, 1e-3), rnd(M, kv_dim, 1e-3)
    gq2, gk2 = torch.empty_like(gq), torch.empty_like(gk)
    def s_qkv_rope():
        gemm.nvfp4_grouped_gemm_rope_packed_split(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv, cs, seq, head, head)
    def s_qkv_plain():
        gemm.nvfp4_grouped_gemm(qx[0], qx[1], qx[4], qw[0], qw[1], b_sg, dq, dk, dv)
    def s_quant_attn():
        tkq.tk_quantize_nhsd_wo_for_gemm(attn, True, True)
    def s_inverse_rope():
        gemm.nvfp4_inverse_rope_packed_qk(gq, gk, cs, seq, head, gq2, gk2)
    def s_split3():
        tkq.tk_group_quantize_dim1_split3_for_gemm(gq2, gk2, gv)
    names = ["qkv_gemm_rope", "qkv_gemm_plain", "quant_attn_out_nhsd", "inverse_rope_dq_dk", "split3_quant"]
    ms, _ = _timed_stages(torch, [s_qkv_rope, s_qkv_plain, s_quant_attn, s_inverse_rope, s_split3], iters=20)
    t = torch.tensor(ms, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = t.tolist()
    fl = 2.0 * M * N * K
    return {"workload": "Llama-3-8B attention side in NVFP4, M=16384 tokens per GPU, heads of 128, sequences of 8192",
            "ms": dict(zip(names, ms)),
            "qkv_gemm_rope_tflops": fl * world / (ms[0] * 1e-3) / 1e12,
            "qkv_gemm_plain_tflops": fl * world / (ms[1] * 1e-3) / 1e12,
            "rope_epilogue_cost": ms[0] / ms[1] - 1.0,
            "quant_attn_out_gbs": M * K * 3.125 * world / (ms[2] * 1e-3) / 1e9,
            "inverse_rope_gbs": M * (q_dim + kv_dim) * 4.0 * world / (ms[3] * 1e-3) / 1e9,
            "split3_quant_gbs": M * N * 3.125 * world / (ms[4] * 1e-3) / 1e9}


def nvfp4_reference_producers_leg(torch, ref, ref_gemm=None):
    """Producers of config 4 (16384 tokens), the reference's compiled kernels and this library's in the same loop on
    the same tensors.  Only entry points whose launch path has no grid-wide software barrier: the optional-mode
    quantiser (tuned TMA kernel behind its scans) in the gradient form of config 4 — row operand round-to-nearest,
    column operand through the Hadamard transform along tokens with the sign vector and Philox SR — the SwiGLU element
    kernels, and the batched-accumulation GEMM."""
    tkq = _mod("tk_quant_v5")
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(29)
    rnd = lambda m, k, s: (s * torch.randn(m, k, generator=g, device=dev)).to(torch.bfloat16)
    M, K, H = M_ROWS, K_COLS, 14336
    out = {}
    def both(name, ref_fn, our_fn, iters):
        r = _time_loop(torch, lambda i: ref_fn(), iters)
        u = _time_loop(torch, lambda i: our_fn(), iters)
        out[name] = {"reference_ms": r, "ours_ms": u, "ours_over_reference": r / u}
    args = (True, False, True, False, "col", True, 20261125, 3, 448.0, "col")
    dy, dh1 = rnd(M, K, 1e-3), rnd(M, H, 1e-3)
    both("grad_operands_16384x4096", lambda: ref.tk_quantize_for_gemm_opt(dy, *args), lambda: tkq.tk_quantize_for_gemm_opt(dy, *args), 20)
    both("grad_operands_16384x14336", lambda: ref.tk_quantize_for_gemm_opt(dh1, *args), lambda: tkq.tk_quantize_for_gemm_opt(dh1, *args), 10)
    h1, h3 = rnd(M, H, 1.0), rnd(M, H, 1.0)
    both("silu_deriv_split_bf16_16384x14336", lambda: ref.tk_silu_deriv_split_bf16(dh1, h3, h1),
         lambda: tkq.tk_silu_deriv_split_bf16(dh1, h3, h1), 10)
    both("silu_mul_split_bf16_16384x14336", lambda: ref.tk_silu_mul_split_bf16(h1, h3), lambda: tkq.tk_silu_mul_split_bf16(h1, h3), 10)
    out["kernels"] = "reference _tk_quant_v5 (nvfp4_v5/tk_quantize.cu), compiled from the reference's sources for sm_100a"
    if ref_gemm is not None and hasattr(ref_gemm, "nvfp4_batched_accum_gemm"):
        gemm = _mod("tk_gemm_c")
        qa = [tkq.tk_quantize_for_gemm(t, False, False) for t in (dh1, h3)]
        del dy, dh1, h1, h3
        qb = [tkq.tk_quantize_for_gemm(rnd(K, H, 0.02), False, False) for _ in range(2)]
        d = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        lists = ([q[0] for q in qa], [q[1] for q in qa], [q[4] for q in qa], [q[0] for q in qb], [q[1] for q in qb], [q[4] for q in qb])
        both("batched_accum_gemm_2x16384x4096x14336", lambda: ref_gemm.nvfp4_batched_accum_gemm(*lists, d),
             lambda: gemm.nvfp4_batched_accum_gemm(*lists, d), 10)
        ref_gemm.nvfp4_batched_accum_gemm(*lists, d)
        d_ref = d.clone()
        gemm.nvfp4_batched_accum_gemm(*lists, d)
        out["batched_accum_gemm_2x16384x4096x14336"]["outputs_bit_identical"] = bool(torch.equal(d, d_ref))
    return out


def mxfp4_reference_producers_leg(torch, ref, ref_gemm=None):
    """The MXFP4 producers of config 5 (65536 tokens, mode 1), the reference's compiled kernels and this library's in
    the same loop on the same tensors: fused RMSNorm + quantiser [65536 x 4096], SwiGLU producer and SiLU-derivative
    pair [65536 x 14336], plain row + column quantiser [65536 x 4096]; with the reference's GEMM module also the gate
    (or up) and down GEMMs of that layer."""
    mxq = _mod("mxfp4_quant_v4")
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(23)
    rnd = lambda m, k, s: (s * torch.randn(m, k, generator=g, device=dev)).to(torch.bfloat16)
    M, K, H = 65536, K_COLS, 14336
    x, gam = rnd(M, K, 1.0), (1 + 0.1 * torch.randn(K, generator=g, device=dev)).to(torch.bfloat16)
    out = {}
    def both(name, ref_fn, our_fn, iters):
        r = _time_loop(torch, lambda i: ref_fn(), iters)
        u = _time_loop(torch, lambda i: our_fn(), iters)
        out[name] = {"reference_ms": r, "ours_ms": u, "ours_over_reference": r / u}
    both("rmsnorm_quant_65536x4096", lambda: ref.mxfp4_fused_rmsnorm_quantize_row_and_col(x, gam, EPS, 1),
         lambda: mxq.mxfp4_fused_rmsnorm_quantize_row_and_col(x, gam, EPS, 1), 10)
    both("quantize_row_and_col_65536x4096", lambda: ref.mxfp4_quantize_row_and_col(x, 1),
         lambda: mxq.mxfp4_quantize_row_and_col(x, 1), 10)
    del x
    h1, h3, dh = rnd(M, H, 1.0), rnd(M, H, 1.0), rnd(M, H, 1e-3)
    both("silu_mul_quant_65536x14336", lambda: ref.mxfp4_fused_silu_mul_quantize_row_and_col(h1, h3, 1),
         lambda: mxq.mxfp4_fused_silu_mul_quantize_row_and_col(h1, h3, 1), 5)
    both("silu_deriv_quant_split2_65536x14336", lambda: ref.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, h1, 1),
         lambda: mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, h1, 1), 5)
    out["kernels"] = "reference mxfp4_quant_v4 (mxfp4_v4/tk_quantize.cu), compiled from the reference's sources for sm_100a"
    if ref_gemm is not None:
        del dh
        gemm = _mod("tk_gemm_c_mx")
        qh = mxq.mxfp4_quantize_for_gemm(h1, 1)                                   # [M, H] row operand
        del h1, h3
        qx = mxq.mxfp4_quantize_for_gemm(rnd(M, K, 1.0), 1)                       # [M, K]
        qw1 = mxq.mxfp4_quantize_for_gemm(rnd(H, K, 0.02), 1)                     # W1 [H, K]
        qw2 = mxq.mxfp4_quantize_for_gemm(rnd(K, H, 0.02), 1)                     # W2 [K, H]
        d_up = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
        d_dn = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
        for name, a, b, d, fl in (("gemm_65536x14336x4096", qx, qw1, d_up, 2.0 * M * H * K),
                                  ("gemm_65536x4096x14336", qh, qw2, d_dn, 2.0 * M * K * H)):
            both(name, lambda: ref_gemm.mxfp4_gemm(a[0], a[1], b[0], b[1], d),
                 lambda: gemm.mxfp4_gemm(a[0], a[1], b[0], b[1], d), 10)
            ref_gemm.mxfp4_gemm(a[0], a[1], b[0], b[1], d)
            d_ref = d.clone()
            gemm.mxfp4_gemm(a[0], a[1], b[0], b[1], d)
            out[name]["outputs_bit_identical"] = bool(torch.equal(d, d_ref))
            del d_ref
            out[name]["ours_tflops"] = fl / (out[name]["ours_ms"] * 1e-3) / 1e12
            out[name]["reference_tflops"] = fl / (out[name]["reference_ms"] * 1e-3) / 1e12
        # the Q projection with the rotary epilogue (heads of 128, sequences of 8192): [M, 4096] = X . Wq^T, every pair rotated
        del d_up, qh, qw2
        qwq = mxq.mxfp4_quantize_for_gemm(rnd(K, K, 0.02), 1)
        ang = torch.rand(8192, 64, generator=g, device=dev) * 6.2831853
        cs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
        name = "gemm_rope_65536x4096x4096"
        both(name, lambda: ref_gemm.mxfp4_gemm_rope_live64(qx[0], qx[1], qwq[0], qwq[1], d_dn, cs, 8192),
             lambda: gemm.mxfp4_gemm_rope_live64(qx[0], qx[1], qwq[0], qwq[1], d_dn, cs, 8192), 10)
        ref_gemm.mxfp4_gemm_rope_live64(qx[0], qx[1], qwq[0], qwq[1], d_dn, cs, 8192)
        d_ref = d_dn.clone()
        gemm.mxfp4_gemm_rope_live64(qx[0], qx[1], qwq[0], qwq[1], d_dn, cs, 8192)
        out[name]["outputs_bit_identical"] = bool(torch.equal(d_dn, d_ref))
        out["gemm_kernels"] = "reference _C_mx.mxfp4_gemm / mxfp4_gemm_rope_live64 (mxfp4_gb200/mxfp4_gb200_gemm.cu), compiled from the reference's sources"
    return out


def mxfp4_layer_leg(torch, dist, world, gamma, peaks):
    """Config 5: MXFP4 (E8M0 / 32-blocks, mode 1) forward AND backward GEMM set of one Llama-3-8B decoder layer
    (QKV [6144,4096], O [4096,4096], W1/W3 [14336,4096], W2 [4096,14336]) on this rank's share of M = 65536 tokens,
    with the producers that feed them.  With N > 1 the layer's weights are FSDP-sharded along their rows and fetched,
    as packed codes + scale tiles in both orientations, by ONE all-gather inside a timed stage of every pass."""
    mxq, gmx = _mod("mxfp4_quant_v4"), _mod("tk_gemm_c_mx")
    K, H, NQKV = K_COLS, 14336, 6144
    M = 65536 // world
    dev = gamma.device
    g = torch.Generator(device="cpu").manual_seed(13)
    def rnd(n, k, s):
        return (s * torch.randn(n, k, generator=g)).to(torch.bfloat16).to(dev)
    wnames = ("qkv", "o", "w1", "w3", "w2")
    wshapes = {"qkv": (NQKV, K), "o": (K, K), "w1": (H, K), "w3": (H, K), "w2": (K, H)}
    wq = {}
    gather_stage = None
    if world == 1:
        wq = {n_: mxq.mxfp4_quantize_row_and_col(rnd(*wshapes[n_], 0.02), 1) for n_ in wnames}
    else:
        fsdp = _mod("fsdp_weights")
        rank = dist.get_rank()
        shards = []
        for n_ in wnames:
            n, k = wshapes[n_]
            w = rnd(n, k, 0.02)
            shards.append(w[rank * n // world:(rank + 1) * n // world].contiguous())
            del w
        def gather_stage():
            got = fsdp.all_gather_mxfp4_weights(shards, None, True, 1, reuse_buffers=True)
            for n_, o_ in zip(wnames, got):
                wq[n_] = o_
        gather_stage()
    x = rnd(M, K, 1.0)
    attn = rnd(M, K, 1.0)
    qkv = torch.empty(M, NQKV, dtype=torch.bfloat16, device=dev)
    o_out = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    h1 = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    h3 = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    y = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    st = {}
    def s_norm_quant():
        st["qx"] = mxq.mxfp4_fused_rmsnorm_quantize_row_and_col(x, gamma, EPS, 1)
    def s_qkv():
        q = st["qx"]; gmx.mxfp4_gemm(q[0], q[1], wq["qkv"][0], wq["qkv"][1], qkv)
    def s_quant_attn():
        st["qa"] = mxq.mxfp4_quantize_row_and_col(attn, 1)
    def s_o():
        q = st["qa"]; gmx.mxfp4_gemm(q[0], q[1], wq["o"][0], wq["o"][1], o_out)
    def s_gate_up():      # the reference runs the two projections as one batched launch (mxfp4_fused_linear.py:9494)
        q = st["qx"]
        gmx.mxfp4_batched_gemm([q[0], q[0]], [q[1], q[1]], [wq["w1"][0], wq["w3"][0]], [wq["w1"][1], wq["w3"][1]], [h1, h3])
    def s_swiglu():
        st["qh"] = mxq.mxfp4_fused_silu_mul_quantize_row_and_col(h1, h3, 1)
    def s_down():
        q = st["qh"]; gmx.mxfp4_gemm(q[0], q[1], wq["w2"][0], wq["w2"][1], y)
    fwd = [("rmsnorm_quant", s_norm_quant), ("qkv_gemm", s_qkv), ("quant_attn_out", s_quant_attn), ("o_gemm", s_o),
           ("gate_up_gemms", s_gate_up), ("swiglu_quant", s_swiglu), ("down_gemm", s_down)]
    # ---- backward: gradient quantisers, dgrads (weights' column operands), wgrads (column operands of both sides)
    dy = rnd(M, K, 1e-3)
    dh = torch.empty(M, H, dtype=torch.bfloat16, device=dev)
    dxf = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    dattn = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    dq, dk, dv = rnd(M, K, 1e-3), rnd(M, (NQKV - K) // 2, 1e-3), rnd(M, (NQKV - K) // 2, 1e-3)   # as attention's backward leaves them
    dxa = torch.empty(M, K, dtype=torch.bfloat16, device=dev)
    dw = {n_: torch.empty(*wshapes[n_], dtype=torch.bfloat16, device=dev) for n_ in wnames}
    def s_q_dy():
        st["gdy"] = mxq.mxfp4_quantize_row_and_col(dy, 1)
    def s_w2_dgrad():
        q = st["gdy"]; gmx.mxfp4_gemm(q[0], q[1], wq["w2"][2], wq["w2"][3], dh)
    def s_w2_wgrad():
        q, f = st["gdy"], st["qh"]; gmx.mxfp4_gemm(q[2], q[3], f[2], f[3], dw["w2"])
    def s_silu_deriv():   # the reference's default producer for the one-pass dgrad (mxfp4_fused_linear.py:10415-10431)
        st["gd"] = mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col_splitcols(dh, h3, h1, 1)
    def s_w13_dgrad():   # dgrad of the fused gate/up projection from the side-by-side [dh1 | dh3] row operand, one launch
        d = st["gd"]
        hs = H // 128
        gmx.mxfp4_split2_dgrad_strided_onepass_gemm(d[0], [d[1].narrow(1, 0, hs), d[1].narrow(1, hs, hs)], [0, H // 2],
                                                    [H // 2, H // 2], [wq["w1"][2], wq["w3"][2]],
                                                    [wq["w1"][3], wq["w3"][3]], dxf, -1)
    def s_w13_wgrad():
        d, f = st["gd"], st["qx"]
        gmx.mxfp4_gemm(d[2], d[3], f[2], f[3], dw["w1"])
        gmx.mxfp4_gemm(d[4], d[5], f[2], f[3], dw["w3"])
    def s_q_do():
        st["gdo"] = mxq.mxfp4_quantize_row_and_col(dxf, 1)
    def s_o_dgrad():
        q = st["gdo"]; gmx.mxfp4_gemm(q[0], q[1], wq["o"][2], wq["o"][3], dattn)
    def s_o_wgrad():
        q, f = st["gdo"], st["qa"]; gmx.mxfp4_gemm(q[2], q[3], f[2], f[3], dw["o"])
    def s_q_dqkv():
        st["gq"] = mxq.mxfp4_quantize_split3_row_and_col(dq, dk, dv, 1)     # no bf16 concatenation (mxfp4_fused_linear.py:3748)
    def s_qkv_dgrad():
        q = st["gq"]; gmx.mxfp4_gemm(q[0], q[1], wq["qkv"][2], wq["qkv"][3], dxa)
    def s_qkv_wgrad():
        q, f = st["gq"], st["qx"]; gmx.mxfp4_gemm(q[2], q[3], f[2], f[3], dw["qkv"])
    bwd = [("quant_dy", s_q_dy), ("w2_dgrad_gemm", s_w2_dgrad), ("w2_wgrad_gemm", s_w2_wgrad),
           ("silu_deriv_quant_splitcols", s_silu_deriv), ("w13_dgrad_onepass_gemm", s_w13_dgrad), ("w13_wgrad_gemms", s_w13_wgrad),
           ("quant_d_o", s_q_do), ("o_dgrad_gemm", s_o_dgrad), ("o_wgrad_gemm", s_o_wgrad), ("quant_d_qkv", s_q_dqkv),
           ("qkv_dgrad_gemm", s_qkv_dgrad), ("qkv_wgrad_gemm", s_qkv_wgrad)]
    stages = ([("weight_all_gather", gather_stage)] if gather_stage is not None else []) + fwd + bwd
    names = [n_ for n_, _ in stages]
    ms, total = _timed_stages(torch, [f for _, f in stages], iters=5)
    t = torch.tensor(ms + [total], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, total = t[:-1].tolist(), t[-1].item()
    by = dict(zip(names, ms))
    fl = {"qkv_gemm": 2.0 * M * NQKV * K, "o_gemm": 2.0 * M * K * K, "gate_up_gemms": 4.0 * M * H * K, "down_gemm": 2.0 * M * K * H,
          "w2_dgrad_gemm": 2.0 * M * H * K, "w2_wgrad_gemm": 2.0 * M * H * K, "w13_dgrad_onepass_gemm": 4.0 * M * H * K,
          "w13_wgrad_gemms": 4.0 * M * H * K, "o_dgrad_gemm": 2.0 * M * K * K, "o_wgrad_gemm": 2.0 * M * K * K,
          "qkv_dgrad_gemm": 2.0 * M * NQKV * K, "qkv_wgrad_gemm": 2.0 * M * NQKV * K}
    gemm_ms = sum(by[n_] for n_ in fl)
    out = {"workload": f"config5: MXFP4 mode 1, one decoder layer's GEMM set forward + backward, M={M} tokens per GPU "
                       f"(65536 / {world})" + (", weights FSDP-sharded and all-gathered as packed FP4 + scales" if world > 1 else ""),
           "ms": by, "step_ms": total,
           "gemm_tflops": {n_: fl[n_] * world / (by[n_] * 1e-3) / 1e12 for n_ in fl},
           "all_gemms_tflops": sum(fl.values()) * world / (gemm_ms * 1e-3) / 1e12,
           "rmsnorm_quant_gbs": M * K * 3.0625 * world / (by["rmsnorm_quant"] * 1e-3) / 1e9,
           "swiglu_quant_gbs": M * H * (4 + 1.0625) * world / (by["swiglu_quant"] * 1e-3) / 1e9,
           "frac_of_nominal_fp4_all_gemms": sum(fl.values()) / (gemm_ms * 1e-3) / 1e12 / 9000.0,
           "frac_of_4x_measured_bf16_all_gemms": sum(fl.values()) / (gemm_ms * 1e-3) / 1e12 / (4.0 * peaks["bf16_tflops"])}
    if world > 1:
        fsdp = _mod("fsdp_weights")
        nbytes = sum(fsdp.gathered_bytes(*wshapes[n_], "mxfp4", True) for n_ in wnames)
        out["weight_all_gather"] = {"ms": by["weight_all_gather"], "bytes_received_per_rank": nbytes,
                                    "bf16_equivalent_bytes": 2 * sum(a * b for a, b in wshapes.values())}
    return out


def rmsnorm_bwd_only(args):
    """sum3 + RMSNorm backward + tiled dgamma on [M, K] bf16 streams; two input sets alternate so that no step
    finds its inputs in L2.  Prints time and algorithmic bandwidth (12 B per element)."""
    import torch
    gemm = importlib.import_module("mfu-fp4-training_b200.tk_gemm_c")
    M, K = (int(v) for v in args.rmsnorm_bwd_only.lower().split("x"))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(5)
    sets = [[(s * torch.randn(M, K, generator=g, device=dev)).to(torch.bfloat16) for s in (1e-3, 1e-3, 1e-3, 1.0)]
            for _ in range(2)]
    gamma = (1 + 0.1 * torch.randn(K, generator=g, device=dev)).to(torch.bfloat16)
    inv = [torch.rsqrt(st[3].float().pow(2).mean(dim=1) + EPS) for st in sets]
    d_sum, dx = torch.empty_like(sets[0][3]), torch.empty_like(sets[0][3])
    partials = torch.empty((M + 255) // 256, K, dtype=torch.float32, device=dev)
    dgamma = torch.empty(K, dtype=torch.float32, device=dev)
    def step(i):
        d0, d1, d2, x = sets[i % 2]
        gemm.sum3_rmsnorm_bwd_out(d0, d1, d2, x, gamma, inv[i % 2], d_sum, dx, partials, dgamma)
    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    steps = min(args.steps, 50)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    print(json.dumps({"rmsnorm_bwd_only": args.rmsnorm_bwd_only, "ms": ms, "algorithmic_gbs": 12.0 * M * K / (ms * 1e-3) / 1e9,
                      "status": importlib.import_module("mfu-fp4-training_b200._lib").device_status()}))


def mx_swiglu_only(args):
    """The one-pass MXFP4 SwiGLU producers at [M, H]: operands of silu(h1) * h3 (5.0625 algorithmic bytes per
    element) and of the dh1 / dh3 pair (8.125).  Prints both times and algorithmic bandwidths."""
    import torch
    mxq = importlib.import_module("mfu-fp4-training_b200.mxfp4_quant_v4")
    M, H = (int(v) for v in args.mx_swiglu_only.lower().split("x"))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(7)
    h1, h3, dh = ((s * torch.randn(M, H, generator=g, device=dev)).to(torch.bfloat16) for s in (1.0, 1.0, 1e-3))
    out = {}
    for name, fn, bytes_per in (("silu_mul", lambda: mxq.mxfp4_fused_silu_mul_quantize_row_and_col(h1, h3, 1), 5.0625),
                                ("silu_deriv_split2",
                                 lambda: mxq.mxfp4_fused_silu_deriv_quantize_split2_row_and_col(dh, h3, h1, 1), 8.125)):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        steps = min(args.steps, 20)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[name] = {"ms": ms, "algorithmic_gbs": bytes_per * M * H / (ms * 1e-3) / 1e9}
    out["status"] = importlib.import_module("mfu-fp4-training_b200._lib").device_status()
    print(json.dumps({"mx_swiglu_only": args.mx_swiglu_only, **out}))


def gemm_only(args):
    """Times one GEMM form alone at one shape on cuda:0 (random codes and scales): the plain NVFP4 GEMM, the fused QKV
    projection with the rotary embedding in its epilogue (--gemm-form rope: heads of 128, sequences of 4096, the last
    sixth of the columns not rotated), two accumulated terms in one launch (--gemm-form accum2), the MXFP4 GEMM
    (--gemm-form mx), or the MXFP4 GEMM with the rotary epilogue on every column pair (--gemm-form mxrope)."""
    import torch
    gemm = importlib.import_module("mfu-fp4-training_b200.tk_gemm_c")
    lib = importlib.import_module("mfu-fp4-training_b200._lib")
    M, N, K = (int(v) for v in args.gemm_only.lower().split("x"))
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    def operand(rows):
        return (torch.randint(0, 256, (rows, K // 2), dtype=torch.uint8, device=dev, generator=g),
                torch.randint(40, 64, (rows // 128, K // 64, 512), dtype=torch.uint8, device=dev, generator=g))
    a, a_sc = operand(M)
    b, b_sc = operand(N)
    sg = torch.full((1,), 1e-3, dtype=torch.float32, device=dev)
    d = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    flops = 2.0 * M * N * K
    if args.gemm_form == "rope":
        seq, head = 4096, 128
        kv = N // 6
        dq, dk, dv = (torch.empty(M, n, dtype=torch.bfloat16, device=dev) for n in (N - 2 * kv, kv, kv))
        ang = torch.rand(seq, head // 2, generator=g, device=dev) * 6.2831853
        cs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
        b_sg = sg.expand(N // 256).contiguous()
        def run():
            gemm.nvfp4_grouped_gemm_rope_packed_split(a, a_sc, sg, b, b_sc, b_sg, dq, dk, dv, cs, seq, head, head)
    elif args.gemm_form == "accum2":
        a2, a2_sc = operand(M)
        b2, b2_sc = operand(N)
        flops *= 2
        def run():
            gemm.nvfp4_batched_accum_gemm([a, a2], [a_sc, a2_sc], [sg, sg], [b, b2], [b_sc, b2_sc], [sg, sg], d)
    elif args.gemm_form in ("mx", "mxrope"):
        gmx = importlib.import_module("mfu-fp4-training_b200.tk_gemm_c_mx")
        def mx_scales(rows):    # E8M0 bytes near 127: one per 32 elements, [rows/128, K/128, 32, 16]
            return torch.randint(120, 132, (rows // 128, K // 128, 32, 16), dtype=torch.uint8, device=dev, generator=g)
        a_e, b_e = mx_scales(M), mx_scales(N)
        if args.gemm_form == "mxrope":     # every column pair rotated, heads of 128, sequences of 4096
            ang = torch.rand(4096, 64, device=dev, generator=g) * 6.2831853
            cs = torch.stack([torch.cos(ang), torch.sin(ang)], dim=-1).contiguous()
            def run():
                gmx.mxfp4_gemm_rope_live64(a, a_e, b, b_e, d, cs, 4096)
        else:
            def run():
                gmx.mxfp4_gemm(a, a_e, b, b_e, d)
    else:
        def run():
            gemm.nvfp4_gemm(a, a_sc, sg, b, b_sc, sg, d)
    for _ in range(args.warmup):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    print(json.dumps({"gemm_only": args.gemm_only, "form": args.gemm_form, "ms": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                      "status": lib.device_status()}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true",
                    help="timed loop only (no per-kernel, end-to-end or CPU legs): the command ncu captures")
    ap.add_argument("--gemm-only", default=None, metavar="MxNxK",
                    help="time only the NVFP4 GEMM at this shape (tuning / ncu capture helper)")
    ap.add_argument("--gemm-form", default="plain", choices=["plain", "rope", "accum2", "mx", "mxrope"],
                    help="with --gemm-only: which epilogue form to time")
    ap.add_argument("--rmsnorm-bwd-only", default=None, metavar="MxK",
                    help="time only the RMSNorm backward (sum3 form) at this shape (tuning / ncu capture helper)")
    ap.add_argument("--mx-swiglu-only", default=None, metavar="MxH",
                    help="time only the one-pass MXFP4 SwiGLU producers at this shape (tuning / ncu capture helper)")
    ap.add_argument("--split3-only", default=None, metavar="M",
                    help="time only the three-stream gradient quantiser (widths 4096/1024/1024) on M rows (ncu capture helper)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.mx_swiglu_only:
        mx_swiglu_only(args)
        return
    if args.split3_only:
        split3_only(args)
        return
    if args.gemm_only:
        gemm_only(args)
        return
    if args.rmsnorm_bwd_only:
        rmsnorm_bwd_only(args)
        return

    if args.impl == "reference":
        run_reference(args)
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the FP4 hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL writes its version banner and debug lines to stdout; stdout carries the one JSON line
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    tkq = importlib.import_module("mfu-fp4-training_b200.tk_quant_v5")
    lib = importlib.import_module("mfu-fp4-training_b200._lib")
    peaks, peak_kind = measured_peaks()

    x_host, g_host = make_inputs()
    x_pin, g_pin = x_host.pin_memory(), g_host.pin_memory()
    n_rot = 3  # rotate over three copies of X (402 MB > L2) so no step finds its input in L2
    xs = [x_pin.cuda(non_blocking=True) for _ in range(n_rot)]
    gamma = g_pin.cuda(non_blocking=True)
    torch.cuda.synchronize()

    def step(i):
        return tkq.tk_fused_norm_quantize(xs[i % n_rot], gamma, EPS, False, True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        out = step(i)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        out = step(i)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = t.item()
    ms_per_step = ms_total / args.steps
    alg = algorithmic_bytes(M_ROWS, K_COLS)
    value = alg * world / (ms_per_step * 1e-3) / 1e9
    if lib.device_status() != 0:
        raise RuntimeError("device status word is non-zero: a kernel gave up a bounded wait")

    if args.quick:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                              "warmup": args.warmup, "ms_per_step": ms_per_step, "quick": True}), flush=True)
            sampler.stop()
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- per-kernel timing through the C ABI (pass 1: statistics, pass 2: quantise) -------
    dev = torch.device("cuda", local_rank)
    u8 = dict(dtype=torch.uint8, device=dev)
    row_fp4 = torch.empty((M_ROWS, K_COLS // 2), **u8); row_sc = torch.empty((M_ROWS * K_COLS // 16,), **u8)
    col_fp4 = torch.empty((K_COLS, M_ROWS // 2), **u8); col_sc = torch.empty((M_ROWS * K_COLS // 16,), **u8)
    inv_rms = torch.empty(M_ROWS, dtype=torch.float32, device=dev)
    amax_sg = torch.empty(2, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    n_k = min(args.steps, 20)
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(n_k)]
    for i in range(3 + n_k):
        xi = xs[i % n_rot]
        if i >= 3:
            ev[i - 3][0].record()
        lib.call("fp4b200_nvfp4_rmsnorm_stats", xi.data_ptr(), gamma.data_ptr(), EPS, M_ROWS, K_COLS,
                 inv_rms.data_ptr(), 1, amax_sg.data_ptr(), stream)
        if i >= 3:
            ev[i - 3][1].record()
        lib.call("fp4b200_nvfp4_quantize_normed", xi.data_ptr(), gamma.data_ptr(), inv_rms.data_ptr(),
                 amax_sg.data_ptr(), M_ROWS, K_COLS, 1, row_fp4.data_ptr(), row_sc.data_ptr(),
                 col_fp4.data_ptr(), col_sc.data_ptr(), stream)
        if i >= 3:
            ev[i - 3][2].record()
    torch.cuda.synchronize()
    t_stats = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    t_quant = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    quant_bytes = M_ROWS * K_COLS * 3.125
    stats_bytes = M_ROWS * K_COLS * 2.0
    achieved = quant_bytes / (t_quant * 1e-3) / 1e9
    traffic = load_traffic()
    roofline = {"bound": "hbm", "kernel": "nvfp4_quantize_strip_kernel<encode_centric, norm, paired> (pass 2)",
                "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                "peak_kind": f"of {peak_kind} copy bandwidth",
                "traffic": traffic.get("nvfp4_quantize_strip_kernel", {}).get("dram_bytes_per_launch_16384x4096"),
                "algorithmic_bytes_per_launch": quant_bytes, "avg_launch_ms": t_quant,
                "other_kernels": {"rmsnorm_stats_pair_kernel + partials reduction (pass 1 stand-alone, two launches)": {
                    "achieved": stats_bytes / (t_stats * 1e-3) / 1e9, "unit": "GB/s", "avg_launch_ms": t_stats,
                    "algorithmic_bytes_per_launch": stats_bytes,
                    "frac": stats_bytes / (t_stats * 1e-3) / 1e9 / peaks["hbm_gbs"]}},
                "fused_op_frac_of_peak": (alg / (ms_per_step * 1e-3) / 1e9) / peaks["hbm_gbs"]}

    # ---- end to end: pinned host X in, all operands + inv_rms + scales back to the host ----
    # Every step copies its own X and gamma from pinned host memory, calls the public entry point and
    # copies every result back to pinned host memory.  As a caller with a steady stream of batches
    # would, the three stages run on three streams with two sets of buffers, so the copy-in of step
    # i+1 and the copy-out of step i-1 overlap the kernels of step i (PCIe is full duplex); nothing is
    # skipped and nothing is reused between steps.
    n_e2e = max(4, min(args.steps, 12))
    h2d = x_pin.numel() * 2 + g_pin.numel() * 2
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty_like(xs[0]) for _ in range(2)]
    g_dev = [torch.empty_like(gamma) for _ in range(2)]
    outs_host = [None, None]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    d2h = 0

    def e2e_step(i):
        nonlocal d2h
        k = i & 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_comp[k])          # the kernels that read this input buffer two steps ago
            x_dev[k].copy_(x_pin, non_blocking=True)
            g_dev[k].copy_(g_pin, non_blocking=True)
            ev_in[k].record(s_in)
        cur.wait_event(ev_in[k])
        o_ = tkq.tk_fused_norm_quantize(x_dev[k], g_dev[k], EPS, False, True)
        ev_comp[k].record(cur)
        res = [o_[0].view(torch.uint8), o_[1].view(torch.uint8), o_[2].view(torch.uint8),
               o_[3].view(torch.uint8), o_[5], o_[7]]
        if outs_host[k] is None:
            outs_host[k] = [torch.empty(r.shape, dtype=r.dtype).pin_memory() for r in res]
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[k])
            s_out.wait_event(ev_out[k])          # the previous copy-out into this set of host buffers
            for hbuf, r in zip(outs_host[k], res):
                hbuf.copy_(r, non_blocking=True)
                r.record_stream(s_out)
            ev_out[k].record(s_out)
        d2h = sum(r.numel() * r.element_size() for r in res)

    for i in range(2):
        e2e_step(i)
    cur.wait_stream(s_out)
    barrier()
    e0.record()
    for i in range(n_e2e):
        e2e_step(i)
    cur.wait_stream(s_in)
    cur.wait_stream(s_out)
    e1.record()
    barrier()
    t2 = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    if world > 1:
        dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = t2.item() / n_e2e
    e2e = {"value": alg * world / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": n_e2e,
           "pipeline": "copy-in, kernels and copy-out on three streams, two buffer sets"}

    del outs_host
    clocks = sampler.stop() if rank == 0 else None      # clocks of the headline's timed region and its end-to-end leg

    # ---- the shape an 8-way split of config 2's tokens gives each GPU: 2048 rows, X (16.8 MB) stays in L2 ----
    # Twenty calls through the C ABI captured in one CUDA graph: at 10 us per call the host's launch path would
    # otherwise be what is timed.
    rows_s = 2048
    x_small = xs[0][:rows_s].contiguous()
    o_small = (torch.empty((rows_s, K_COLS // 2), **u8), torch.empty((rows_s * K_COLS // 16,), **u8),
               torch.empty((K_COLS, rows_s // 2), **u8), torch.empty((rows_s * K_COLS // 16,), **u8))
    side = torch.cuda.Stream()

    def small_call(st):
        lib.call("fp4b200_nvfp4_fused_norm_quantize", x_small.data_ptr(), gamma.data_ptr(), EPS, rows_s, K_COLS, inv_rms.data_ptr(),
                 1, 1, o_small[0].data_ptr(), o_small[1].data_ptr(), o_small[2].data_ptr(), o_small[3].data_ptr(),
                 amax_sg.data_ptr(), st)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        small_call(side.cuda_stream)          # the stream's first call creates the library's per-stream scratch
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(20):
            small_call(torch.cuda.current_stream().cuda_stream)
    small_ms = _time_loop(torch, lambda i: graph.replay(), 20, warm=3) / 20
    small = {"rows": rows_s, "ms": small_ms, "value": algorithmic_bytes(rows_s, K_COLS) / (small_ms * 1e-3) / 1e9, "unit": UNIT,
             "frac_of_measured_hbm": algorithmic_bytes(rows_s, K_COLS) / (small_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
             "note": "strong-scaling point: 16384 / 8 tokens per GPU; the input (16.8 MB) and the outputs stay in L2, so the "
                     "figure is a rate against the HBM copy bandwidth, not HBM traffic; 20 calls per CUDA-graph replay"}
    del graph

    # ---- the same loop with the caller's promise that no input is produced by the kernel launched just before its call
    # (true of this loop): the statistics kernel of call i+1 then fills its ring while the quantiser of call i drains
    before = lib.load().fp4b200_set_pdl_early_reads(1)
    early_ms = _time_loop(torch, step, min(args.steps, 200), warm=5)
    lib.load().fp4b200_set_pdl_early_reads(before)
    early = {"ms_per_step": early_ms, "value": alg / (early_ms * 1e-3) / 1e9, "unit": UNIT,
             "note": "fp4b200_set_pdl_early_reads(1): not the default, because in a training step the producer's input is "
                     "what the previous kernel wrote"}

    # ---- the reference's own kernels on this box (one GPU only; present when oracle/build_ref.sh was run) ----
    refs = load_reference_kernels() if world == 1 else {}
    ref_quant = None
    if "_tk_quant_v5" in refs:
        rq = refs["_tk_quant_v5"]
        ref_ms = _time_loop(torch, lambda i: rq.tk_fused_norm_quantize(xs[i % n_rot], gamma, EPS, False, True), 50, warm=5)
        ours_ms = _time_loop(torch, lambda i: tkq.tk_fused_norm_quantize(xs[i % n_rot], gamma, EPS, False, True), 50, warm=5)
        ref_quant = {"kernel": "reference tk_fused_norm_quantize (barrier-free branch, tk_quantize.cu:8048-8108), compiled "
                               "from the reference's sources for sm_100a", "ms": ref_ms,
                     "value": alg / (ref_ms * 1e-3) / 1e9, "unit": UNIT, "ours_ms_same_loop": ours_ms,
                     "ours_over_reference": ref_ms / ours_ms}
    ref_nv = None
    if "_tk_quant_v5" in refs:
        try:
            ref_nv = nvfp4_reference_producers_leg(torch, refs["_tk_quant_v5"], refs.get("_C"))
        except Exception as e:                       # the reference's kernels are evidence beside the line, never fatal
            ref_nv = {"error": str(e)[:300]}
        torch.cuda.empty_cache()
    ref_mx = None
    if "mxfp4_quant_v4" in refs:
        try:
            ref_mx = mxfp4_reference_producers_leg(torch, refs["mxfp4_quant_v4"], refs.get("_C_mx"))
        except Exception as e:                       # the reference's kernels are evidence beside the line, never fatal
            ref_mx = {"error": str(e)[:300]}
        torch.cuda.empty_cache()
    gemm_shapes, roofline_gemm = gemm_roofline_leg(torch, peaks, local_rank, world, refs, traffic)
    torch.cuda.empty_cache()
    cfg1 = config1_leg(torch, dev) if rank == 0 else None
    ffn = ffn_forward_leg(torch, dist, world, local_rank, xs[0], gamma, peaks)
    torch.cuda.empty_cache()
    ffn_bwd = ffn_backward_leg(torch, dist, world, xs[0], gamma, peaks)
    torch.cuda.empty_cache()
    mx_layer = mxfp4_layer_leg(torch, dist, world, gamma, peaks)
    torch.cuda.empty_cache()
    attn_side = attention_side_leg(torch, dist, world, peaks)

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_run(x_host, g_host)
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16->e2m1/e4m3 (fp32 scale math)", "data": "synthetic",
                "config": {"workload": WORKLOAD, "rows_per_gpu": M_ROWS, "cols": K_COLS,
                           "l2": "inputs rotate over 3 copies of X (402 MB > 126 MB L2) between steps",
                           "sharding": f"token dimension, {world} x [{M_ROWS}x{K_COLS}] per-rank batches, no collective"},
                "clocks": clocks, "e2e": e2e, "gpu_launches": 2 * args.steps, "roofline": roofline,
                "cpu_baseline": cpu, "strong_scaling_point": small, "with_early_reads_promise": early, "roofline_gemm": roofline_gemm,
                "gemm_shapes": gemm_shapes, "reference_kernels_same_box": {"fused_rmsnorm_nvfp4_quant": ref_quant, "nvfp4_producers": ref_nv,
                                                                            "mxfp4_producers": ref_mx,
                                                                            "load_errors": {k: v for k, v in refs.items() if k.endswith("_error")}},
                "config1_quantize_gemm": cfg1, "ffn_forward": ffn, "ffn_backward": ffn_bwd, "mxfp4_layer": mx_layer,
                "attention_side": attn_side}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def load_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernels the roofline blocks name,
    from the ncu captures: a small JSON kept beside the profile summaries, {} when it is missing."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}


if __name__ == "__main__":
    main()

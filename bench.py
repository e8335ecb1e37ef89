#!/usr/bin/env python
"""Benchmark of the W2A8 GEMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-sweeps]

Headline workload (every N): the Llama-3-70B fused gate+up projection, M=4096 tokens, N=57344, K=8192,
group 128, fp16 output; weights N-sharded over the ranks, fp16 output all-gathered ("strong" scaling: total work
fixed).  One step = one GEMM (+ all-gather when N > 1).  value = 2*M*N*K / time.  Outside the timed region every
rank compares sampled output columns of every rank's slice with the CPU oracle and the integer partial sums of a
sampled tile bit-exactly ("parity"); a failed check makes the run exit non-zero.  The down projection of the same
benchmark config (N=8192, K=28672) and the other exchange variant are reported under "config3".

At N=1 rank 0 additionally reports (outside the timed region) the decode sweep (Llama-2-7B shapes,
M in {1,4,8,16,32}, HBM GB/s over packed-weight + scale bytes) and the prefill sweep (M in {2048,4096,8192},
N=K=8192, int8 TOPS), and times the CPU restatement of the reference path on a bounded sample.

`--impl reference` times the reference's CPU route (unpack_matrix -> dequantize_from_uint2 -> fp32 matmul,
all host threads) on a bounded N-slab of the same workload; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "w2a8_gemm_tops"
UNIT = "TOPS"
WORKLOAD = dict(name="llama3_70b_gate_up_prefill", M=4096, N=57344, K=8192, G=128)
WORKLOAD_DOWN = dict(name="llama3_70b_down_prefill", M=4096, N=8192, K=28672, G=128)


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                        source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (a few ms per sample) while the timed region runs.
    Only reads: no clock, power or mode setting is touched."""

    def __init__(self, gpu_index: int, period_s: float = 0.005):
        self.gpu, self.period, self.samples, self._stop, self._t = gpu_index, period_s, [], False, None
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            idx = gpu_index
            if visible:
                try:
                    idx = int(visible.split(",")[gpu_index])
                except Exception:
                    idx = gpu_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(idx)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop:
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((sm, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()
        return self

    def __exit__(self, *a):
        self._stop = True
        if self._t is not None:
            self._t.join(timeout=1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        seen = set()
        for _, r in self.samples:
            for k, bit in names.items():
                if r & bit:
                    seen.add(k)
        sm = [s for s, _ in self.samples]
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(self.max_sm), "reasons": sorted(seen),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------------
# CPU restatement of the reference path (oracle), timed on the host cores
# --------------------------------------------------------------------------------------------------
def cpu_reference_step(x_q, x_scale, w_packed, w_scale, G):
    """unpack_matrix -> dequantize_from_uint2 -> fp32 matmul (torch, all threads).  Returns seconds."""
    import torch
    from oracle import w2a8_oracle as O
    t0 = time.perf_counter()
    codes = O.unpack_matrix(w_packed)
    wdq = O.dequantize_from_uint2(np.ascontiguousarray(codes.T), w_scale, G)
    xs = torch.from_numpy(x_q).float() * torch.from_numpy(x_scale)[:, None]
    y = xs @ torch.from_numpy(wdq).float()
    _ = y.to(torch.float16)
    return time.perf_counter() - t0


def cpu_sample(n_slab: int):
    from slimkernels_b200 import workloads as W
    M, K, G = WORKLOAD["M"], WORKLOAD["K"], WORKLOAD["G"]
    rng = np.random.default_rng(0)
    x_q, x_scale = W.make_activation(M, K, rng=rng)
    w_packed = rng.integers(0, 256, size=(n_slab, K // 4), dtype=np.uint8)
    w_scale = rng.uniform(0.001, 0.01, size=(K // G, n_slab)).astype(np.float16)
    return x_q, x_scale, w_packed, w_scale


def run_cpu_baseline(n_slab=2048, reps=2):
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    x_q, x_scale, w_packed, w_scale = cpu_sample(n_slab)
    best = min(cpu_reference_step(x_q, x_scale, w_packed, w_scale, WORKLOAD["G"]) for _ in range(reps))
    ops = 2.0 * WORKLOAD["M"] * n_slab * WORKLOAD["K"]
    return {"value": ops / best / 1e12, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "seconds_per_sample": best,
            "sample": f"M={WORKLOAD['M']} x N-slab {n_slab} of {WORKLOAD['N']} x K={WORKLOAD['K']}: "
                      f"unpack_matrix + dequantize_from_uint2 (numpy) + fp32 matmul (torch, {cores} threads), best of {reps}"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_slab = 1024
    x_q, x_scale, w_packed, w_scale = cpu_sample(n_slab)
    for _ in range(args.warmup):
        cpu_reference_step(x_q, x_scale, w_packed, w_scale, WORKLOAD["G"])
    t = [cpu_reference_step(x_q, x_scale, w_packed, w_scale, WORKLOAD["G"]) for _ in range(args.steps)]
    total = sum(t)
    ops = 2.0 * WORKLOAD["M"] * n_slab * WORKLOAD["K"] * args.steps
    value = ops / total / 1e12
    sample = (f"each step = M={WORKLOAD['M']} x N-slab {n_slab} of {WORKLOAD['N']} x K={WORKLOAD['K']}, reference CPU route "
              f"(unpack_matrix + dequantize_from_uint2 in numpy, fp32 matmul in torch) restated in oracle/")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": config_dict(args.gpus),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def config_dict(n_gpus, fused=True):
    how = "peer stores in the GEMM epilogue over NVLink" if fused else "NCCL all_gather after the GEMM"
    return {"workload": f"{WORKLOAD['name']}: M={WORKLOAD['M']} N={WORKLOAD['N']} K={WORKLOAD['K']} G={WORKLOAD['G']} "
                        f"int8 x 2-bit -> fp16, seed 0 synthetic (benchmark config 3, gate+up)",
            "parallelism": (f"N-sharded x{n_gpus}, output all-gathered ({how}; --nccl-gather selects the NCCL "
                            f"exchange)") if n_gpus > 1 else "single GPU",
            "l2": "inputs larger than L2 (weights 117 MB + activations 34 MB + output 470 MB per step)"}


# --------------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------------
def time_events(fn, iters, stream):
    import torch
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record(stream)
    for _ in range(iters):
        fn()
    e.record(stream)
    e.synchronize()
    return s.elapsed_time(e) / iters   # ms


def decode_sweep(dev, peaks):
    """Llama-2-7B decode shapes (and the two Llama-3-70B MLP projections at decode size): CUDA graph of 64 GEMMs
    cycling weight copies that total > 2x L2."""
    import torch
    from slimkernels_b200 import workloads as W
    from slimkernels_b200.torch import W2A8Plan
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    out = []
    rng = np.random.default_rng(0)
    shapes = dict(W.LLAMA2_7B_SHAPES)
    shapes.update({"llama3_70b_gate_up": (57344, 8192), "llama3_70b_down": (8192, 28672)})
    for name, (N, K) in shapes.items():
        G = 128
        wbytes = N * K // 4 + (K // G) * N * 2
        ncopies = min(64, max(2, int(np.ceil(2.0 * l2 / wbytes)) + 1))
        plans = []
        for _ in range(ncopies):
            wp = torch.from_numpy(rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)).to(dev)
            ws = torch.from_numpy(rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)).to(dev)
            wt = torch.ops.slimkernels.w2a8_repack(wp)
            torch.cuda.synchronize(dev)
            plans.append(W2A8Plan(wt, ws, N=N, K=K, group_size=G, tiled=True))
            del wp
        for M in W.DECODE_M:
            x_q = torch.from_numpy(rng.integers(-127, 128, size=(M, K), dtype=np.int8)).to(dev)
            xs = torch.from_numpy(rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)).to(dev)
            outs = [torch.empty(M, N, dtype=torch.float16, device=dev) for _ in range(2)]
            calls = 64
            st = torch.cuda.Stream(dev)
            with torch.cuda.stream(st):
                for i in range(min(ncopies, 4)):
                    plans[i].gemm(x_q, xs, out=outs[i % 2])
                st.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    for i in range(calls):
                        plans[i % ncopies].gemm(x_q, xs, out=outs[i % 2])
                for _ in range(3):
                    g.replay()
                st.synchronize()
                ms_graph = time_events(g.replay, 10, st) / calls
                # single launches of one plan, back to back (L2-warm, launch-bound): reported for context
                ms_single = time_events(lambda: plans[0].gemm(x_q, xs, out=outs[0]), 50, st)
                # the floor of this launch geometry: the same chain with an empty kernel (same grid, cluster, block,
                # shared memory, dependent launch; barrier set-up, tensor-memory allocation, the barriers; no bytes)
                for i in range(4):
                    plans[i % ncopies].launch_floor_probe(M)
                st.synchronize()
                gf = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gf, stream=st):
                    for i in range(calls):
                        plans[i % ncopies].launch_floor_probe(M)
                for _ in range(3):
                    gf.replay()
                st.synchronize()
                ms_floor = time_events(gf.replay, 10, st) / calls
            us = ms_graph * 1e3
            us_floor = ms_floor * 1e3
            gbs = wbytes / (ms_graph * 1e-3) / 1e9
            stream_us = wbytes / (peaks["hbm_gbs"] * 1e9) * 1e6
            desc, q = kernel_description(plans[0], M)
            out.append({"shape": name, "N": N, "K": K, "M": M, "us": round(us, 3), "gbs": round(gbs, 1),
                        "frac_hbm": round(gbs / peaks["hbm_gbs"], 4), "us_single_launch_l2_warm": round(ms_single * 1e3, 3),
                        "us_launch_floor": round(us_floor, 3),
                        "us_streaming_at_peak": round(stream_us, 3),
                        "gbs_above_floor": round(wbytes / max(us - us_floor, 1e-3) / 1e3, 1),
                        "frac_hbm_ceiling_floor_plus_streaming": round(stream_us / (us_floor + stream_us), 4),
                        "weight_copies": ncopies, "algorithmic_bytes": wbytes,
                        "kernel": desc})
        del plans
        torch.cuda.empty_cache()
    return out


def side_kernels_sweep(dev, peaks):
    """The HBM-bound kernels either side of the GEMM (Llama-3-70B MLP block shapes): weight preparation, per-token
    int8 quantiser, fused SiLU*up re-quantiser.  GB/s over the bytes each must move, against the measured HBM peak;
    buffers are larger than L2 or cycled so that every pass streams from HBM."""
    import torch
    from slimkernels_b200.torch import prepare_weight_gpu, quantize_activation_int8, silu_mul_quantize_int8
    out = []
    st = torch.cuda.current_stream(dev)
    gen = torch.Generator(device=dev)
    gen.manual_seed(0)

    def add(name, shape, fn, nbytes, iters):
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        ms = time_events(fn, iters, st)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.append({"kernel": name, "shape": shape, "us": round(ms * 1e3, 2), "gbs": round(gbs, 1),
                    "frac_hbm": round(gbs / peaks["hbm_gbs"], 4), "algorithmic_bytes": nbytes})

    K, N, G = 8192, 28672, 128                                   # one Llama-3-70B gate (or up) projection
    w = torch.randn(K, N, device=dev, dtype=torch.float32, generator=gen) * 0.02
    add("quantize_pack_weight_kernel", f"W float32 [{K}, {N}] G={G}", lambda: prepare_weight_gpu(w, G),
        4 * K * N + K * N // 4 + 6 * (K // G) * N, 5)
    del w
    M, H, I = 8192, 8192, 28672
    x = torch.randn(M, H, device=dev, dtype=torch.float16, generator=gen)
    add("quantize_activation_kernel", f"x float16 [{M}, {H}]", lambda: quantize_activation_int8(x), 3 * M * H + 4 * M, 10)
    del x
    M = 2048
    gu = torch.randn(M, 2 * I, device=dev, dtype=torch.float16, generator=gen)
    add("silu_mul_quantize_kernel", f"gate_up float16 [{M}, {2 * I}]", lambda: silu_mul_quantize_int8(gu),
        4 * M * I + M * I + 4 * M, 10)
    del gu
    torch.cuda.empty_cache()
    return out


def mlp_block_sweep(dev, peaks):
    """Benchmark config 4: the Llama-2-7B MLP block (hidden 4096, intermediate 11008) through W2A8LlamaMLP: token
    quantiser, fused gate+up GEMM, SiLU*up + re-quantiser, down GEMM (four launches), fp16 in and out.  Also the
    Llama-3-70B down projection of config 3 on one GPU (M=4096, N=8192, K=28672)."""
    import torch
    from slimkernels_b200.torch import W2A8Linear, W2A8LlamaMLP, W2A8Plan
    rng = np.random.default_rng(0)
    H, I, G = 4096, 11008, 128
    st = torch.cuda.current_stream(dev)

    def rand_linear(N, K):
        wp = torch.from_numpy(rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)).to(dev)
        ws = torch.from_numpy(rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)).to(dev)
        return W2A8Linear(wp, ws, group_size=G)

    wbytes = (2 * I * H + H * I) // 4 + ((H // G) * 2 * I + (I // G) * H) * 2
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    ncopies = max(2, int(np.ceil(2.0 * l2 / wbytes)) + 1)
    mlps = [W2A8LlamaMLP(rand_linear(2 * I, H), rand_linear(H, I)) for _ in range(ncopies)]
    mlp = mlps[0]
    out = {"block": [], "llama3_70b_down": None,
           "note": "four launches per call (token quantiser, gate+up GEMM, SiLU*up re-quantiser, down GEMM) chained by "
                   "programmatic dependent launch; M <= 16 also with COLD weights: a CUDA graph of calls cycling "
                   f"{ncopies} copies of the block's weights ({wbytes} bytes each, > 2 x L2 together)"}
    for M in (1, 16, 512, 4096):
        x = torch.randn(M, H, device=dev, dtype=torch.float16)
        for _ in range(3):
            mlp(x)
        torch.cuda.synchronize(dev)
        ms = time_events(lambda: mlp(x), 30 if M <= 512 else 10, st)
        ops = 6.0 * M * H * I
        row = {"M": M, "us": round(ms * 1e3, 2), "tops": round(ops / (ms * 1e-3) / 1e12, 2),
               "weight_gbs_l2_warm": round(wbytes / (ms * 1e-3) / 1e9, 1)}
        if M <= 16:
            stc = torch.cuda.Stream(dev)
            with torch.cuda.stream(stc):
                for m_ in mlps:
                    m_(x)
                stc.synchronize()
                g = torch.cuda.CUDAGraph()
                calls = 2 * ncopies
                with torch.cuda.graph(g, stream=stc):
                    for i in range(calls):
                        mlps[i % ncopies](x)
                for _ in range(3):
                    g.replay()
                stc.synchronize()
                ms_cold = time_events(g.replay, 10, stc) / calls
            gbs = wbytes / (ms_cold * 1e-3) / 1e9
            row.update({"us_cold_weights": round(ms_cold * 1e3, 2), "weight_gbs_cold": round(gbs, 1),
                        "frac_hbm_cold": round(gbs / peaks["hbm_gbs"], 4)})
        out["block"].append(row)
    del mlps
    del mlp
    N, K, M = 8192, 28672, 4096
    lin = rand_linear(N, K)
    x_q = torch.from_numpy(rng.integers(-127, 128, size=(M, K), dtype=np.int8)).to(dev)
    xs = torch.from_numpy(rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)).to(dev)
    y = torch.empty(M, N, dtype=torch.float16, device=dev)
    plan = lin.plan()
    for _ in range(3):
        plan.gemm(x_q, xs, out=y)
    torch.cuda.synchronize(dev)
    ms = time_events(lambda: plan.gemm(x_q, xs, out=y), 10, st)
    tops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
    out["llama3_70b_down"] = {"M": M, "N": N, "K": K, "us": round(ms * 1e3, 2), "tops": round(tops, 1),
                              "frac_of_2x_bf16_burst": round(tops / (2 * peaks["bf16_tflops"]), 4)}
    del lin, plan
    torch.cuda.empty_cache()
    return out


def prefill_sweep(dev, peaks):
    import torch
    from slimkernels_b200 import workloads as W
    from slimkernels_b200.torch import W2A8Plan
    rng = np.random.default_rng(0)
    N, K = W.PREFILL_NK
    G = 128
    wp = torch.from_numpy(rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)).to(dev)
    ws = torch.from_numpy(rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)).to(dev)
    plan = W2A8Plan(wp, ws, group_size=G)
    out = []
    st = torch.cuda.current_stream(dev)
    for M in W.PREFILL_M:
        x_q = torch.from_numpy(rng.integers(-127, 128, size=(M, K), dtype=np.int8)).to(dev)
        xs = torch.from_numpy(rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)).to(dev)
        y = torch.empty(M, N, dtype=torch.float16, device=dev)
        for _ in range(3):
            plan.gemm(x_q, xs, out=y)
        torch.cuda.synchronize(dev)
        ms = time_events(lambda: plan.gemm(x_q, xs, out=y), 20, st)
        tops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        out.append({"M": M, "N": N, "K": K, "us": round(ms * 1e3, 2), "tops": round(tops, 1),
                    "frac_of_2x_bf16_burst": round(tops / (2 * peaks["bf16_tflops"]), 4),
                    "frac_of_2x_bf16_sustained": round(tops / (2 * peaks["bf16_tflops_sustained"]), 4),
                    "frac_of_nominal_4500": round(tops / 4500.0, 4)})
    # library int8 GEMM on the same box, for context (cuBLASLt through torch._int_mm): not our kernel
    try:
        a = torch.randint(-127, 127, (8192, 8192), dtype=torch.int8, device=dev)
        b = torch.randint(-2, 2, (8192, 8192), dtype=torch.int8, device=dev).t()
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize(dev)
        ms = time_events(lambda: torch._int_mm(a, b), 20, st)
        lib_tops = 2.0 * 8192 ** 3 / (ms * 1e-3) / 1e12
    except Exception:
        lib_tops = None
    return out, lib_tops


def kernel_description(plan, M):
    """Names the kernel the plan launches for M tokens, from sk_w2a8_query_launch (nothing is assumed here)."""
    q = plan.query_launch(M)
    kind = {1: "w2a8_umma_kernel (tcgen05.mma kind::i8, weights expanded to int8 in shared memory)",
            2: "w2a8_simt_kernel (CUDA cores)",
            3: "w2a8_decode_kernel (tcgen05.mma kind::i8, weights expanded into tensor memory, split-K over a cluster)",
            5: "w2a8_stream_kernel (tcgen05.mma kind::i8, weights expanded into tensor memory, K range of the whole "
               "problem cut into equal CTA ranges)",
            4: "w2a8_pair_kernel (tcgen05.mma cta_group::2 kind::i8, two CTAs share one token tile)"}.get(q["kernel"], "?")
    return f"{kind}: token tile {q['token_tile']}, split-K {q['split_k']}, {q['ctas']} CTAs", q


def measured_traffic_ratio():
    """dram read bytes / algorithmic read bytes of the prefill kernel, from the ncu capture summarised under profiles/."""
    path = os.path.join(ROOT, "profiles", "w2a8_umma_prefill_M4096_N8192_K8192.json")
    try:
        d = json.load(open(path))
        return float(d["dram_bytes_read"]) / float(d["algorithmic_bytes_read"]), os.path.relpath(path, ROOT)
    except Exception:
        return None, None


def rank_weights(seed, rank, n_local, K, G):
    """The slice of rank `rank`: every rank can re-draw any rank's slice on the host (the parity check needs columns of
    all slices)."""
    rng = np.random.default_rng([seed, rank])
    wp = rng.integers(0, 256, size=(n_local, K // 4), dtype=np.uint8)
    ws = rng.uniform(0.001, 0.01, size=(K // G, n_local)).astype(np.float16)
    return wp, ws


def parity_check(y_full, x_q_np, x_scale_np, wl, world, rank, seed, plan_cls, dev, local_wp, local_ws, cols_total=64):
    """Outside the timed region: sampled output columns spread over every rank's slice against the CPU oracle (the
    reference route: unpack -> dequantise -> fp32 matmul), and the per-group int32 partial sums of one sampled
    128-feature tile x 256 tokens of this rank's slice bit-exactly."""
    import torch
    from oracle import w2a8_oracle as O
    M, N, K, G = wl["M"], wl["N"], wl["K"], wl["G"]
    n_local = N // world
    per = max(1, cols_total // world)
    rs = np.random.default_rng([seed, 1234])
    max_err, checked = 0.0, 0
    for q in range(world):
        wp_q, ws_q = rank_weights(seed, q, n_local, K, G)
        cols = np.sort(rs.choice(n_local, size=per, replace=False))
        ref = O.w2a8_gemm_dequant_path(x_q_np, x_scale_np, np.ascontiguousarray(wp_q[cols]),
                                       np.ascontiguousarray(ws_q[:, cols]), G)
        got = y_full[:, torch.from_numpy(q * n_local + cols).to(y_full.device)].float().cpu().numpy()
        max_err = max(max_err, float(np.abs(got - ref).max()))
        checked += per
        del wp_q, ws_q
    # integer partial sums of one tile of this rank's slice, through the same kernel variant (256-token tile)
    t0 = int(rs.integers(0, n_local // 128)) * 128
    rows = torch.arange(t0, t0 + 128, device=dev)
    sub = plan_cls(local_wp[rows].contiguous(), local_ws[:, rows].contiguous(), group_size=G)
    mt = min(M, 256)
    xq_d = torch.from_numpy(x_q_np[:mt]).to(dev)
    p = sub.partials(xq_d).cpu().numpy()
    wp_r, _ = rank_weights(seed, rank, n_local, K, G)
    p_ref = O.w2a8_partials(x_q_np[:mt], np.ascontiguousarray(wp_r[t0:t0 + 128]), G)
    exact = bool(np.array_equal(p, p_ref))
    return {"max_abs_err": max_err, "partials_exact": exact, "cols_checked": checked, "tol": 1e-2,
            "partials_checked": f"[{K // G} groups, {mt} tokens, features {rank * n_local + t0}..+128]"}


def measure_k_sharded(wl, seed, args, dev, world, rank, steps):
    """The down projection split along K (the layout a tensor-parallel MLP block needs behind an N-sharded gate+up):
    every rank multiplies its K slice, the partial sums are reduce-scattered by token rows.  Device-timed step (max
    over ranks) for the fused exchange (peer stores from the GEMM's epilogue) and for NCCL all-to-all after the GEMM;
    the two must agree bit for bit, and sampled columns of rank 0's rows are checked against the CPU oracle."""
    import torch
    import torch.distributed as dist
    from oracle import w2a8_oracle as O
    from slimkernels_b200.torch.sharded import KShardedW2A8Gemm
    M, N, K, G = wl["M"], wl["N"], wl["K"], wl["G"]
    per = K // world
    rows = M // world
    if K % (world * G) or M % world or rows % 256:
        return {"skipped": f"K={K} / M={M} do not split over {world} ranks in whole groups and 256-token tiles"}

    def k_slice(r):       # every rank can re-draw any rank's slice on the host (for the check)
        rng = np.random.default_rng([seed, 77, r])
        return (rng.integers(0, 256, size=(N, per // 4), dtype=np.uint8),
                rng.uniform(0.001, 0.01, size=(per // G, N)).astype(np.float16),
                rng.integers(-127, 128, size=(M, per), dtype=np.int8),
                rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32))

    wp_np, ws_np, xq_np, xs_np = k_slice(rank)
    wp, ws = torch.from_numpy(wp_np).to(dev), torch.from_numpy(ws_np).to(dev)
    d_x, d_xs = torch.from_numpy(xq_np).to(dev), torch.from_numpy(xs_np).to(dev)
    stream = torch.cuda.current_stream(dev)
    out = {"workload": wl["name"] + "_k_sharded", "M": M, "N": N, "K": K, "rows_per_rank": rows,
           "bytes_sent_per_rank": (world - 1) * rows * N * 2}
    results = {}
    for fused in (True, False):
        op = KShardedW2A8Gemm(wp, ws, group_size=G, fused=fused)
        for _ in range(3):
            y = op(d_x, d_xs)
        dist.barrier(); torch.cuda.synchronize(dev)
        ms = time_events(lambda: op(d_x, d_xs), steps, stream)
        dist.barrier(); torch.cuda.synchronize(dev)
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        results[fused] = op(d_x, d_xs).clone()
        out["fused_peer_stores" if fused else "nccl_all_to_all"] = {
            "ms_per_step": round(ms, 4), "tops": round(2.0 * M * N * K / (ms * 1e-3) / 1e12, 2)}
        del op
    same = torch.tensor([1 if torch.equal(results[True], results[False]) else 0], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    out["fused_equals_nccl_bitwise"] = bool(same.item())
    ok = True
    if rank == 0:
        cols = np.sort(np.random.default_rng([seed, 4321]).choice(N, size=32, replace=False))
        ref = np.zeros((rows, len(cols)), dtype=np.float32)
        for r in range(world):
            wp_r, ws_r, xq_r, xs_r = k_slice(r)
            ref += O.w2a8_gemm_dequant_path(xq_r[:rows], xs_r[:rows], np.ascontiguousarray(wp_r[cols]),
                                            np.ascontiguousarray(ws_r[:, cols]), G).astype(np.float32)
        err = float(np.abs(results[True].float().cpu().numpy()[:, cols] - ref).max())
        out["parity"] = {"max_abs_err": round(err, 6), "tol": 1e-2, "cols_checked": int(len(cols)), "rows_checked": rows,
                         "ok": bool(err <= 1e-2 and out["fused_equals_nccl_bitwise"])}
        ok = out["parity"]["ok"]
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.broadcast(flag, 0)
    out["_ok"] = bool(flag.item())
    del wp, ws, d_x, d_xs, results
    torch.cuda.empty_cache()
    return out


def measure_tp_mlp(seed, dev, world, rank, steps):
    """Llama-3-70B MLP block (hidden 8192, intermediate 28672, 4096 tokens) tensor-parallel over the ranks: gate+up
    split by output features, SiLU*up local, down split along K with the reduce-scatter fused into its epilogue (or
    NCCL all-to-all after it).  One exchange per block.  Device-timed, max over ranks; the two exchange variants must
    agree bit for bit (parity against the oracle is the 2-GPU unit test's job at a size the oracle can do)."""
    import torch
    import torch.distributed as dist
    from slimkernels_b200.torch.sharded import TensorParallelW2A8LlamaMLP
    M, H, I, G = 4096, 8192, 28672, 128
    per = I // world
    if I % (world * G) or M % world or (M // world) % 256:
        return {"skipped": f"intermediate {I} / tokens {M} do not split over {world} ranks in whole groups and tiles"}
    rng = np.random.default_rng([seed, 99, rank])
    t = lambda a: torch.from_numpy(a).to(dev)
    gl = t(rng.integers(0, 256, size=(2 * per, H // 4), dtype=np.uint8))
    gs = t(rng.uniform(0.001, 0.01, size=(H // G, 2 * per)).astype(np.float16))
    dl = t(rng.integers(0, 256, size=(H, per // 4), dtype=np.uint8))
    ds = t(rng.uniform(0.001, 0.01, size=(per // G, H)).astype(np.float16))
    x = t((np.random.default_rng([seed, 98]).standard_normal((M, H)) * 0.5).astype(np.float16))   # replicated
    stream = torch.cuda.current_stream(dev)
    ops = 2.0 * M * (2 * I * H + H * I)
    out = {"workload": "llama3_70b_mlp_block_tensor_parallel", "M": M, "hidden": H, "intermediate": I,
           "bytes_sent_per_rank": (world - 1) * (M // world) * H * 2,
           "launches_per_block": "quantise, gate+up GEMM, SiLU*up + re-quantise, down GEMM (+ reduce-scatter), fp32 sum of the partials"}
    res = {}
    for fused in (True, False):
        block = TensorParallelW2A8LlamaMLP(gl, gs, dl, ds, group_size=G, fused=fused)
        for _ in range(3):
            block(x)
        dist.barrier(); torch.cuda.synchronize(dev)
        ms = time_events(lambda: block(x), steps, stream)
        dist.barrier(); torch.cuda.synchronize(dev)
        tt = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
        res[fused] = block(x).clone()
        out["fused_peer_stores" if fused else "nccl_all_to_all"] = {"ms_per_block": round(ms, 4),
                                                                    "tops": round(ops / (ms * 1e-3) / 1e12, 2)}
        del block
    same = torch.tensor([1 if torch.equal(res[True], res[False]) else 0], device=dev)
    dist.all_reduce(same, op=dist.ReduceOp.MIN)
    out["fused_equals_nccl_bitwise"] = bool(same.item())
    out["finite"] = bool(torch.isfinite(res[True].float()).all().item())
    del gl, gs, dl, ds, x, res
    torch.cuda.empty_cache()
    return out


def measure_workload(wl, seed, args, dev, world, rank, fused, steps, peaks, with_e2e=False, with_parity=True):
    """One N-sharded GEMM (+ exchange) workload: device-timed step (max over ranks), this rank's GEMM alone (warmed,
    min / median / max over ranks), exchange figures, parity.  Returns a dict (same on every rank)."""
    import torch
    import torch.distributed as dist
    from slimkernels_b200 import workloads as W
    from slimkernels_b200.torch import W2A8Plan
    from slimkernels_b200.torch.sharded import ShardedW2A8Gemm, shard_bounds

    M, N, K, G = wl["M"], wl["N"], wl["K"], wl["G"]
    lo, hi = shard_bounds(N, world, rank)
    n_local = hi - lo
    wp_np, ws_np = rank_weights(seed, rank, n_local, K, G)
    wp, ws = torch.from_numpy(wp_np).to(dev), torch.from_numpy(ws_np).to(dev)
    del wp_np, ws_np
    x_q_np, x_scale_np = W.make_activation(M, K, seed=seed)        # replicated activations
    h_x = torch.from_numpy(x_q_np).pin_memory()
    h_xs = torch.from_numpy(x_scale_np).pin_memory()
    d_x, d_xs = h_x.to(dev), h_xs.to(dev)
    op = ShardedW2A8Gemm(wp, ws, N, group_size=G, fused=fused)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def over_ranks(ms):
        if world == 1:
            return ms, ms, ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        g = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(g, t)
        v = sorted(float(a.item()) for a in g)
        return v[0], v[len(v) // 2], v[-1]

    for _ in range(max(args.warmup, 3)):
        y = op(d_x, d_xs)
    barrier()
    with ClockSampler(dev.index) as clk:
        barrier()
        ms_step = time_events(lambda: op(d_x, d_xs), steps, stream)
        barrier()
    ms_step = over_ranks(ms_step)[2]
    clocks = clk.summary()
    res = {"workload": wl["name"], "M": M, "N": N, "K": K, "ms_per_step": round(ms_step, 4),
           "tops": round(2.0 * M * N * K / (ms_step * 1e-3) / 1e12, 2), "steps": steps, "clocks": clocks,
           "exchange": "none" if world == 1 else ("peer stores in the GEMM epilogue" if fused else "NCCL all-gather after the GEMM")}

    # this rank's GEMM alone: same plan, its own [M, N_local] buffer made and warmed BEFORE the timed loop
    for _ in range(3):
        op.local_gemm(d_x, d_xs)
    barrier()
    ms_g = time_events(lambda: op.local_gemm(d_x, d_xs), steps, stream)
    barrier()
    g_min, g_med, g_max = over_ranks(ms_g)
    desc, q = kernel_description(op.plan, M)
    res["gemm_only"] = {"ms_min": round(g_min, 4), "ms_median": round(g_med, 4), "ms_max": round(g_max, 4),
                        "tops_whole_job": round(2.0 * M * N * K / (g_max * 1e-3) / 1e12, 2), "kernel": desc}
    res["_launch"] = q
    res["_ms_kernel"] = g_max if world > 1 else ms_step
    res["_n_local"] = n_local

    if world > 1:
        sent = (world - 1) * M * n_local * 2                       # bytes this rank must deliver to (and receive from) its peers
        # link peak measured in the same run: NCCL all-gather of the same bytes (bus bandwidth = bytes received per
        # rank / time = the per-direction rate the links sustain for this exchange pattern)
        src = torch.empty(M, n_local, dtype=torch.float16, device=dev)
        dst = torch.empty(world * M, n_local, dtype=torch.float16, device=dev)
        for _ in range(3):
            dist.all_gather_into_tensor(dst, src)
        barrier()
        ms_ag = over_ranks(time_events(lambda: dist.all_gather_into_tensor(dst, src), max(5, steps // 2), stream))[2]
        barrier()
        peak_gbs = sent / (ms_ag * 1e-3) / 1e9
        del src, dst
        link_bound_ms = sent / (peak_gbs * 1e9) * 1e3
        bound_ms = max(link_bound_ms, g_max)
        res["exchange_figures"] = {
            "bytes_sent_per_rank": sent, "bytes_received_per_rank": sent,
            "achieved_gbs_per_direction": round(sent / (ms_step * 1e-3) / 1e9, 1),
            "link_peak_gbs_per_direction_measured": round(peak_gbs, 1),
            "link_peak_how": f"NCCL all_gather_into_tensor of the same {sent} received bytes per rank in this run: {round(ms_ag, 4)} ms",
            "link_bound_ms": round(link_bound_ms, 4), "gemm_bound_ms": round(g_max, 4),
            "step_over_bound": round(ms_step / bound_ms, 3),
            "frac_of_bound": round(bound_ms / ms_step, 4),
            "note": "a gather that lands the whole [M, N] on every rank cannot finish before max(link_bound_ms, gemm_bound_ms)"}

    if with_parity:
        y = op(d_x, d_xs)
        torch.cuda.synchronize(dev)
        par = parity_check(y, x_q_np, x_scale_np, wl, world, rank, seed, W2A8Plan, dev, wp, ws,
                           cols_total=64 if K <= 8192 else 32)
        if world > 1:
            t = torch.tensor([par["max_abs_err"], 0.0 if par["partials_exact"] else 1.0], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            par["max_abs_err"], par["partials_exact"] = float(t[0].item()), bool(t[1].item() == 0.0)
            par["ranks_checked"] = world
        par["max_abs_err"] = round(par["max_abs_err"], 6)
        par["ok"] = bool(par["max_abs_err"] <= par["tol"] and par["partials_exact"])
        res["parity"] = par

    if with_e2e:
        h_out = torch.empty(M, n_local, dtype=torch.float16).pin_memory()

        def e2e_step():
            if world == 1:
                op.plan.gemm_host(h_x, h_xs, h_out)   # the host-buffer call of the public API: copies and GEMM chunks overlap
                return
            d_x.copy_(h_x, non_blocking=True)
            d_xs.copy_(h_xs, non_blocking=True)
            yy = op(d_x, d_xs)
            h_out.copy_(yy[:, lo:hi], non_blocking=True)

        for _ in range(2):
            e2e_step()
        barrier()
        e2e_steps = max(2, min(steps, 10))
        ms_e2e = over_ranks(time_events(e2e_step, e2e_steps, stream))[2]
        barrier()
        res["e2e"] = {"value": round(2.0 * M * N * K / (ms_e2e * 1e-3) / 1e12, 3), "unit": UNIT,
                      "h2d_bytes_per_step": int(world * (h_x.numel() + h_xs.numel() * 4)),
                      "d2h_bytes_per_step": int(M * N * 2), "ms_per_step": round(ms_e2e, 4),
                      "note": "per step: activations H2D from pinned memory on every rank, GEMM (+ all-gather), each rank's "
                              "output slice D2H; on one GPU through W2A8Plan.gemm_host (token chunks, copies and GEMMs "
                              "overlapped on three streams)"}
        del h_out
    del op, wp, ws, d_x, d_xs, h_x, h_xs
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import torch
    import torch.distributed as dist
    from slimkernels_b200.torch import load_extension

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device visible; the W2A8 path has no CPU fallback")
    load_extension()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py: --gpus N > 1 must be launched with torch.distributed.run")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = read_peaks()
    fused = world > 1 and not args.nccl_gather

    # ---- headline workload: timed region of K steps with device-resident inputs, then e2e and parity
    head = measure_workload(WORKLOAD, 0, args, dev, world, rank, fused, args.steps, peaks, with_e2e=True)
    M, N, K, G = WORKLOAD["M"], WORKLOAD["N"], WORKLOAD["K"], WORKLOAD["G"]
    n_local = head["_n_local"]
    ms_kernel = head["_ms_kernel"]
    tops_kernel = 2.0 * M * n_local * K / (ms_kernel * 1e-3) / 1e12
    peak_int8 = 2.0 * peaks["bf16_tflops"]
    alg_read = n_local * K // 4 + (K // G) * n_local * 2 + M * K + M * 4
    alg_write = M * n_local * 2
    ratio, ratio_src = measured_traffic_ratio()
    traffic = int((ratio or 1.0) * alg_read + alg_write)
    roofline = {"bound": "tensor", "achieved": round(tops_kernel, 2), "peak": round(peak_int8, 1), "unit": "TOP/s",
                "frac": round(tops_kernel / peak_int8, 4), "traffic": traffic,
                "traffic_how": {"algorithmic_bytes_read": alg_read, "algorithmic_bytes_write": alg_write,
                                "measured_read_over_algorithmic": ratio, "from": ratio_src,
                                "note": "dram bytes of the ncu capture of the M=4096 N=K=8192 case, scaled by the bytes this "
                                        "launch moves (this workload is too large to capture); writes counted once"},
                "kernel": head["gemm_only"]["kernel"], "ms_per_launch": round(ms_kernel, 4),
                "ms_per_launch_over_ranks": {k: head["gemm_only"][k] for k in ("ms_min", "ms_median", "ms_max")},
                "peak_note": f"2 x {peaks['source']} bf16 burst TFLOP/s (no int8 figure is measured on this pool); "
                             f"vs 2 x sustained: {round(tops_kernel / (2 * peaks['bf16_tflops_sustained']), 4)}; "
                             f"vs nominal 4500: {round(tops_kernel / 4500.0, 4)}",
                "algorithmic_ops_per_launch": 2.0 * M * n_local * K}

    line = {"metric": METRIC, "value": head["tops"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 x int2 -> int32 -> fp32 scale -> fp16",
            "data": "synthetic", "config": config_dict(world, fused), "clocks": head["clocks"], "e2e": head["e2e"],
            "gpu_launches": args.steps, "roofline": roofline, "peaks": peaks, "parity": head["parity"],
            "gemm_only": head["gemm_only"]}
    if world > 1:
        line["exchange"] = head["exchange_figures"]

    def strip(d):
        return {k: v for k, v in d.items() if not k.startswith("_")}

    # ---- the other GEMM of benchmark config 3 (down projection, N-sharded the same way), the other exchange, and
    # the down projection split along K with the reduce-scatter fused into the GEMM's epilogue
    k_sharded_ok = True
    if not args.no_sweeps or world > 1:
        few = max(3, min(args.steps, 10))
        extra = {}
        def guarded(name, fn):
            # an extra workload that raises (the same way on every rank: shapes, memory) is reported, not fatal: the
            # headline measurement above stands by itself
            try:
                return fn()
            except Exception as exc:            # noqa: BLE001
                return {"error": f"{name}: {type(exc).__name__}: {exc}"[:400]}

        extra["down_proj"] = guarded("down_proj", lambda: strip(
            measure_workload(WORKLOAD_DOWN, 1, args, dev, world, rank, fused, few, peaks)))
        if world > 1:
            extra["gate_up_other_exchange"] = guarded("gate_up_other_exchange", lambda: strip(
                measure_workload(WORKLOAD, 0, args, dev, world, rank, not fused, few, peaks)))
            extra["down_proj_other_exchange"] = guarded("down_proj_other_exchange", lambda: strip(
                measure_workload(WORKLOAD_DOWN, 1, args, dev, world, rank, not fused, few, peaks)))
            ks = guarded("down_proj_k_sharded", lambda: measure_k_sharded(WORKLOAD_DOWN, 2, args, dev, world, rank, few))
            k_sharded_ok = ks.pop("_ok", True)
            extra["down_proj_k_sharded"] = ks
            tp = guarded("mlp_block_tensor_parallel", lambda: measure_tp_mlp(3, dev, world, rank, few))
            k_sharded_ok = k_sharded_ok and tp.get("fused_equals_nccl_bitwise", True) and tp.get("finite", True)
            extra["mlp_block_tensor_parallel"] = tp
        line["config3"] = extra

    if world == 1 and not args.no_sweeps:
        line["decode_sweep"] = decode_sweep(dev, peaks)
        pre, lib_tops = prefill_sweep(dev, peaks)
        line["prefill_sweep"] = pre
        line["library_int8_gemm_tops_8192"] = None if lib_tops is None else round(lib_tops, 1)
        line["side_kernels"] = side_kernels_sweep(dev, peaks)
        line["mlp_block"] = mlp_block_sweep(dev, peaks)
    if world == 1 and rank == 0:
        line["cpu_baseline"] = run_cpu_baseline()
    ok = line["parity"]["ok"] and k_sharded_ok and \
        all(v.get("parity", {"ok": True})["ok"] for v in line.get("config3", {}).values())
    line["parity_all_ok"] = bool(ok)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("bench.py: parity check failed (see the \"parity\" keys of the line above)")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweeps", action="store_true", help="skip the decode / prefill sweeps at N=1")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="N>1: exchange the output with NCCL all-gather after the GEMM instead of peer stores in its epilogue")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

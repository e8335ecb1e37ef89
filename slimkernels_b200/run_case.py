"""Run one W2A8 GEMM shape a few times on cuda:0 and print its device time.

    python -m slimkernels_b200.run_case --M 2048 --N 8192 --K 8192 [--iters 5] [--token-tile 256] [--split-k 1]

Small, deterministic and quick: the command profilers are pointed at (one kernel, few launches).
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from . import capi
from .torch import W2A8Plan, load_extension


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--M", type=int, required=True)
    ap.add_argument("--N", type=int, required=True)
    ap.add_argument("--K", type=int, required=True)
    ap.add_argument("--G", type=int, default=128)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--token-tile", type=int, default=0)
    ap.add_argument("--split-k", type=int, default=0)
    ap.add_argument("--persistent", type=int, default=0, help="0 auto, 1 one CTA per tile, 2 resident CTAs walk the tiles")
    ap.add_argument("--weight-copies", type=int, default=1, help="cycle this many distinct weight buffers")
    args = ap.parse_args()
    load_extension()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(0)
    M, N, K, G = args.M, args.N, args.K, args.G
    plans = []
    for _ in range(args.weight_copies):
        wp = torch.from_numpy(rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)).to(dev)
        ws = torch.from_numpy(rng.uniform(0.001, 0.01, size=(K // G, N)).astype(np.float16)).to(dev)
        plan = W2A8Plan(wp, ws, group_size=G)
        plan.set_option(capi.SK_OPT_TOKEN_TILE, args.token_tile)
        plan.set_option(capi.SK_OPT_SPLIT_K, args.split_k)
        plan.set_option(capi.SK_OPT_PERSISTENT, args.persistent)
        plans.append(plan)
    x_q = torch.from_numpy(rng.integers(-127, 128, size=(M, K), dtype=np.int8)).to(dev)
    xs = torch.from_numpy(rng.uniform(0.005, 0.02, size=(M,)).astype(np.float32)).to(dev)
    out = torch.empty(M, N, dtype=torch.float16, device=dev)
    for i in range(args.warmup):
        plans[i % len(plans)].gemm(x_q, xs, out=out)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(args.iters):
        plans[i % len(plans)].gemm(x_q, xs, out=out)
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / args.iters
    assert plans[0].device_status() == 0
    wbytes = N * K // 4 + (K // G) * N * 2
    print(json.dumps({"M": M, "N": N, "K": K, "G": G, "us": round(ms * 1e3, 2),
                      "tops": round(2.0 * M * N * K / (ms * 1e-3) / 1e12, 1),
                      "weight_gbs": round(wbytes / (ms * 1e-3) / 1e9, 1), "checksum": float(out.float().sum())}))


if __name__ == "__main__":
    main()

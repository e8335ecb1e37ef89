"""N-sharded execution on CPU ranks (gloo, world size 2): slicing, all-gather and the [R, M, N/R] -> [M, N]
re-ordering, with the device GEMM replaced by the CPU oracle.  The CUDA GEMM itself is covered by the gpu tests."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


class OraclePlan:
    """Stand-in for W2A8Plan on CPU ranks: same call surface, computed by the oracle."""

    def __init__(self, w_packed, w_scale, group_size=128, zero_point=1, out_dtype=torch.float16):
        self.w_packed, self.w_scale, self.G, self.zp, self.dt = w_packed.numpy(), w_scale.numpy(), group_size, zero_point, out_dtype

    def gemm(self, x_q, x_scale, out=None):
        from oracle import w2a8_oracle as O
        y = torch.from_numpy(O.w2a8_gemm_int_path(x_q.numpy(), x_scale.numpy(), self.w_packed, self.w_scale, self.G, self.zp))
        if out is None:
            return y.to(self.dt)
        out.copy_(y.to(self.dt))
        return out


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200 import workloads as W
        from slimkernels_b200.torch.sharded import ShardedW2A8Gemm, shard_bounds, shard_weight
        M, N, K, G = 6, 512, 256, 128
        x_q, x_scale, w_packed, w_scale = W.make_problem(M, N, K, G, seed=0)
        lo, hi = shard_bounds(N, world, rank)
        assert (lo, hi) == (rank * N // world, (rank + 1) * N // world)
        wl, sl = shard_weight(torch.from_numpy(w_packed), torch.from_numpy(w_scale), world, rank)
        assert wl.is_contiguous() and sl.is_contiguous() and wl.shape == (N // world, K // 4) and sl.shape == (K // G, N // world)
        op = ShardedW2A8Gemm(wl, sl, N, group_size=G, plan_factory=OraclePlan)
        y = op(torch.from_numpy(x_q), torch.from_numpy(x_scale))
        ref = O.w2a8_gemm_int_path(x_q, x_scale, w_packed, w_scale, G).astype(np.float16)
        q.put((rank, bool(np.array_equal(y.numpy(), ref)), tuple(y.shape)))
    finally:
        dist.destroy_process_group()


def test_two_rank_shard_and_gather_on_cpu():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    for _, equal, shape in results:
        assert equal and shape == (6, 512)


def _worker_k(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200 import workloads as W
        from slimkernels_b200.torch.sharded import KShardedW2A8Gemm, shard_weight_k
        M, N, K, G = 8, 256, 512, 128
        x_q, _, w_packed, w_scale = W.make_problem(M, N, K, G, seed=1)
        rng = np.random.default_rng(7)
        scales = rng.uniform(0.005, 0.02, size=(world, M)).astype(np.float32)      # every rank quantised its own slice
        per = K // world
        wl, sl = shard_weight_k(torch.from_numpy(w_packed), torch.from_numpy(w_scale), world, rank, G)
        assert wl.shape == (N, per // 4) and sl.shape == (per // G, N) and wl.is_contiguous() and sl.is_contiguous()
        op = KShardedW2A8Gemm(wl, sl, group_size=G, plan_factory=OraclePlan)
        xl = torch.from_numpy(np.ascontiguousarray(x_q[:, rank * per:(rank + 1) * per]))
        mine = op(xl, torch.from_numpy(scales[rank]))
        full = op.forward_full(xl, torch.from_numpy(scales[rank]))
        ref = sum(O.w2a8_gemm_int_path(np.ascontiguousarray(x_q[:, r * per:(r + 1) * per]), scales[r],
                                       np.ascontiguousarray(w_packed[:, r * per // 4:(r + 1) * per // 4]),
                                       w_scale[r * per // G:(r + 1) * per // G], G) for r in range(world))
        rows = M // world
        err_mine = float(np.abs(mine.float().numpy() - ref[rank * rows:(rank + 1) * rows]).max())
        err_full = float(np.abs(full.float().numpy() - ref).max())
        q.put((rank, err_mine, err_full, tuple(mine.shape), tuple(full.shape)))
    finally:
        dist.destroy_process_group()


def test_two_rank_k_sharded_reduce_scatter_on_cpu():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_k, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    for _, err_mine, err_full, shape_mine, shape_full in results:
        assert shape_mine == (4, 256) and shape_full == (8, 256)
        assert err_mine <= 1e-2 and err_full <= 1e-2      # partials travel in fp16, the sum runs in fp32


def test_shard_bounds_rejects_ragged_split():
    from slimkernels_b200.torch.sharded import shard_bounds
    with pytest.raises(ValueError):
        shard_bounds(4096 + 128, 8, 0)
    assert shard_bounds(57344, 8, 7) == (50176, 57344)
    assert shard_bounds(8192, 8, 3) == (3072, 4096)


# --------------------------------------------------------------------------------------------------
# Failure behaviour, made on the host: a rank that arrives late, and a rank that never takes part.
# --------------------------------------------------------------------------------------------------
def _worker_fail(rank, world, port, q, mode):
    """mode 'late': rank 1 joins the exchange 1 s late (inside the limit).  mode 'missing': rank 1 never calls the
    op.  mode 'liveness': as 'missing', noticed by the control group's barrier before anything is launched."""
    import time
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from slimkernels_b200 import workloads as W
    from slimkernels_b200.torch.sharded import ExchangeTimeout, ShardedW2A8Gemm, shard_weight
    M, N, K, G = 6, 512, 256, 128
    x_q, x_scale, w_packed, w_scale = W.make_problem(M, N, K, G, seed=0)
    wl, sl = shard_weight(torch.from_numpy(w_packed), torch.from_numpy(w_scale), world, rank)
    limit = 20.0 if mode == "late" else 1.5
    control = dist.new_group(backend="gloo") if mode == "liveness" else None
    op = ShardedW2A8Gemm(wl, sl, N, group_size=G, plan_factory=OraclePlan, exchange_timeout_s=limit,
                         control_group=control)
    xq, xs = torch.from_numpy(x_q), torch.from_numpy(x_scale)
    out = None
    if mode == "late":
        if rank == 1:
            time.sleep(1.0)
        y = op(xq, xs)
        out = (rank, "ok", tuple(y.shape), 0.0)
    elif rank == 1:
        time.sleep(6.0)                       # alive on the host, but never joins the exchange
        out = (rank, "absent", (), 0.0)
    else:
        t0 = time.perf_counter()
        try:
            op(xq, xs)
            out = (rank, "no error", (), time.perf_counter() - t0)
        except ExchangeTimeout as exc:
            ok = exc.rank == 0 and exc.step == 0 and exc.limit_s == limit and "step 0" in str(exc)
            out = (rank, "timeout" if ok else f"bad exception fields: {exc}", (exc.what,), time.perf_counter() - t0)
    q.put(out)
    q.close()
    q.join_thread()
    os._exit(0)      # the group is unusable after an expired wait: leave without the collective teardown


def _run_fail(mode):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_fail, args=(r, world, port, q, mode)) for r in range(world)]
    for p in procs:
        p.start()
    results = dict((r[0], r) for r in (q.get(timeout=90) for _ in range(world)))
    for p in procs:
        p.join(timeout=60)
    return results


def test_late_rank_still_completes_inside_the_limit():
    res = _run_fail("late")
    assert res[0][1] == "ok" and res[1][1] == "ok" and res[0][2] == (6, 512)


def test_missing_rank_surfaces_as_exchange_timeout():
    res = _run_fail("missing")
    assert res[0][1] == "timeout", res[0]
    assert "all-gather" in res[0][2][0]
    assert 1.0 <= res[0][3] < 5.5, f"the error took {res[0][3]:.1f} s to surface (limit 1.5 s)"


def test_missing_rank_is_noticed_by_the_liveness_barrier_before_the_launch():
    res = _run_fail("liveness")
    assert res[0][1] == "timeout", res[0]
    assert "liveness" in res[0][2][0]
    assert res[0][3] < 5.5


def test_shard_gate_up_keeps_gate_and_up_rows_of_the_same_features_together():
    from slimkernels_b200.torch.sharded import shard_gate_up
    inter, world = 8, 4
    packed = torch.arange(2 * inter * 3, dtype=torch.uint8).view(2 * inter, 3)
    scale = torch.arange(2 * 2 * inter, dtype=torch.float16).view(2, 2 * inter)
    gates, ups = [], []
    for r in range(world):
        p_l, s_l = shard_gate_up(packed, scale, world, r)
        per = inter // world
        assert p_l.shape == (2 * per, 3) and s_l.shape == (2, 2 * per)
        gates.append(p_l[:per]); ups.append(p_l[per:])
        assert torch.equal(s_l[:, :per], scale[:, r * per:(r + 1) * per])
        assert torch.equal(s_l[:, per:], scale[:, inter + r * per:inter + (r + 1) * per])
    assert torch.equal(torch.cat(gates), packed[:inter]) and torch.equal(torch.cat(ups), packed[inter:])
    with pytest.raises(ValueError):
        shard_gate_up(packed, scale, 3, 0)


def _worker_tp(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200.torch.sharded import TensorParallelW2A8LlamaMLP, shard_gate_up, shard_weight_k
        M, H, I, G = 4, 256, 512, 128
        rng = np.random.default_rng(5)
        x = (rng.standard_normal((M, H)) * 0.5).astype(np.float16)
        gu_p = rng.integers(0, 256, size=(2 * I, H // 4), dtype=np.uint8)
        gu_s = rng.uniform(0.001, 0.01, size=(H // G, 2 * I)).astype(np.float16)
        dn_p = rng.integers(0, 256, size=(H, I // 4), dtype=np.uint8)
        dn_s = rng.uniform(0.001, 0.01, size=(I // G, H)).astype(np.float16)

        def quantize(t):                      # CPU stand-ins for the two activation kernels: the oracle's rules
            qv, sv = O.quantize_activation_int8(t.numpy())
            return torch.from_numpy(qv), torch.from_numpy(sv)

        def silu_mul_quantize(gate_up):
            gu = gate_up.numpy().astype(np.float32)
            inter = gu.shape[1] // 2
            g, u = gu[:, :inter], gu[:, inter:]
            return quantize(torch.from_numpy(((g / (1.0 + np.exp(-g))) * u).astype(np.float32)))

        gl, gs = shard_gate_up(torch.from_numpy(gu_p), torch.from_numpy(gu_s), world, rank)
        dl, ds = shard_weight_k(torch.from_numpy(dn_p), torch.from_numpy(dn_s), world, rank, G)
        block = TensorParallelW2A8LlamaMLP(gl, gs, dl, ds, group_size=G, fused=False, plan_factory=OraclePlan,
                                           activation_ops=(quantize, silu_mul_quantize))
        mine = block(torch.from_numpy(x))
        full = block.forward_full(torch.from_numpy(x))
        per = I // world
        ref = np.zeros((M, H), dtype=np.float32)
        for r in range(world):
            rows = np.concatenate([np.arange(r * per, (r + 1) * per), np.arange(I + r * per, I + (r + 1) * per)])
            part = O.llama_mlp(x, np.ascontiguousarray(gu_p[rows]), np.ascontiguousarray(gu_s[:, rows]),
                               np.ascontiguousarray(dn_p[:, r * per // 4:(r + 1) * per // 4]),
                               dn_s[r * per // G:(r + 1) * per // G], G)
            ref += part.astype(np.float16).astype(np.float32)
        mr = M // world
        q.put((rank, float(np.abs(mine.float().numpy() - ref[rank * mr:(rank + 1) * mr]).max()),
               float(np.abs(full.float().numpy() - ref).max()), tuple(mine.shape), tuple(full.shape)))
    finally:
        dist.destroy_process_group()


def test_two_rank_tensor_parallel_mlp_block_on_cpu():
    """The block's host logic (which rows of gate+up a rank owns, local SiLU*up with per-rank token scales, K-sharded
    down, reduce-scatter by token rows) on two gloo ranks, with the oracle standing in for every device kernel."""
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_tp, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, err_mine, err_full, shape_mine, shape_full in results:
        assert shape_mine == (2, 256) and shape_full == (4, 256)
        assert err_mine <= 1e-2 and err_full <= 1e-2

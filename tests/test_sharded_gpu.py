"""N-sharded W2A8 GEMM + all-gather and K-sharded GEMM + reduce-scatter on 2 GPUs (skipped where fewer are visible)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q, fused=False):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200 import workloads as W
        from slimkernels_b200.torch.sharded import ShardedW2A8Gemm, shard_weight
        M, N, K, G = 300, 1024, 512, 128
        x_q, x_scale, w_packed, w_scale = W.make_problem(M, N, K, G, seed=0)
        wl, sl = shard_weight(torch.from_numpy(w_packed).to(dev), torch.from_numpy(w_scale).to(dev), world, rank)
        op = ShardedW2A8Gemm(wl, sl, N, group_size=G, fused=fused)
        y = op(torch.from_numpy(x_q).to(dev), torch.from_numpy(x_scale).to(dev))
        torch.cuda.synchronize(dev)
        ref = O.w2a8_gemm_dequant_path(x_q, x_scale, w_packed, w_scale, G)
        q.put((rank, float(np.abs(y.float().cpu().numpy() - ref).max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", [False, True], ids=["nccl_allgather", "peer_store_epilogue"])
def test_two_gpu_shard_and_allgather(built_libs, fused):
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, fused)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, err in results:
        assert err <= 1e-2


def _worker_overlap(rank, world, port, q):
    """Fused exchange, three steps in a row with different activations: the result of step 1 is read on a SIDE stream
    while step 2 runs (two output buffers alternate, so step 2 writes elsewhere), and step 3 -- which reuses step 1's
    buffer -- is launched only after that reader is done."""
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200 import workloads as W
        from slimkernels_b200.torch.sharded import ShardedW2A8Gemm, shard_weight
        M, N, K, G = 512, 2048, 1024, 128
        _, _, w_packed, w_scale = W.make_problem(M, N, K, G, seed=0)
        wl, sl = shard_weight(torch.from_numpy(w_packed).to(dev), torch.from_numpy(w_scale).to(dev), world, rank)
        op = ShardedW2A8Gemm(wl, sl, N, group_size=G, fused=True)
        xs_np = [W.make_activation(M, K, seed=10 + i) for i in range(3)]
        xs = [(torch.from_numpy(a).to(dev), torch.from_numpy(b).to(dev)) for a, b in xs_np]
        refs = [O.w2a8_gemm_dequant_path(a, b, w_packed, w_scale, G) for a, b in xs_np]
        main, side = torch.cuda.current_stream(dev), torch.cuda.Stream(dev)
        errs = []
        for rep in range(4):                         # several rounds, so that the ranks drift apart if they can
            y1 = op(*xs[0])
            side.wait_stream(main)
            with torch.cuda.stream(side):
                c1 = y1.float() * 1.0                # the consumer of step 1, concurrent with step 2
            y2 = op(*xs[1])                          # other buffer
            c2 = y2.float() * 1.0
            main.wait_stream(side)                   # step 3 reuses step 1's buffer: order it behind the reader
            y3 = op(*xs[2])
            assert y3.data_ptr() == y1.data_ptr() and y2.data_ptr() != y1.data_ptr()
            c3 = y3.float() * 1.0
            torch.cuda.synchronize(dev)
            errs.append(max(float(np.abs(c.cpu().numpy() - r).max()) for c, r in zip((c1, c2, c3), refs)))
        q.put((rank, max(errs)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_fused_result_can_be_read_while_the_next_step_runs(built_libs):
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_overlap, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, err in results:
        assert err <= 1e-2


def _worker_k(rank, world, port, q, fused=False):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200 import workloads as W
        from slimkernels_b200.torch.sharded import KShardedW2A8Gemm, shard_weight_k
        M, N, K, G = (1024, 384, 2048, 128) if fused else (256, 512, 2048, 128)   # fused: M/R = 2 tiles of 256 tokens
        x_q, _, w_packed, w_scale = W.make_problem(M, N, K, G, seed=2)
        scales = np.random.default_rng(9).uniform(0.005, 0.02, size=(world, M)).astype(np.float32)
        per = K // world
        wl, sl = shard_weight_k(torch.from_numpy(w_packed).to(dev), torch.from_numpy(w_scale).to(dev), world, rank, G)
        op = KShardedW2A8Gemm(wl, sl, group_size=G, fused=fused)
        xl = torch.from_numpy(np.ascontiguousarray(x_q[:, rank * per:(rank + 1) * per])).to(dev)
        xs = torch.from_numpy(scales[rank]).to(dev)
        mine = op(xl, xs)
        full = op.forward_full(xl, xs)
        torch.cuda.synchronize(dev)
        if fused:
            # the fused exchange and the NCCL one add the same fp16 partials in the same order: bit-identical
            plain = KShardedW2A8Gemm(wl, sl, group_size=G)(xl, xs)
            assert torch.equal(mine, plain)
            assert torch.equal(op(xl, xs), mine) and torch.equal(op(xl, xs), mine)    # both receive buffers
        ref = sum(O.w2a8_gemm_dequant_path(np.ascontiguousarray(x_q[:, r * per:(r + 1) * per]), scales[r],
                                           np.ascontiguousarray(w_packed[:, r * per // 4:(r + 1) * per // 4]),
                                           w_scale[r * per // G:(r + 1) * per // G], G) for r in range(world))
        rows = M // world
        q.put((rank, float(np.abs(mine.float().cpu().numpy() - ref[rank * rows:(rank + 1) * rows]).max()),
               float(np.abs(full.float().cpu().numpy() - ref).max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("fused", [False, True])
def test_two_gpu_k_sharded_reduce_scatter(built_libs, fused):
    """K-sharded down-projection style GEMM: partial products on each GPU, reduce-scatter by token rows -- through
    NCCL after the GEMM, or (fused) by peer stores from the GEMM's epilogue into the owning rank's receive buffer."""
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_k, args=(r, world, port, q, fused)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, err_mine, err_full in results:
        assert err_mine <= 1e-2 and err_full <= 1e-2


def _worker_tp(rank, world, port, q):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import w2a8_oracle as O
        from slimkernels_b200.torch.sharded import TensorParallelW2A8LlamaMLP, shard_gate_up, shard_weight_k
        M, H, I, G = 512, 512, 1024, 128          # M/R = one 256-token tile, I/R = 512 = 4 groups of the down projection
        rng = np.random.default_rng(5)
        x = (rng.standard_normal((M, H)) * 0.5).astype(np.float16)
        gu_p = rng.integers(0, 256, size=(2 * I, H // 4), dtype=np.uint8)
        gu_s = rng.uniform(0.001, 0.01, size=(H // G, 2 * I)).astype(np.float16)
        dn_p = rng.integers(0, 256, size=(H, I // 4), dtype=np.uint8)
        dn_s = rng.uniform(0.001, 0.01, size=(I // G, H)).astype(np.float16)
        t = lambda a: torch.from_numpy(a).to(dev)
        gl, gs = shard_gate_up(t(gu_p), t(gu_s), world, rank)
        dl, ds = shard_weight_k(t(dn_p), t(dn_s), world, rank, G)
        outs = {}
        for fused in (True, False):
            block = TensorParallelW2A8LlamaMLP(gl, gs, dl, ds, group_size=G, fused=fused)
            outs[fused] = (block(t(x)).clone(), block.forward_full(t(x)).clone())
        torch.cuda.synchronize(dev)
        assert torch.equal(outs[True][0], outs[False][0]) and torch.equal(outs[True][1], outs[False][1])
        # reference: the single-GPU block of the oracle on every rank's slices, partials rounded to fp16, summed
        per = I // world
        ref = np.zeros((M, H), dtype=np.float32)
        for r in range(world):
            rows = np.concatenate([np.arange(r * per, (r + 1) * per), np.arange(I + r * per, I + (r + 1) * per)])
            part = O.llama_mlp(x, np.ascontiguousarray(gu_p[rows]), np.ascontiguousarray(gu_s[:, rows]),
                               np.ascontiguousarray(dn_p[:, r * per // 4:(r + 1) * per // 4]),
                               dn_s[r * per // G:(r + 1) * per // G], G)
            ref += part.astype(np.float16).astype(np.float32)
        mr = M // world
        mine, full = outs[True]
        q.put((rank, float(np.abs(mine.float().cpu().numpy() - ref[rank * mr:(rank + 1) * mr]).max()),
               float(np.abs(full.float().cpu().numpy() - ref).max()), float(np.abs(ref).max())))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpu_tensor_parallel_mlp_block(built_libs):
    """Llama MLP block over two GPUs with one exchange: gate+up split by features, SiLU*up local, down split along K
    with the reduce-scatter in its epilogue.  Checked against the oracle's block applied to each rank's slices."""
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_tp, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, err_mine, err_full, scale in results:
        assert err_mine <= 1e-2 * max(1.0, scale) and err_full <= 1e-2 * max(1.0, scale)

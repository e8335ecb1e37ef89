"""N-sharded W2A8 GEMM + NCCL all-gather on 2 GPUs (skipped where fewer are visible)."""
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

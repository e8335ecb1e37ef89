"""Sharded execution of one W2A8 GEMM across the GPUs of a node (one process per GPU): N-sharded with an all-gather
(ShardedW2A8Gemm) and K-sharded with a reduce-scatter (KShardedW2A8Gemm, for a projection whose input is already
split by features, like the down projection behind an N-sharded gate+up).

N-sharding:

Output features are independent, so rank r owns rows [r*N/R, (r+1)*N/R) of w_packed and the matching
columns of w_scale; activations are replicated; K is not split, so no reduction is needed.  The only
exchange is an all-gather of the fp16/bf16 output over NVLink (NCCL through torch.distributed).
The reference has no multi-GPU code; this is the one parallel strategy the W2A8 path needs.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .ops import W2A8Plan


def shard_bounds(N: int, world: int, rank: int, multiple: int = 128):
    """[lo, hi) of the output features rank owns: equal slices, which must be multiples of `multiple`."""
    if N % (world * multiple) != 0:
        raise ValueError(f"N={N} must be a multiple of world_size*{multiple}={world * multiple}")
    per = N // world
    return rank * per, (rank + 1) * per


def shard_weight(w_packed, w_scale, world: int, rank: int):
    """This rank's slice of (w_packed [N, K/4], w_scale [K/G, N]) as contiguous tensors."""
    lo, hi = shard_bounds(w_packed.shape[0], world, rank)
    return w_packed[lo:hi].contiguous(), w_scale[:, lo:hi].contiguous()


class ShardedW2A8Gemm:
    """Holds this rank's weight slice; ``forward`` returns the full [M, N] output on every rank."""

    def __init__(self, w_packed_local, w_scale_local, N_total: int, group=None, group_size=128, zero_point=1,
                 out_dtype=torch.float16, plan_factory=W2A8Plan, fused=False):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N_total = N_total
        self.N_local = w_packed_local.shape[0]
        assert self.N_local * self.world == N_total
        self.out_dtype = out_dtype
        # plan_factory exists so that the sharding / gathering logic can be exercised on CPU ranks (gloo) with a
        # stand-in for the device GEMM; the product default is the CUDA plan and nothing else
        self.plan = plan_factory(w_packed_local, w_scale_local, group_size=group_size, zero_point=zero_point,
                                 out_dtype=out_dtype)
        self._bufs = {}
        self.fused = bool(fused) and self.world > 1
        self._symm = {}

    def _buffers(self, M, device):
        key = (M, device)
        if key not in self._bufs:
            local = torch.empty(M, self.N_local, dtype=self.out_dtype, device=device)
            gathered = torch.empty(self.world, M, self.N_local, dtype=self.out_dtype, device=device)
            full = torch.empty(M, self.N_total, dtype=self.out_dtype, device=device)
            self._bufs[key] = (local, gathered, full)
        return self._bufs[key]

    def local_gemm(self, x_q, x_scale):
        local, _, _ = self._buffers(x_q.shape[0], x_q.device)
        return self.plan.gemm(x_q, x_scale, out=local)

    def _symmetric(self, M, device):
        """[M, N_total] output buffer in symmetric memory + the peers' pointers to it (this rank's first, then the
        others in ring order so that the ranks do not all write to the same peer at the same time)."""
        key = (M, device)
        if key not in self._symm:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group if self.group is not None else dist.group.WORLD
            buf = symm_mem.empty((M, self.N_total), dtype=self.out_dtype, device=device)
            hdl = symm_mem.rendezvous(buf, group)
            ptrs = [int(hdl.buffer_ptrs[(self.rank + i) % self.world]) for i in range(self.world)]
            self._symm[key] = (buf, hdl, ptrs)
        return self._symm[key]

    def forward_fused(self, x_q, x_scale):
        M = x_q.shape[0]
        buf, hdl, ptrs = self._symmetric(M, x_q.device)
        self.plan.gemm_scatter(x_q, x_scale, ptrs, self.N_total, self.rank * self.N_local)
        hdl.barrier()          # every rank's tiles have landed everywhere (stream-ordered device barrier)
        return buf

    def forward(self, x_q, x_scale):
        if self.fused:
            return self.forward_fused(x_q, x_scale)
        M = x_q.shape[0]
        local, gathered, full = self._buffers(M, x_q.device)
        self.plan.gemm(x_q, x_scale, out=local)
        if self.world == 1:
            return local
        dist.all_gather_into_tensor(gathered.view(self.world * M, self.N_local), local, group=self.group)
        # [R, M, N/R] -> [M, R, N/R] == [M, N]
        full.view(M, self.world, self.N_local).copy_(gathered.permute(1, 0, 2))
        return full

    __call__ = forward


def shard_weight_k(w_packed, w_scale, world: int, rank: int, group_size: int = 128):
    """This rank's K slice of (w_packed [N, K/4], w_scale [K/G, N]): in-features [r K/R, (r+1) K/R), whole groups."""
    K = w_packed.shape[1] * 4
    if K % (world * group_size) != 0:
        raise ValueError(f"K={K} must be a multiple of world_size*group_size={world * group_size}")
    per = K // world
    return (w_packed[:, rank * per // 4:(rank + 1) * per // 4].contiguous(),
            w_scale[rank * per // group_size:(rank + 1) * per // group_size].contiguous())


class KShardedW2A8Gemm:
    """K-sharded W2A8 GEMM: rank r holds the weight columns (in-features) [r K/R, (r+1) K/R) and receives the matching
    slice of the activations, quantised per token ON ITS OWN slice (x_q_local int8 [M, K/R], x_scale_local fp32 [M]).

    Every rank computes a partial [M, N]; the partials are reduce-scattered by token rows: rank r ends up with rows
    [r M/R, (r+1) M/R) of the sum (``forward``), or ``forward_full`` all-gathers them back to [M, N].  The exchange
    moves the partials in the output dtype and sums them in fp32 in rank order (deterministic), rounding once.
    M must be a multiple of the world size.
    """

    def __init__(self, w_packed_local, w_scale_local, group=None, group_size=128, zero_point=1,
                 out_dtype=torch.float16, plan_factory=W2A8Plan):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N = w_packed_local.shape[0]
        self.out_dtype = out_dtype
        self.plan = plan_factory(w_packed_local, w_scale_local, group_size=group_size, zero_point=zero_point,
                                 out_dtype=out_dtype)

    def forward(self, x_q_local, x_scale_local):
        M = x_q_local.shape[0]
        partial = self.plan.gemm(x_q_local, x_scale_local)                   # [M, N], this rank's share of the sum
        if self.world == 1:
            return partial
        if M % self.world != 0:
            raise ValueError(f"M={M} must be a multiple of the world size {self.world}")
        rows = M // self.world
        recv = torch.empty_like(partial)                                     # [R, M/R, N]: block j from rank j
        dist.all_to_all_single(recv, partial.contiguous(), group=self.group)
        return recv.view(self.world, rows, self.N).float().sum(dim=0).to(self.out_dtype)

    def forward_full(self, x_q_local, x_scale_local):
        mine = self.forward(x_q_local, x_scale_local)
        if self.world == 1:
            return mine
        full = torch.empty(self.world * mine.shape[0], self.N, dtype=self.out_dtype, device=mine.device)
        dist.all_gather_into_tensor(full, mine.contiguous(), group=self.group)
        return full

    __call__ = forward

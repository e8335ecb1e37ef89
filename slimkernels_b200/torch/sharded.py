"""Sharded execution of one W2A8 GEMM across the GPUs of a node (one process per GPU): N-sharded with an all-gather
(ShardedW2A8Gemm) and K-sharded with a reduce-scatter (KShardedW2A8Gemm, for a projection whose input is already
split by features, like the down projection behind an N-sharded gate+up).

N-sharding:

Output features are independent, so rank r owns rows [r*N/R, (r+1)*N/R) of w_packed and the matching
columns of w_scale; activations are replicated; K is not split, so no reduction is needed.  The only
exchange is an all-gather of the fp16/bf16 output over NVLink: either NCCL after the GEMM, or (fused=True) the
GEMM's epilogue stores every finished tile into every rank's output buffer through peer pointers.
The reference has no multi-GPU code; this is the one parallel strategy the W2A8 path needs.

Failure behaviour.  The reference aborts the process on any CUDA error
(slimkernels/cute/gemm/wgmma_sm90_W2A8.cu:489-505); here a rank that is late or gone surfaces as a Python
exception (ExchangeTimeout) on the ranks that are still alive, raised on the HOST before the next launch:
  * every blocking collective on CPU tensors is issued asynchronously and waited for with a limit;
  * with a `control_group` (a gloo group over the same ranks) every step starts with a monitored barrier on
    the host, so a missing rank is noticed before a kernel that would wait for it is launched.
Nothing here makes a GPU wait without a limit, and no test hangs or faults a GPU.
"""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist

from .ops import W2A8Plan


class ExchangeTimeout(RuntimeError):
    """A rank did not take part in an exchange within the limit.  Carries rank, step and what was waited for."""

    def __init__(self, rank: int, step: int, what: str, limit_s: float, detail: str = ""):
        self.rank, self.step, self.what, self.limit_s = rank, step, what, limit_s
        super().__init__(f"rank {rank}, step {step}: {what} did not complete within {limit_s:.3g} s"
                         + (f" ({detail})" if detail else ""))


def _wait_with_limit(work, rank: int, step: int, what: str, limit_s):
    """Waits for an asynchronous collective.  CPU (gloo) work honours the limit and raises ExchangeTimeout;
    CUDA (NCCL) work is stream-ordered, so wait() only orders the stream and the limit is enforced by the process
    group's own timeout (init_process_group(timeout=...)) and, where given, by the control group."""
    if work is None:
        return
    try:
        if limit_s is None:
            work.wait()
        else:
            work.wait(datetime.timedelta(seconds=float(limit_s)))
    except RuntimeError as exc:      # gloo reports expiry (and peers that closed their connection) this way
        raise ExchangeTimeout(rank, step, what, float(limit_s or 0.0), str(exc).splitlines()[0]) from exc


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


class _Liveness:
    """Host-side check that every rank is still taking part, made before a step is launched."""

    def __init__(self, control_group, limit_s, rank):
        self.group, self.limit_s, self.rank = control_group, limit_s, rank

    def check(self, step: int):
        if self.group is None or self.limit_s is None:
            return
        try:
            dist.monitored_barrier(self.group, timeout=datetime.timedelta(seconds=float(self.limit_s)))
        except RuntimeError as exc:
            raise ExchangeTimeout(self.rank, step, "liveness barrier before the launch", float(self.limit_s),
                                  str(exc).splitlines()[0]) from exc


class ShardedW2A8Gemm:
    """Holds this rank's weight slice; ``forward`` returns the full [M, N] output on every rank.

    The returned tensor is a buffer owned by the op and is reused: it stays valid until the SECOND next call with
    the same M (two buffers alternate), so a consumer may still read step i's result while step i+1 runs, also on
    another stream, but must be ordered before step i+2 is launched.

    exchange_timeout_s: limit for the host-side waits (CPU collectives, liveness barrier); None = no limit.
    control_group: optional gloo group over the same ranks for the liveness barrier that precedes every launch.
    """

    def __init__(self, w_packed_local, w_scale_local, N_total: int, group=None, group_size=128, zero_point=1,
                 out_dtype=torch.float16, plan_factory=W2A8Plan, fused=False, exchange_timeout_s=None,
                 control_group=None):
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
        self.fused = bool(fused) and self.world > 1
        self.timeout_s = exchange_timeout_s
        self._live = _Liveness(control_group, exchange_timeout_s, self.rank)
        self._local = {}       # (M, device) -> [M, N_local]
        self._gather = {}      # (M, device) -> ([R, M, N_local], [[M, N_total]] x 2)
        self._symm = {}        # (M, device) -> [(buffer, handle, peer pointers)] x 2
        self._step = 0

    # ---- buffers (made on first use of a token count, then kept; only what the chosen exchange needs)
    def _local_buffer(self, M, device):
        key = (M, device)
        if key not in self._local:
            self._local[key] = torch.empty(M, self.N_local, dtype=self.out_dtype, device=device)
        return self._local[key]

    def _gather_buffers(self, M, device):
        key = (M, device)
        if key not in self._gather:
            gathered = torch.empty(self.world, M, self.N_local, dtype=self.out_dtype, device=device)
            full = [torch.empty(M, self.N_total, dtype=self.out_dtype, device=device) for _ in range(2)]
            self._gather[key] = (gathered, full)
        return self._gather[key]

    def _symmetric(self, M, device):
        """Two [M, N_total] output buffers in symmetric memory, each with the peers' pointers to it (this rank's
        first, then the others in ring order so that the ranks do not all write to the same peer at the same time)."""
        key = (M, device)
        if key not in self._symm:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group if self.group is not None else dist.group.WORLD
            slots = []
            for _ in range(2):
                buf = symm_mem.empty((M, self.N_total), dtype=self.out_dtype, device=device)
                hdl = symm_mem.rendezvous(buf, group)
                ptrs = [int(hdl.buffer_ptrs[(self.rank + i) % self.world]) for i in range(self.world)]
                slots.append((buf, hdl, ptrs))
            self._symm[key] = slots
        return self._symm[key]

    def local_gemm(self, x_q, x_scale):
        """This rank's GEMM alone (no exchange): [M, N_local]."""
        return self.plan.gemm(x_q, x_scale, out=self._local_buffer(x_q.shape[0], x_q.device))

    def forward_fused(self, x_q, x_scale):
        """GEMM whose epilogue stores every tile into all ranks' buffers, then one stream-ordered device barrier.
        Two buffers alternate: a rank that is a step ahead writes into the buffer its peers are NOT reading (a
        rank passes the barrier of step i+1 only after every rank's stream has reached it, i.e. after every
        rank's same-stream consumers of step i are done), so step i+2 may overwrite step i's buffer."""
        M = x_q.shape[0]
        self._live.check(self._step)
        buf, hdl, ptrs = self._symmetric(M, x_q.device)[self._step & 1]
        self.plan.gemm_scatter(x_q, x_scale, ptrs, self.N_total, self.rank * self.N_local)
        hdl.barrier()          # every rank's tiles have landed everywhere
        self._step += 1
        return buf

    def forward(self, x_q, x_scale):
        if self.fused:
            return self.forward_fused(x_q, x_scale)
        M = x_q.shape[0]
        local = self.local_gemm(x_q, x_scale)
        if self.world == 1:
            return local
        self._live.check(self._step)
        gathered, fulls = self._gather_buffers(M, x_q.device)
        full = fulls[self._step & 1]
        work = dist.all_gather_into_tensor(gathered.view(self.world * M, self.N_local), local, group=self.group,
                                           async_op=True)
        _wait_with_limit(work, self.rank, self._step, "all-gather of the output", self.timeout_s)
        # [R, M, N/R] -> [M, R, N/R] == [M, N]
        full.view(M, self.world, self.N_local).copy_(gathered.permute(1, 0, 2))
        self._step += 1
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

    ``fused=True``: the scatter half runs inside the GEMM.  Every rank owns a [R, M/R, N] buffer in symmetric memory
    (two of them, alternating by call); the epilogue of rank r's GEMM stores token-row block d of its partial straight
    into block r of rank d's buffer (peer stores, one destination per tile, nothing is loaded from a peer), one
    stream-ordered barrier follows, and every rank adds its R blocks in rank order.  Needs M/R to be a multiple of the
    GEMM's token tile (256 for M > 128).  The returned rows are a fresh tensor; the receive buffer of a call is
    overwritten by the second next call.
    """

    def __init__(self, w_packed_local, w_scale_local, group=None, group_size=128, zero_point=1,
                 out_dtype=torch.float16, plan_factory=W2A8Plan, exchange_timeout_s=None, control_group=None,
                 fused=False):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.N = w_packed_local.shape[0]
        self.out_dtype = out_dtype
        self.plan = plan_factory(w_packed_local, w_scale_local, group_size=group_size, zero_point=zero_point,
                                 out_dtype=out_dtype)
        self.timeout_s = exchange_timeout_s
        self._live = _Liveness(control_group, exchange_timeout_s, self.rank)
        self._step = 0
        self.fused = fused and self.world > 1
        self._symm = {}

    def _add_blocks(self, blocks):
        """[R, rows, N] partial sums -> [rows, N]: fp32 sum in rank order, rounded once."""
        if blocks.is_cuda and self.N % 8 == 0:
            return torch.ops.slimkernels.sum_row_blocks(blocks)          # one pass over the data
        acc = blocks[0].float()
        for r in range(1, blocks.shape[0]):
            acc = acc + blocks[r].float()
        return acc.to(self.out_dtype)

    def _symmetric(self, M, device):
        """Two [R, M/R, N] receive buffers in symmetric memory, each with every rank's pointer to it in rank order."""
        key = (M, device)
        if key not in self._symm:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")   # plain peer stores only
            import torch.distributed._symmetric_memory as symm_mem
            group = self.group if self.group is not None else dist.group.WORLD
            slots = []
            for _ in range(2):
                buf = symm_mem.empty((M, self.N), dtype=self.out_dtype, device=device)
                hdl = symm_mem.rendezvous(buf, group)
                ptrs = [int(hdl.buffer_ptrs[d]) for d in range(self.world)]
                slots.append((buf, hdl, ptrs))
            self._symm[key] = slots
        return self._symm[key]

    def forward_fused(self, x_q_local, x_scale_local):
        M = x_q_local.shape[0]
        if M % self.world != 0:
            raise ValueError(f"M={M} must be a multiple of the world size {self.world}")
        rows = M // self.world
        self._live.check(self._step)
        buf, hdl, ptrs = self._symmetric(M, x_q_local.device)[self._step & 1]
        # block d of this rank's partial -> block `rank` of rank d's buffer
        self.plan.gemm_rowscatter(x_q_local, x_scale_local, ptrs, rows, self.rank * rows, self.N)
        hdl.barrier()          # every rank's blocks have landed
        self._step += 1
        return self._add_blocks(buf.view(self.world, rows, self.N))

    def forward(self, x_q_local, x_scale_local):
        if self.fused:
            return self.forward_fused(x_q_local, x_scale_local)
        M = x_q_local.shape[0]
        partial = self.plan.gemm(x_q_local, x_scale_local)                   # [M, N], this rank's share of the sum
        if self.world == 1:
            return partial
        if M % self.world != 0:
            raise ValueError(f"M={M} must be a multiple of the world size {self.world}")
        self._live.check(self._step)
        rows = M // self.world
        recv = torch.empty_like(partial)                                     # [R, M/R, N]: block j from rank j
        work = dist.all_to_all_single(recv, partial.contiguous(), group=self.group, async_op=True)
        _wait_with_limit(work, self.rank, self._step, "exchange of the partial sums", self.timeout_s)
        self._step += 1
        return self._add_blocks(recv.view(self.world, rows, self.N))

    def forward_full(self, x_q_local, x_scale_local):
        mine = self.forward(x_q_local, x_scale_local)
        if self.world == 1:
            return mine
        full = torch.empty(self.world * mine.shape[0], self.N, dtype=self.out_dtype, device=mine.device)
        work = dist.all_gather_into_tensor(full, mine.contiguous(), group=self.group, async_op=True)
        _wait_with_limit(work, self.rank, self._step, "all-gather of the reduced rows", self.timeout_s)
        return full

    __call__ = forward


def shard_gate_up(gate_up_packed, gate_up_scale, world: int, rank: int):
    """This rank's share of a fused gate+up weight ([2*inter, K/4] packed, gate rows first; scales [K/G, 2*inter]):
    gate rows [r I/R, (r+1) I/R) followed by the up rows of the same features, so that SiLU(gate)*up stays local."""
    two_i = gate_up_packed.shape[0]
    if two_i % (2 * world) != 0:
        raise ValueError(f"2*inter={two_i} must be a multiple of 2*world_size={2 * world}")
    inter = two_i // 2
    per = inter // world
    rows = torch.cat([torch.arange(rank * per, (rank + 1) * per), torch.arange(inter + rank * per, inter + (rank + 1) * per)])
    rows = rows.to(gate_up_packed.device)
    return gate_up_packed[rows].contiguous(), gate_up_scale[:, rows].contiguous()


class TensorParallelW2A8LlamaMLP:
    """down( SiLU(gate(x)) * up(x) ) over R ranks with ONE exchange: gate+up split along their output features
    (``shard_gate_up``), SiLU*up and its re-quantisation local to the rank (per-token scales over the rank's slice of
    the intermediate features), down split along K (``shard_weight_k``) with the partial sums reduce-scattered by
    token rows -- inside the down GEMM's epilogue when ``fused`` (``KShardedW2A8Gemm``).

    x fp16 [M, hidden], replicated.  ``forward`` returns rows [r M/R, (r+1) M/R) of the block's output,
    ``forward_full`` all-gathers [M, hidden].  Numerically this is the sum over ranks of the single-GPU block applied to
    each rank's slices (each partial rounded to the output dtype once before the fp32 sum).
    """

    def __init__(self, gate_up_packed_local, gate_up_scale_local, down_packed_local, down_scale_local, group=None,
                 group_size=128, zero_point=1, out_dtype=torch.float16, fused=True, exchange_timeout_s=None,
                 control_group=None, plan_factory=W2A8Plan, activation_ops=None):
        # activation_ops: (quantize_activation_int8, silu_mul_quantize_int8) stand-ins, for tests without a GPU
        self._act = activation_ops
        self.gate_up = plan_factory(gate_up_packed_local, gate_up_scale_local, group_size=group_size,
                                    zero_point=zero_point, out_dtype=torch.float16)
        self.down = KShardedW2A8Gemm(down_packed_local, down_scale_local, group=group, group_size=group_size,
                                     zero_point=zero_point, out_dtype=out_dtype, plan_factory=plan_factory,
                                     exchange_timeout_s=exchange_timeout_s, control_group=control_group, fused=fused)

    def _hidden(self, x):
        if self._act is not None:
            quantize_activation_int8, silu_mul_quantize_int8 = self._act
        else:
            from .modules import quantize_activation_int8, silu_mul_quantize_int8
        x_q, x_s = quantize_activation_int8(x)
        gate_up = self.gate_up.gemm(x_q, x_s)                 # [M, 2 I/R]: this rank's gate columns, then its up columns
        return silu_mul_quantize_int8(gate_up)                # int8 [M, I/R], fp32 [M]

    def forward(self, x):
        return self.down(*self._hidden(x))

    def forward_full(self, x):
        return self.down.forward_full(*self._hidden(x))

    __call__ = forward

"""`slimkernels::w2a8_gemm` and its plan object.

The reference has no torch-facing quantised op (slimkernels/torch/llama.py only wraps HF generate);
the call shape follows its notebook wrapper ``wint2_gemm(activation, weight, scale) -> out``
(triton.ipynb:235-270): weights and scales in, a freshly allocated [M, N] tensor out, computed on the
current CUDA stream.  All compute happens in lib/libsk_w2a8.so behind the C ABI; if the extension is not
built or no sm_100 GPU is present the calls raise — there is no CPU or eager fallback.
"""
from __future__ import annotations

import weakref

import torch

from .. import _build

_loaded = False


def load_extension() -> None:
    """Loads lib/libsk_w2a8_torch.so (registers torch.ops.slimkernels.*).  Raises if it is not built."""
    global _loaded
    if _loaded:
        return
    import os
    if not os.path.exists(_build.TORCH_LIB):
        raise ImportError(f"{_build.TORCH_LIB} is not built; run `python -m slimkernels_b200._build`")
    torch.ops.load_library(_build.TORCH_LIB)
    _loaded = True


class W2A8Plan:
    """One weight matrix bound to its device (wraps sk_w2a8_plan).

    w_packed uint8 [N, K/4] (matrix_packer layout) or, with ``tiled=True``, the 1-D output of
    ``repack_weight``; w_scale float16 [K/G, N].  The tensors must stay alive as long as the plan.
    """

    def __init__(self, w, w_scale, N=None, K=None, group_size=128, zero_point=1, out_dtype=torch.float16,
                 tiled=False):
        load_extension()
        if not tiled:
            N, K = w.shape[0], w.shape[1] * 4
        if out_dtype not in (torch.float16, torch.bfloat16):
            raise TypeError("out_dtype must be torch.float16 or torch.bfloat16")
        self.N, self.K, self.group_size, self.zero_point = int(N), int(K), int(group_size), int(zero_point)
        self.out_dtype, self.tiled = out_dtype, tiled
        self._w, self._w_scale = w, w_scale          # keep the device buffers alive
        self._bf16 = out_dtype == torch.bfloat16
        self._h = torch.ops.slimkernels.w2a8_plan_create(w, w_scale, self.N, self.K, self.group_size,
                                                         self.zero_point, self._bf16, tiled)
        self._fin = weakref.finalize(self, _destroy, self._h)

    def set_option(self, key: int, value: int) -> None:
        torch.ops.slimkernels.w2a8_plan_set_option(self._h, key, value)

    def gemm(self, x_q, x_scale, out=None):
        if out is None:
            return torch.ops.slimkernels.w2a8_plan_gemm(self._h, x_q, x_scale, self.N, self.K, self._bf16)
        torch.ops.slimkernels.w2a8_plan_gemm_out(self._h, x_q, x_scale, out, self.K)
        return out

    def gemm_host(self, h_x_q, h_x_scale, h_out, chunk_tokens: int = 512):
        """The GEMM for operands that live in (pinned) HOST memory: int8 [M, K] and float32 [M] in, [M, N] out.

        The tokens are cut into chunks; the host->device copy of chunk i+1, the GEMM of chunk i and the
        device->host copy of chunk i-1 run on three streams at once, so a call costs about as much as its largest leg
        (for a wide layer that is the copy of the output over PCIe) instead of the sum of the three.  Device staging
        buffers are allocated on first use and kept.  Returns h_out; the caller's stream waits for everything.
        """
        dev = self._w.device
        M = h_x_q.shape[0]
        if h_x_q.device.type != "cpu" or h_out.device.type != "cpu" or h_x_scale.device.type != "cpu":
            raise TypeError("gemm_host takes host tensors")
        if tuple(h_out.shape) != (M, self.N) or h_out.dtype != self.out_dtype or h_x_q.shape[1] != self.K:
            raise ValueError("shape / dtype mismatch")
        st = getattr(self, "_host_state", None)
        if st is None or st["M"] < M:
            st = {"M": M, "x": torch.empty(M, self.K, dtype=torch.int8, device=dev),
                  "xs": torch.empty(M, dtype=torch.float32, device=dev),
                  "out": torch.empty(M, self.N, dtype=self.out_dtype, device=dev),
                  "s_in": torch.cuda.Stream(dev), "s_out": torch.cuda.Stream(dev)}
            self._host_state = st
        cur = torch.cuda.current_stream(dev)
        s_in, s_out = st["s_in"], st["s_out"]
        s_in.wait_stream(cur)                     # earlier users of the staging buffers are done
        s_out.wait_stream(cur)
        for lo in range(0, M, chunk_tokens):
            hi = min(M, lo + chunk_tokens)
            with torch.cuda.stream(s_in):
                st["x"][lo:hi].copy_(h_x_q[lo:hi], non_blocking=True)
                st["xs"][lo:hi].copy_(h_x_scale[lo:hi], non_blocking=True)
                ev_in = s_in.record_event()
            cur.wait_event(ev_in)
            self.gemm(st["x"][lo:hi], st["xs"][lo:hi], out=st["out"][lo:hi])
            ev_c = cur.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                h_out[lo:hi].copy_(st["out"][lo:hi], non_blocking=True)
        cur.wait_stream(s_out)
        return h_out

    def gemm_scatter(self, x_q, x_scale, out_ptrs, ld_out: int, col_offset: int) -> None:
        """Writes the [M, N] result at column `col_offset` of every [M, ld_out] buffer in `out_ptrs` (raw device
        pointers: this GPU's buffer first, then peer-mapped buffers of the other ranks)."""
        torch.ops.slimkernels.w2a8_plan_gemm_scatter(self._h, x_q, x_scale, list(out_ptrs), ld_out, col_offset, self.K)

    def gemm_rowscatter(self, x_q, x_scale, out_ptrs, rows_per_dest: int, dst_row0: int, ld_out: int) -> None:
        """Deals the token rows of the [M, N] result out: rows [d * rows_per_dest, (d + 1) * rows_per_dest) go to
        the buffer `out_ptrs[d]` only (raw device pointers, rank order; peer-mapped unless this GPU's), at rows
        dst_row0 .. of it.  The scatter half of a reduce-scatter of K-sharded partial sums."""
        torch.ops.slimkernels.w2a8_plan_gemm_rowscatter(self._h, x_q, x_scale, list(out_ptrs), rows_per_dest, dst_row0,
                                                       ld_out, self.K)

    def partials(self, x_q):
        return torch.ops.slimkernels.w2a8_plan_partials(self._h, x_q, self.N, self.K, self.group_size)

    def device_status(self) -> int:
        return torch.ops.slimkernels.w2a8_plan_device_status(self._h)

    def launch_floor_probe(self, M: int) -> None:
        """Launches the empty kernel with the launch geometry of a decode-sized GEMM (measurement aid)."""
        torch.ops.slimkernels.w2a8_plan_launch_floor_probe(self._h, self._w, int(M))

    def query_launch(self, M: int) -> dict:
        """The launch the plan makes for M tokens: token tile, split-K factor, CTAs and kernel kind
        (1 general tcgen05 kernel, 2 CUDA-core checker, 3 decode tcgen05 kernel)."""
        t, s, c, k = torch.ops.slimkernels.w2a8_plan_query_launch(self._h, int(M))
        return {"token_tile": t, "split_k": s, "ctas": c, "kernel": k}


def _destroy(handle):
    try:
        torch.ops.slimkernels.w2a8_plan_destroy(handle)
    except Exception:
        pass


def w2a8_gemm(x_q, x_scale, w_packed, w_scale, group_size: int = 128, zero_point: int = 1,
              out_dtype=torch.float16):
    """out[M, N] = x_scale[:, None] * sum_g w_scale[g] * (x_q[:, g] @ (codes[:, g] - zero_point).T).

    x_q int8 [M, K], x_scale float32 [M], w_packed uint8 [N, K/4] (first code of a byte in bits 7:6),
    w_scale float16 [K/group_size, N].  This is the registered op ``torch.ops.slimkernels.w2a8_gemm``: the plan
    (tiled weight copy) is built on first use of a weight tensor and kept, weakly, while that tensor object is
    alive and unmodified (it is rebuilt after an in-place write and dropped with the tensor).
    """
    load_extension()
    return torch.ops.slimkernels.w2a8_gemm(x_q, x_scale, w_packed, w_scale, group_size, zero_point, out_dtype)


def w2a8_partials(x_q, w_packed, w_scale, group_size: int = 128, zero_point: int = 1):
    """int32 [K/G, M, N]: the exact per-group integer partial sums the GEMM scales and adds."""
    load_extension()
    return torch.ops.slimkernels.w2a8_partials(x_q, w_packed, w_scale, group_size, zero_point)


def repack_weight(w_packed):
    load_extension()
    return torch.ops.slimkernels.w2a8_repack(w_packed)


def unrepack_weight(w_tiled, N: int, K: int):
    load_extension()
    return torch.ops.slimkernels.w2a8_unrepack(w_tiled, N, K)

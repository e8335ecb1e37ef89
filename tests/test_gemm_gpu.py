"""Parity of the sm_100a W2A8 GEMM with the CPU oracle, through the C ABI.

Bars: per-group int32 partial sums bit-exact; outputs within 1e-2 max-abs of the fp32 dequantise-then-matmul
reference path (plus half an output ulp is already inside that bound for these value ranges).
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import w2a8_oracle as O
from slimkernels_b200 import capi

pytestmark = pytest.mark.gpu

TOL = 1e-2   # max-abs vs fp32 dequant-matmul, stated by the benchmark spec


@pytest.fixture(scope="module", autouse=True)
def _need_gpu(built_libs):
    if not torch.cuda.is_available():
        pytest.fail("GPU tests selected but no CUDA device is visible")
    assert torch.cuda.get_device_capability(0)[0] == 10, "these kernels are sm_100a only"


from gpu_util import DeviceProblem, random_problem, to_np  # noqa: E402


def _check(prob_np, G=128, zp=1, dtype=torch.float16, force=None, ld_out=None, check_partials=True):
    x_q, xs, wp, ws = prob_np
    dp = DeviceProblem(x_q, xs, wp, ws, G, zp, dtype)
    if force:
        dp.force(**force)
    y = to_np(dp.gemm(ld_out=ld_out))
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws, G, zp)
    N = wp.shape[0]
    err = np.abs(y[:, :N] - y_ref).max()
    tol = TOL if dtype == torch.float16 else TOL + np.abs(y_ref).max() * 2.0 ** -8
    assert np.isfinite(y[:, :N]).all()
    assert err <= tol, f"max abs err {err}"
    if ld_out:
        assert np.isnan(y[:, N:]).all(), "wrote outside the N columns"
    if check_partials:
        p = to_np(dp.partials())
        np.testing.assert_array_equal(p, O.w2a8_partials(x_q, wp, G, zp))
    return err


def test_golden_vectors(golden):
    i = 0
    while f"gemm{i}_shape" in golden.files:
        M, N, K, G = (int(v) for v in golden[f"gemm{i}_shape"])
        x_q, xs = golden[f"gemm{i}_x_q"], golden[f"gemm{i}_x_scale"]
        wp, ws = golden[f"gemm{i}_w_packed"], golden[f"gemm{i}_w_scale"]
        if K % 32 == 0:
            dp = DeviceProblem(x_q, xs, wp, ws, G, 1)
            y = to_np(dp.gemm())
            assert np.abs(y - golden[f"gemm{i}_y_ref"]).max() <= TOL
            np.testing.assert_array_equal(to_np(dp.partials()), golden[f"gemm{i}_partials_zp1"])
        i += 1
    assert i >= 6


@pytest.mark.parametrize("zp", [1, 2])
def test_config0_full(zp):
    """Benchmark config 0: M=16, N=K=4096, G=128, seed 0."""
    from slimkernels_b200 import workloads as W
    prob = W.make_problem(16, 4096, 4096, 128, seed=0)
    _check(prob, 128, zp)


@pytest.mark.parametrize("token_tile", [16, 32, 64, 128, 192, 256])
@pytest.mark.parametrize("split_k", [1, 2, 4, 8])
def test_every_tile_and_split(token_tile, split_k):
    if token_tile >= 128 and split_k > 1:
        pytest.skip("split-K is for small token tiles")
    M = {16: 13, 32: 32, 64: 70, 128: 200, 192: 400, 256: 300}[token_tile]
    prob = random_problem(M, 384, 1024, 128, seed=token_tile + split_k)
    _check(prob, force=dict(kernel=capi.KERNEL_TCGEN05, token_tile=token_tile, split_k=split_k))


@pytest.mark.parametrize("token_tile", [16, 32])
@pytest.mark.parametrize("split_k", [1, 2, 4, 8])
@pytest.mark.parametrize("K", [128, 640, 1408, 4096])
def test_decode_kernel_every_tile_split_and_depth(token_tile, split_k, K):
    """The decode kernel (four K blocks per stage, weights expanded into tensor memory): K-block counts that are
    and are not multiples of its stage (1, 5, 11, 32), every cluster size, ragged M and N."""
    if split_k > K // 128:
        pytest.skip("more splits than groups")
    M = {16: 13, 32: 29}[token_tile]
    prob = random_problem(M, 392, K, 128, seed=token_tile + split_k + K)
    _check(prob, force=dict(kernel=capi.KERNEL_TCGEN05_DECODE, token_tile=token_tile, split_k=split_k))


@pytest.mark.parametrize("M,N,K,ctas", [
    (1, 128, 256, 0),        # one tile, one half stage: a single CTA writes it out directly
    (13, 392, 1024, 0),      # ragged M and N; every CTA one half stage
    (16, 392, 4096, 5),      # ranges of 12.8 half stages: tiles shared by two and three CTAs, cuts inside tiles
    (7, 1000, 2048, 3),      # ranges longer than a tile: direct tiles and shared tiles in one CTA
    (16, 640, 8192, 37),     # uneven cut of 160 half stages
    (29, 392, 1408 + 128, 4),  # 32-token tile, K = 12 K blocks
    (32, 1280, 4096, 296),   # more CTAs asked for than half stages exist: clamped
])
def test_balanced_split_decode_kernel(M, N, K, ctas):
    """The decode kernel that cuts the K range of the whole problem into equal CTA ranges: partial sums of shared
    tiles meet in the plan's scratch buffer and are added in slot order, so repeated launches are bit-identical."""
    x_q, xs, wp, ws = random_problem(M, N, K, 128, seed=M + N + K)
    dp = DeviceProblem(x_q, xs, wp, ws).force(kernel=capi.KERNEL_TCGEN05_DECODE_BALANCED)
    if ctas:
        dp.plan.set_option(capi.SK_OPT_STREAM_CTAS, ctas)
    q = dp.plan.query_launch(M)
    assert q["kernel"] == capi.KERNEL_TCGEN05_DECODE_BALANCED and q["split_k"] == 1
    assert q["ctas"] == min(ctas or 2 * torch.cuda.get_device_properties(0).multi_processor_count, (N + 127) // 128 * (K // 256))
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)
    y = [dp.gemm() for _ in range(3)]
    assert np.abs(to_np(y[0]) - y_ref).max() <= TOL
    assert torch.equal(y[0], y[1]) and torch.equal(y[0], y[2])
    # against the kernel that splits over clusters: same arithmetic up to the order of the fp32 partial sums
    y_cluster = dp.force(kernel=capi.KERNEL_TCGEN05_DECODE, split_k=1).gemm()
    assert np.abs(to_np(y[0]) - to_np(y_cluster)).max() <= 4e-3 * max(1.0, float(np.abs(y_ref).max()))
    # debug partials of a plan forced to the balanced kernel come from the cluster kernel: bit-exact
    dp.force(kernel=capi.KERNEL_TCGEN05_DECODE_BALANCED)
    np.testing.assert_array_equal(to_np(dp.partials()), O.w2a8_partials(x_q, wp, 128))


def test_balanced_split_kernel_falls_back_where_it_does_not_apply():
    # K = 5 K blocks (odd): no whole half stages; several token tiles; a forced split
    x_q, xs, wp, ws = random_problem(8, 256, 640, 128, seed=11)
    dp = DeviceProblem(x_q, xs, wp, ws)
    with pytest.raises(capi.SkError):
        dp.plan.set_option(capi.SK_OPT_KERNEL, capi.KERNEL_TCGEN05_DECODE_BALANCED)   # the plan has no scratch buffer
    x_q, xs, wp, ws = random_problem(40, 256, 1024, 128, seed=12)
    dp = DeviceProblem(x_q, xs, wp, ws).force(kernel=capi.KERNEL_TCGEN05_DECODE_BALANCED, token_tile=16)
    assert dp.plan.query_launch(40)["kernel"] == capi.KERNEL_TCGEN05_DECODE      # three token tiles
    assert np.abs(to_np(dp.gemm()) - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL
    dp.force(kernel=capi.KERNEL_TCGEN05_DECODE_BALANCED, split_k=2)
    assert dp.plan.query_launch(8)["kernel"] == capi.KERNEL_TCGEN05_DECODE
    # group size 64: general kernel
    x_q, xs, wp, ws = random_problem(8, 256, 1024, 64, seed=13)
    dp = DeviceProblem(x_q, xs, wp, ws, group_size=64)
    with pytest.raises(capi.SkError):
        dp.plan.set_option(capi.SK_OPT_KERNEL, capi.KERNEL_TCGEN05_DECODE_BALANCED)


def test_balanced_split_is_the_default_for_large_decode_problems():
    """From 64 K blocks per SM on (16-token tile) the balanced split is the default; 32-token tiles stay with clusters."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    N = 448 * 128
    for K in (2048, 4096):      # 48 and 97 K blocks per SM on 148 SMs
        x_q, xs, wp, ws = random_problem(16, N, K, 128, seed=K)
        dp = DeviceProblem(x_q, xs, wp, ws)
        big = (N // 128) * (K // 128) >= 64 * sms
        want = capi.KERNEL_TCGEN05_DECODE_BALANCED if big else capi.KERNEL_TCGEN05_DECODE
        assert dp.plan.query_launch(16)["kernel"] == want
        assert dp.plan.query_launch(32)["kernel"] == capi.KERNEL_TCGEN05_DECODE
        y = to_np(dp.gemm())
        cols = np.arange(0, N, 997)
        y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp[cols], ws[:, cols])
        assert np.abs(y[:, cols] - y_ref).max() <= TOL


@pytest.mark.parametrize("extra,K,M", [(2, 2048, 16), (9, 2048, 13), (36, 4096, 29), (44, 1024, 16), (60, 2048, 32), (41, 2048, 16)])
def test_decode_kernel_mixed_launch_when_there_are_more_tiles_than_sms(extra, K, M):
    """More feature tiles than SMs (but fewer than CTA slots): one CTA per tile for one tile per SM, the tiles beyond
    that split 4 ways (few of them) or 2 ways (an even number of them) inside clusters of four."""
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    tiles1 = (sms // 4) * 4
    n_tiles = tiles1 + extra
    N = n_tiles * 128 - 5                     # ragged last tile
    x_q, xs, wp, ws = random_problem(M, N, K, 128, seed=extra + K)
    dp = DeviceProblem(x_q, xs, wp, ws)
    q = dp.plan.query_launch(M)
    slots = 2 * sms
    if tiles1 + 4 * extra <= slots and K // 128 >= 16:
        want = 4
    elif extra % 2 == 0 and tiles1 + 2 * extra <= slots and K // 128 >= 8:
        want = 2
    else:
        want = 1
    assert q["kernel"] == capi.KERNEL_TCGEN05_DECODE and q["split_k"] == want
    assert q["ctas"] == (tiles1 + extra * want if want > 1 else n_tiles)
    y = dp.gemm()
    cols = np.unique(np.concatenate([np.arange(0, N, 701), np.arange(tiles1 * 128 - 64, N)]))   # incl. every split tile
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp[cols], ws[:, cols])
    assert np.abs(to_np(y)[:, cols] - y_ref).max() <= TOL
    assert torch.equal(dp.gemm(), y)
    # against a plain launch (one CTA per tile)
    y_plain = dp.force(kernel=capi.KERNEL_TCGEN05_DECODE, split_k=1).gemm()
    assert np.abs(to_np(y) - to_np(y_plain)).max() <= 4e-3 * max(1.0, float(np.abs(y_ref).max()))


def test_decode_kernel_is_the_default_for_small_batches():
    x_q, xs, wp, ws = random_problem(8, 512, 2048, 128, seed=3)
    dp = DeviceProblem(x_q, xs, wp, ws)
    assert dp.plan.query_launch(8)["kernel"] == capi.KERNEL_TCGEN05_DECODE
    assert dp.plan.query_launch(64)["kernel"] == capi.KERNEL_TCGEN05
    y = to_np(dp.gemm())
    y_general = to_np(dp.force(kernel=capi.KERNEL_TCGEN05).gemm())
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)
    assert np.abs(y - y_ref).max() <= TOL and np.abs(y_general - y_ref).max() <= TOL
    # several token tiles in one launch
    x_q, xs, wp, ws = random_problem(61, 256, 1024, 128, seed=4)
    dp = DeviceProblem(x_q, xs, wp, ws).force(kernel=capi.KERNEL_TCGEN05_DECODE, token_tile=16)
    assert np.abs(to_np(dp.gemm()) - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL


@pytest.mark.parametrize("token_tile,M,N,K,G", [
    (128, 1000, 2400, 384, 128),    # 8 x 19 = 152 tiles > 148 SMs: some CTAs walk two tiles, ragged edges
    (256, 2000, 2400, 384, 128),
    (128, 2304, 2432, 320, 64),     # 342 tiles, groups spanning half a K block, 5 groups per tile (odd)
    (256, 4600, 2176, 128, 128),    # one group per tile: fewer groups than accumulator buffers
])
def test_persistent_tile_walk(token_tile, M, N, K, G):
    """More tiles than SMs: a resident set of CTAs walks the tiles; bit-identical to one CTA per tile."""
    x_q, xs, wp, ws = random_problem(M, N, K, G, seed=token_tile + M)
    dp = DeviceProblem(x_q, xs, wp, ws, group_size=G)
    y_one = to_np(dp.force(token_tile=token_tile, persistent=1).gemm())
    y_walk = to_np(dp.force(token_tile=token_tile, persistent=2).gemm())
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws, group_size=G)
    assert np.abs(y_walk - y_ref).max() <= TOL
    assert np.array_equal(y_walk, y_one)
    assert np.array_equal(y_walk, to_np(dp.gemm()))   # and again: nothing left over from the first launch


@pytest.mark.parametrize("M,N,K,G", [
    (1, 128, 128, 128), (1, 8, 32, 32), (7, 130, 256, 128), (33, 200, 384, 128), (5, 136, 352, 32),
    (16, 264, 512, 64), (9, 128, 768, 256), (129, 257, 1408, 128), (300, 1000, 640, 128),
])
def test_ragged_shapes(M, N, K, G):
    _check(random_problem(M, N, K, G, seed=M + N + K), G=G)


@pytest.mark.parametrize("token_tile,M,N", [(64, 50, 392), (128, 200, 1000), (256, 300, 264), (256, 700, 1280)])
def test_tma_store_output_matches_thread_stores(token_tile, M, N):
    """General kernel, one CTA per tile: the tile leaves through one TMA store (clipped at ragged edges) or through
    the epilogue threads' vector stores; same bits either way, nothing written outside [M, N]."""
    x_q, xs, wp, ws = random_problem(M, N, 512, 128, seed=M + N)
    dp = DeviceProblem(x_q, xs, wp, ws)
    y_threads = to_np(dp.force(kernel=capi.KERNEL_TCGEN05, token_tile=token_tile, tma_store=1).gemm(ld_out=N + 64))
    y_tma = to_np(dp.force(kernel=capi.KERNEL_TCGEN05, token_tile=token_tile, tma_store=2).gemm(ld_out=N + 64))
    assert np.isnan(y_tma[:, N:]).all()
    np.testing.assert_array_equal(y_tma[:, :N], y_threads[:, :N])
    assert np.abs(y_tma[:, :N] - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (300, 1000, 640), (700, 1280, 1408), (1025, 512, 4096), (130, 256, 256)])
def test_pair_kernel_against_oracle_and_single_cta_kernel(M, N, K):
    """The prefill kernel on pairs of CTAs (cta_group::2: two CTAs share a 256-token tile, each loading half of it):
    ragged token and feature edges, one and many K blocks; outputs bit-identical to the one-CTA kernel (same
    arithmetic in the same order), integer partial sums bit-exact."""
    prob = random_problem(M, N, K, 128, seed=M + K)
    x_q, xs, wp, ws = prob
    dp = DeviceProblem(x_q, xs, wp, ws).force(kernel=capi.KERNEL_TCGEN05_PAIR, token_tile=256)
    assert dp.plan.query_launch(M)["kernel"] == capi.KERNEL_TCGEN05_PAIR
    y_pair = dp.gemm(ld_out=N + 8)
    p_pair = to_np(dp.partials())
    y_one = dp.force(kernel=capi.KERNEL_TCGEN05, token_tile=256).gemm(ld_out=N + 8)
    assert dp.plan.query_launch(M)["kernel"] == capi.KERNEL_TCGEN05
    assert torch.equal(y_pair[:, :N], y_one[:, :N])
    assert torch.isnan(y_pair[:, N:]).all()
    assert np.abs(to_np(y_pair)[:, :N] - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL
    np.testing.assert_array_equal(p_pair, O.w2a8_partials(x_q, wp, 128))


def test_pair_kernel_needs_an_even_number_of_feature_tiles():
    x_q, xs, wp, ws = random_problem(300, 384, 256, 128, seed=12)      # three feature tiles: one CTA per tile
    dp = DeviceProblem(x_q, xs, wp, ws)
    assert dp.plan.query_launch(300)["kernel"] == capi.KERNEL_TCGEN05
    assert dp.force(kernel=capi.KERNEL_TCGEN05_PAIR).plan.query_launch(300)["kernel"] == capi.KERNEL_TCGEN05
    assert np.abs(to_np(dp.gemm()) - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL


@pytest.mark.parametrize("ld_extra", [0, 8, 3])      # TMA stores, TMA stores into a wider buffer, thread stores (odd pitch)
def test_row_scatter_deals_token_rows_to_their_destinations(ld_extra):
    """sk_w2a8_gemm_rowscatter on one GPU with two local destination buffers standing in for two ranks' buffers."""
    M, N, K, rows = 512, 384, 512, 256
    x_q, xs, wp, ws = random_problem(M, N, K, 128, seed=77)
    dp = DeviceProblem(x_q, xs, wp, ws)
    y = dp.gemm()
    ld = N + ld_extra
    bufs = [torch.zeros(2 * rows, ld, dtype=torch.float16, device="cuda") for _ in range(2)]
    lib = capi.load()
    ptrs = (ctypes.c_void_p * 2)(bufs[0].data_ptr(), bufs[1].data_ptr())
    rc = lib.sk_w2a8_gemm_rowscatter(dp.plan.handle, M, dp.x_q.data_ptr(), K, dp.x_scale.data_ptr(), ptrs, 2, rows, rows,
                                     ld, dp.stream())     # "this rank" is rank 1: its blocks land at rows 256..511
    assert rc == capi.SK_OK
    torch.cuda.synchronize()
    assert dp.plan.device_status() == 0
    for d in range(2):
        assert torch.equal(bufs[d][rows:, :N], y[d * rows:(d + 1) * rows])
        assert not bufs[d][:rows].any() and not bufs[d][:, N:].any()
    # rows per destination that are not whole token tiles, a decode-sized call, a wrong total: refused, nothing launched
    assert lib.sk_w2a8_gemm_rowscatter(dp.plan.handle, M, dp.x_q.data_ptr(), K, dp.x_scale.data_ptr(), ptrs, 2, rows - 1, 0,
                                       ld, dp.stream()) == capi.SK_ERR_BAD_SHAPE
    assert lib.sk_w2a8_gemm_rowscatter(dp.plan.handle, 32, dp.x_q.data_ptr(), K, dp.x_scale.data_ptr(), ptrs, 2, 16, 0,
                                       ld, dp.stream()) == capi.SK_ERR_UNAVAILABLE
    assert lib.sk_w2a8_gemm_rowscatter(dp.plan.handle, 128, dp.x_q.data_ptr(), K, dp.x_scale.data_ptr(), ptrs, 2, 64, 0,
                                       ld, dp.stream()) == capi.SK_ERR_UNAVAILABLE      # 128-token tile, 64 rows each


@pytest.mark.parametrize("zp", [0, 1, 2, 3])
def test_expander_shared_memory_image_matches_tma_of_pre_expanded_weights(zp):
    """One 128 x 128 block: what the expander threads leave in shared memory (2-bit -> int8, swizzled K-major) against
    what the TMA leaves there for the same values given as int8 -- byte for byte -- and against the 128-byte swizzle
    written out on the host."""
    from slimkernels_b200 import format as F
    rng = np.random.default_rng(40 + zp)
    codes = rng.integers(0, 4, size=(128, 128), dtype=np.uint8)                 # [feature row, k]
    packed = F.pack_matrix(codes)                                                # matrix_packer layout [128, 32]
    dev = torch.device("cuda")
    lib = capi.load()
    d_packed = torch.from_numpy(packed).to(dev)
    tiled = torch.empty(4096, dtype=torch.uint8, device=dev)                     # one tiled block
    assert lib.sk_w2a8_tiled_bytes(128, 128) == 4096
    assert lib.sk_w2a8_repack(d_packed.data_ptr(), 128, 128, tiled.data_ptr(), torch.cuda.current_stream().cuda_stream) == capi.SK_OK
    expanded = (codes.astype(np.int16) - zp).astype(np.int8)
    d_exp = torch.from_numpy(expanded).to(dev)
    img_a = torch.zeros(16384, dtype=torch.uint8, device=dev)
    img_b = torch.zeros(16384, dtype=torch.uint8, device=dev)
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    rc = lib.sk_w2a8_debug_expander_image(tiled.data_ptr(), zp, d_exp.data_ptr(), img_a.data_ptr(), img_b.data_ptr(),
                                          flags.data_ptr(), flags.data_ptr() + 4, torch.cuda.current_stream().cuda_stream)
    assert rc == capi.SK_OK
    torch.cuda.synchronize()
    mism, status = flags.cpu().tolist()
    assert status == 0 and mism == 0
    a = img_a.cpu().numpy().view(np.int8).reshape(128, 8, 16)
    assert np.array_equal(a, img_b.cpu().numpy().view(np.int8).reshape(128, 8, 16))
    # row r at r * 128 bytes, its 16-byte chunk c at chunk position c ^ (r & 7)
    want = np.empty_like(a)
    for r in range(128):
        for c in range(8):
            want[r, c ^ (r & 7)] = expanded[r, 16 * c:16 * c + 16]
    assert np.array_equal(a, want)


def test_checker_kernel_matches_oracle():
    prob = random_problem(19, 200, 512, 128, seed=5)
    _check(prob, force=dict(kernel=capi.KERNEL_CUDA_CORE))


def test_wider_output_buffer_and_padded_activation_rows():
    x_q, xs, wp, ws = random_problem(24, 256, 512, 128, seed=9)
    _check((x_q, xs, wp, ws), ld_out=256 + 64, check_partials=False)
    dp = DeviceProblem(x_q, xs, wp, ws, ld_x=512 + 64)
    y = to_np(dp.gemm())
    assert np.abs(y - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL


@pytest.mark.parametrize("zp", [0, 3])
def test_other_zero_points(zp):
    """Zero points 0 and 3 reach |code - zp| = 3: the largest per-group sums (128 * 127 * 3) and the tightest depth bound
    of the int32 running sums under the accumulator bias 2^22."""
    _check(random_problem(20, 256, 512, 128, seed=zp), zp=zp)


def test_many_groups_accuracy():
    """K = 28672 (224 groups, the 70B down-projection depth): accumulated rounding stays inside the tolerance."""
    x_q, xs, wp, ws = random_problem(48, 256, 28672, 128, seed=77)
    for tile in (64, 256):
        dp = DeviceProblem(x_q, xs, wp, ws).force(token_tile=tile)
        y = to_np(dp.gemm())
        y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)
        assert np.abs(y - y_ref).max() <= TOL
        # and well inside it, against the same arithmetic in fp32 on the CPU
        assert np.abs(y - O.w2a8_gemm_int_path(x_q, xs, wp, ws)).max() <= 6e-3


def test_bf16_output():
    _check(random_problem(40, 256, 512, 128, seed=3), dtype=torch.bfloat16, check_partials=False)


def test_extreme_codes_and_activations():
    """All-max / all-min operands reach the partial-sum bound 128*127*2 without overflow or saturation."""
    M, N, K = 16, 128, 256
    for code_byte, xv, zp in [(0xFF, 127, 1), (0x00, -127, 1), (0x00, 127, 2), (0xFF, -127, 2)]:
        x_q = np.full((M, K), xv, dtype=np.int8)
        xs = np.full((M,), 0.01, dtype=np.float32)
        wp = np.full((N, K // 4), code_byte, dtype=np.uint8)
        ws = np.full((K // 128, N), 0.005, dtype=np.float16)
        dp = DeviceProblem(x_q, xs, wp, ws, 128, zp)
        np.testing.assert_array_equal(to_np(dp.partials()), O.w2a8_partials(x_q, wp, 128, zp))
        assert np.abs(to_np(dp.gemm()) - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws, 128, zp)).max() <= TOL


def test_repack_round_trip_on_device():
    from slimkernels_b200 import format as F
    lib = capi.load()
    rng = np.random.default_rng(2)
    for N, K in [(128, 128), (200, 160), (5, 32), (1000, 1408)]:
        wp = rng.integers(0, 256, size=(N, K // 4), dtype=np.uint8)
        d_wp = torch.from_numpy(wp).cuda()
        nbytes = lib.sk_w2a8_tiled_bytes(N, K)
        assert nbytes == F.tiled_nbytes(N, K)
        d_t = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        assert lib.sk_w2a8_repack(d_wp.data_ptr(), N, K, d_t.data_ptr(), None) == 0
        np.testing.assert_array_equal(d_t.cpu().numpy(), F.repack_tiled(wp))
        d_back = torch.zeros_like(d_wp)
        assert lib.sk_w2a8_unrepack(d_t.data_ptr(), N, K, d_back.data_ptr(), None) == 0
        np.testing.assert_array_equal(O.unpack_matrix(d_back.cpu().numpy()), O.unpack_matrix(wp))


def test_plan_from_tiled_weights():
    x_q, xs, wp, ws = random_problem(16, 256, 512, 128, seed=21)
    lib = capi.load()
    d_wp = torch.from_numpy(wp).cuda()
    d_t = torch.empty(lib.sk_w2a8_tiled_bytes(256, 512), dtype=torch.uint8, device="cuda")
    assert lib.sk_w2a8_repack(d_wp.data_ptr(), 256, 512, d_t.data_ptr(), None) == 0
    torch.cuda.synchronize()
    d_ws = torch.from_numpy(ws).cuda()
    plan = capi.Plan(0, 256, 512, 128, 1, d_t.data_ptr(), d_ws.data_ptr(), w_layout=capi.SK_WEIGHT_TILED)
    d_x, d_xs = torch.from_numpy(x_q).cuda(), torch.from_numpy(xs).cuda()
    out = torch.empty(16, 256, dtype=torch.float16, device="cuda")
    plan.gemm(16, d_x.data_ptr(), 512, d_xs.data_ptr(), out.data_ptr(), 256, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.abs(to_np(out) - O.w2a8_gemm_dequant_path(x_q, xs, wp, ws)).max() <= TOL
    with pytest.raises(capi.SkError):
        plan.set_option(capi.SK_OPT_KERNEL, capi.KERNEL_CUDA_CORE)   # needs the row-major bytes


def test_argument_errors_on_device():
    x_q, xs, wp, ws = random_problem(4, 128, 128, 128, seed=1)
    dp = DeviceProblem(x_q, xs, wp, ws)
    lib = capi.load()
    out = torch.empty(4, 128, dtype=torch.float16, device="cuda")
    h = dp.plan.handle
    assert lib.sk_w2a8_gemm(h, 0, dp.x_q.data_ptr(), 128, dp.x_scale.data_ptr(), out.data_ptr(), 128, None) == capi.SK_ERR_BAD_SHAPE
    assert lib.sk_w2a8_gemm(h, 4, dp.x_q.data_ptr(), 64, dp.x_scale.data_ptr(), out.data_ptr(), 128, None) == capi.SK_ERR_BAD_SHAPE
    assert lib.sk_w2a8_gemm(h, 4, dp.x_q.data_ptr(), 128, dp.x_scale.data_ptr(), out.data_ptr(), 64, None) == capi.SK_ERR_BAD_SHAPE
    assert lib.sk_w2a8_gemm(h, 4, dp.x_q.data_ptr() + 1, 128, dp.x_scale.data_ptr(), out.data_ptr(), 128, None) == capi.SK_ERR_BAD_ALIGNMENT
    assert lib.sk_w2a8_gemm(h, 4, dp.x_q.data_ptr(), 136, dp.x_scale.data_ptr(), out.data_ptr(), 128, None) == capi.SK_ERR_BAD_ALIGNMENT
    assert lib.sk_w2a8_gemm(h, 4, None, 128, dp.x_scale.data_ptr(), out.data_ptr(), 128, None) == capi.SK_ERR_NULL_POINTER


def test_decode_shapes_property_linearity():
    """Llama-2-7B decode shapes at full size: GPU tcgen05 kernel == GPU checker kernel bit for bit on the
    integer partials, and y(x1 + x2) == y(x1) + y(x2) for activations that stay in int8 range."""
    from slimkernels_b200 import workloads as W
    for name, (N, K) in W.LLAMA2_7B_SHAPES.items():
        x_q, xs, wp, ws = random_problem(32, N, K, 128, seed=N % 97)
        x_q = (x_q // 2).astype(np.int8)
        dp = DeviceProblem(x_q, xs, wp, ws)
        p_tc = dp.partials()
        dp.force(kernel=capi.KERNEL_CUDA_CORE)
        p_cc = dp.partials()
        assert torch.equal(p_tc, p_cc), name
        dp.force()
        # linearity on the integer level: P(x) + P(x') == P(x + x')
        x2 = np.roll(x_q, 1, axis=0)
        dp2 = DeviceProblem(x2, xs, wp, ws)
        dps = DeviceProblem((x_q + x2).astype(np.int8), xs, wp, ws)
        assert torch.equal(p_tc + dp2.partials(), dps.partials()), name
        # sampled rows against the CPU oracle
        rows = np.array([0, 1, N // 2, N - 1])
        y = to_np(dp.gemm())
        y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp[rows], ws[:, rows])
        assert np.abs(y[:, rows] - y_ref).max() <= TOL, name


def test_prefill_shape_against_checker_and_sampled_oracle():
    """M=2048, N=K=8192 (benchmark config 2, smallest M): full output vs the CUDA-core checker kernel, sampled
    output columns vs the CPU oracle."""
    M, N, K = 2048, 8192, 8192
    x_q, xs, wp, ws = random_problem(M, N, K, 128, seed=42)
    dp = DeviceProblem(x_q, xs, wp, ws)
    y = dp.gemm()
    dp.force(kernel=capi.KERNEL_CUDA_CORE)
    y_cc = dp.gemm()
    # two fp32 evaluation orders, each rounded to fp16 (ulp 2e-3 at |y| in [2, 4)): at most a few ulps apart
    assert (y.float() - y_cc.float()).abs().max().item() <= 6e-3
    cols = np.arange(0, N, 509)
    y_ref = O.w2a8_gemm_dequant_path(x_q, xs, wp[cols], ws[:, cols])
    assert np.abs(to_np(y)[:, cols] - y_ref).max() <= TOL

"""GPU parity of the three GEMM kernels against the CPU oracle, through the C ABI.

Tolerances (relative Frobenius error against the UNROUNDED fp64 oracle): 1e-3 for
fp32, 5e-3 for fp16/bf16 — the figures the benchmark specification states."""
import numpy as np
import pytest

from frisk_b200 import capi
from oracle import gemm_oracle, inputs
from oracle.numerics import from_storage, rel_frobenius, to_storage
from tests.util import Guarded, to_device, to_host

pytestmark = pytest.mark.gpu
TOL = {"fp32": 1e-3, "fp16": 5e-3, "bf16": 5e-3}
TC_ALGOS = [capi.ALGO_TCGEN05, capi.ALGO_TCGEN05_PAIR]
SKINNY_ALGOS = [capi.ALGO_SKINNY]


@pytest.fixture(scope="module")
def ctx():
    c = capi.Context(0)
    yield c
    c.close()


def run_gemm(ctx, a, b, dtype_ab, dtype_c, M, N, K, ta, tb, c_init=None, algo=capi.ALGO_AUTO, offset=0):
    """a, b in storage form -> (C storage-form numpy, guards_ok)."""
    import torch
    ga = Guarded(a.shape, dtype_ab, fill=a, offset=offset)
    gb = Guarded(b.shape, dtype_ab, fill=b, offset=offset)
    gc = Guarded((M, N), dtype_c, fill=c_init, offset=offset)
    if c_init is None:
        gc.view.fill_(float("nan"))
    desc = capi.gemm_desc(M, N, K, dtype_ab, dtype_c, ta, tb, clear_accum=c_init is None, algo=algo)
    before_a, before_b = ga.raw.clone(), gb.raw.clone()
    ctx.gemm(desc, ga.view.data_ptr(), gb.view.data_ptr(), gc.view.data_ptr(),
             stream=torch.cuda.current_stream().cuda_stream)
    ctx.check(torch.cuda.current_stream().cuda_stream)
    ok = gc.guards_intact() and torch.equal(before_a, ga.raw) and torch.equal(before_b, gb.raw)
    return gc.host(), ok


def check(ctx, M, N, K, dtype_ab, dtype_c, ta, tb, seed, accumulate=False, algo=capi.ALGO_AUTO, dist="uniform",
          offset=0):
    a, b = inputs.gemm_inputs(M, N, K, dtype_ab, ta, tb, seed, dist)
    c_init = None
    if accumulate:
        rng = np.random.default_rng(seed + 1000)
        c_init = to_storage(rng.standard_normal((M, N), dtype=np.float32), dtype_c)
    got, ok = run_gemm(ctx, a, b, dtype_ab, dtype_c, M, N, K, ta, tb, c_init, algo, offset)
    assert ok, "guard zone or input changed"
    ref = gemm_oracle.gemm_fp64(a, b, dtype_ab, ta, tb, c_init, dtype_c)
    gotf = from_storage(got, dtype_c)
    assert np.isfinite(gotf).all()
    err = rel_frobenius(gotf, ref)
    assert err <= TOL[dtype_ab], (M, N, K, dtype_ab, dtype_c, ta, tb, err)
    return err


# ------------------------------------------------------------------ fp32: CUDA cores and split-bf16 tensor cores
F32_ALGOS = [capi.ALGO_AUTO, capi.ALGO_SIMT_F32, capi.ALGO_F32_SPLIT]


@pytest.mark.parametrize("algo", F32_ALGOS)
def test_f32_config_1024(ctx, algo):
    spec = inputs.WORKLOADS["gemm_f32_1024"]
    err = check(ctx, spec["M"], spec["N"], spec["K"], "fp32", "fp32", False, False, spec["seed"], algo=algo)
    assert err < 1e-5  # fp32 accumulation of 1024 terms is far inside the 1e-3 budget
    # the tensor-core path adds nine exact-product GEMMs of a three-term bf16 split: fp32-GEMM accuracy
    assert err < 2e-6 or algo == capi.ALGO_SIMT_F32, err


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_f32_split_transposes_accumulate_unaligned(ctx, ta, tb):
    S = capi.ALGO_F32_SPLIT
    assert check(ctx, 264, 136, 72, "fp32", "fp32", ta, tb, 14, algo=S) < 2e-6
    assert check(ctx, 520, 328, 200, "fp32", "fp32", ta, tb, 15, accumulate=True, algo=S) < 2e-6
    assert check(ctx, 72, 264, 136, "fp32", "fp32", ta, tb, 16, algo=S, offset=4) < 2e-6  # scalar loads and stores
    with pytest.raises(ValueError):
        check(ctx, 100, 77, 51, "fp32", "fp32", ta, tb, 11, algo=S)  # extents must be multiples of 8


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_f32_simt_shared_k_ranges(ctx, ta, tb):
    """Shapes whose tiles are fewer than the SMs or do not divide among them: every tile's k range is shared
    between workers (tickets, partial tiles), with ragged edges and a ragged last k stage."""
    S = capi.ALGO_SIMT_F32
    check(ctx, 520, 328, 200, "fp32", "fp32", ta, tb, 15, accumulate=True, algo=S)
    check(ctx, 130, 70, 1500, "fp32", "fp32", ta, tb, 17, algo=S)
    check(ctx, 64, 64, 9000, "fp32", "fp32", ta, tb, 18, algo=S)          # one tile, 141 stages over 141 workers
    check(ctx, 1024, 1024, 96, "fp32", "fp32", ta, tb, 19, algo=S)       # 256 tiles of two stages


def test_f32_simt_rerun_is_bit_identical(ctx):
    a, b = inputs.gemm_inputs(1024, 1024, 1024, "fp32", False, False, 5, "uniform")
    first, ok1 = run_gemm(ctx, a, b, "fp32", "fp32", 1024, 1024, 1024, False, False, algo=capi.ALGO_SIMT_F32)
    for _ in range(3):
        again, ok2 = run_gemm(ctx, a, b, "fp32", "fp32", 1024, 1024, 1024, False, False, algo=capi.ALGO_SIMT_F32)
        assert ok1 and ok2 and np.array_equal(first, again)


def test_f32_config_1024_built_through_the_ir_builders(ctx):
    """The same workload the way the benchmark states it: the bind_test-style kernel (8 x 8 grid of
    128-thread blocks, 128 x 32 / 32 x 128 shared tiles, test/python/bind_test.py:28-58) built with
    the builders over f32 memrefs, then executed, against the fp64 oracle."""
    import torch

    import frisk_b200 as F
    from tests.test_frontend import build_bind_test_module
    spec = inputs.WORKLOADS["gemm_f32_1024"]
    M, N, K = spec["M"], spec["N"], spec["K"]
    mod = build_bind_test_module(clear_accum=True, with_side_ops=False, dtype_name="f32", shape=(M, N))
    assert mod.verify() and "frisk.gemm" in str(mod) and "memref<1024x1024xf32, 1>" in str(mod)
    a, b = inputs.gemm_inputs(**spec)
    ta, tb = to_device(a, "fp32"), to_device(b, "fp32")
    tc = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    F.execute(mod, ta, tb, tc, torch.empty(M, dtype=torch.float32, device="cuda"))
    torch.cuda.synchronize()
    err = rel_frobenius(to_host(tc, "fp32"), gemm_oracle.gemm_fp64(a, b, "fp32"))
    assert err <= TOL["fp32"] and err < 1e-5, err


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_f32_transposes_ragged(ctx, ta, tb):
    check(ctx, 100, 77, 51, "fp32", "fp32", ta, tb, 11)
    check(ctx, 129, 65, 17, "fp32", "fp32", ta, tb, 12, accumulate=True)
    check(ctx, 256, 128, 64, "fp32", "fp32", ta, tb, 13)


def test_f32_tiny_and_odd_offsets(ctx):
    check(ctx, 1, 1, 1, "fp32", "fp32", False, False, 1)
    check(ctx, 3, 5, 7, "fp32", "fp32", False, False, 2, offset=4)  # 4-byte aligned only: scalar paths
    check(ctx, 64, 64, 64, "fp32", "fp32", False, True, 3, offset=4)


# ------------------------------------------------------------------ tcgen05
@pytest.mark.parametrize("algo", TC_ALGOS)
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_tc_single_tile(ctx, dtype, algo):
    # one tile; 1, 2, 5 and 7 k-blocks (ring wrap-around with 4 / 6 stages)
    for K in (64, 128, 320, 448):
        check(ctx, 128, 256, K, dtype, dtype, False, True, 21, algo=algo, dist="normal_rsqrt_k")
        check(ctx, 256, 256, K, dtype, dtype, False, True, 21, algo=algo, dist="normal_rsqrt_k")


@pytest.mark.parametrize("algo", TC_ALGOS)
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, True), (True, False)])
def test_tc_layouts(ctx, dtype, ta, tb, algo):
    check(ctx, 256, 512, 256, dtype, dtype, ta, tb, 22, algo=algo, dist="normal_rsqrt_k")


@pytest.mark.parametrize("algo", TC_ALGOS)
@pytest.mark.parametrize("ta,tb", [(False, True), (False, False), (True, True), (True, False)])
def test_tc_ragged_edges(ctx, ta, tb, algo):
    # M, N not multiples of the tile; K not a multiple of the k-block (TMA zero fill)
    check(ctx, 200, 264, 72, "bf16", "bf16", ta, tb, 23, algo=algo, dist="normal_rsqrt_k")
    check(ctx, 8, 8, 8, "fp16", "fp16", ta, tb, 24, algo=algo)
    check(ctx, 304, 520, 200, "fp16", "fp16", ta, tb, 24, algo=algo, dist="normal_rsqrt_k")


@pytest.mark.parametrize("algo", TC_ALGOS)
def test_tc_f32_output_and_accumulate(ctx, algo):
    check(ctx, 384, 256, 192, "fp16", "fp32", False, True, 25, algo=algo, dist="normal_rsqrt_k")
    check(ctx, 384, 256, 192, "bf16", "fp32", False, True, 26, accumulate=True, algo=algo)
    check(ctx, 130, 520, 136, "fp16", "fp16", False, True, 27, accumulate=True, algo=algo)


@pytest.mark.parametrize("algo", TC_ALGOS)
def test_tc_many_tiles_persistent(ctx, algo):
    # more tiles than SMs (or SM pairs): every CTA walks several tiles and both accumulators
    check(ctx, 2048, 4096, 256, "bf16", "bf16", False, True, 28, algo=algo, dist="normal_rsqrt_k")
    check(ctx, 4096, 4096, 128, "fp16", "fp16", False, False, 28, algo=algo, dist="normal_rsqrt_k")


@pytest.mark.parametrize("tb", [True, False])
def test_tc_tail_wave_of_half_tiles(ctx, tb):
    # 16 x 10 = 160 tiles on 148 SMs: the 12 tiles of the last wave run as 24 half-width items
    check(ctx, 2048, 2560, 192, "bf16", "bf16", False, tb, 29, algo=capi.ALGO_TCGEN05, dist="normal_rsqrt_k")
    # ragged N: the second half of the last tile column lies wholly outside the matrix
    check(ctx, 2048, 2400, 64, "fp16", "fp32", False, tb, 30, algo=capi.ALGO_TCGEN05, dist="normal_rsqrt_k")


@pytest.mark.parametrize("algo", [capi.ALGO_TCGEN05, capi.ALGO_TCGEN05_PAIR])
@pytest.mark.parametrize("dtype_c", ["fp16", "fp32"])
def test_tc_store_boxes_at_ragged_edges(ctx, algo, dtype_c):
    """Overwriting stores leave as 32-row x 128-byte boxes through TMA: tiles whose last boxes lie partly or wholly
    outside C (ragged M and N), several tiles per CTA so that the two boxes of a warp are reused across tiles."""
    check(ctx, 2100, 2400, 64, "fp16", dtype_c, False, True, 41, algo=algo, dist="normal_rsqrt_k")
    check(ctx, 5000, 4904, 128, "bf16", "bf16" if dtype_c == "fp16" else "fp32", False, True, 42, algo=algo,
          dist="normal_rsqrt_k")
    check(ctx, 300, 520, 96, "fp16", dtype_c, False, False, 43, algo=algo, dist="normal_rsqrt_k")


@pytest.mark.parametrize("tb", [True, False])
def test_tc_pair_few_tiles_all_split_in_k(ctx, tb):
    """Fewer 256 x 256 tiles than half the CTA pairs and a K worth halving: EVERY tile runs as two K halves that
    meet through the fp32 scratch (ragged edges, fp32 and 16-bit outputs, accumulate, repeat on the same scratch)."""
    P = capi.ALGO_TCGEN05_PAIR
    for _ in range(2):
        check(ctx, 1024, 2048, 4096, "fp16", "fp16", False, tb, 61, algo=capi.ALGO_AUTO, dist="normal_rsqrt_k")
    check(ctx, 1000, 1800, 2048, "bf16", "fp32", False, tb, 62, algo=P, dist="normal_rsqrt_k")
    check(ctx, 520, 304, 1024, "bf16", "bf16", False, tb, 63, accumulate=True, algo=P, dist="normal_rsqrt_k")
    check(ctx, 256, 256, 8192, "fp16", "fp16", False, tb, 64, algo=capi.ALGO_AUTO, dist="normal_rsqrt_k")


@pytest.mark.parametrize("tb", [True, False])
def test_tc_pair_tail_wave_split_in_k(ctx, tb):
    # 8 x 10 = 80 tiles of 256x256 on 74 CTA pairs: the 6 tiles of the last wave run as 12 K halves
    # that meet through the fp32 scratch
    P = capi.ALGO_TCGEN05_PAIR
    check(ctx, 2048, 2560, 512, "bf16", "bf16", False, tb, 36, algo=P, dist="normal_rsqrt_k")
    check(ctx, 2048, 2560, 1024, "fp16", "fp32", False, tb, 37, accumulate=True, algo=P, dist="normal_rsqrt_k")
    check(ctx, 2000, 2500 // 8 * 8, 576, "fp16", "fp16", False, tb, 38, algo=P, dist="normal_rsqrt_k")
    a, b = inputs.gemm_inputs(2048, 2560, 512, "bf16", False, tb, 39, "normal_rsqrt_k")
    first, _ = run_gemm(ctx, a, b, "bf16", "bf16", 2048, 2560, 512, False, tb, algo=P)
    for _ in range(3):  # tickets must be clean again after every launch; the sum is order-independent
        again, ok = run_gemm(ctx, a, b, "bf16", "bf16", 2048, 2560, 512, False, tb, algo=P)
        assert ok and np.array_equal(first, again)


def test_tc_config_4096_nt(ctx):
    """Full benchmark size: rows sampled against the fp64 oracle, the whole matrix against
    size-independent properties (deterministic rerun; C(2A) = 2C exactly in fp16)."""
    import torch
    spec = inputs.WORKLOADS["gemm_f16_4096_nt"]
    M, N, K = spec["M"], spec["N"], spec["K"]
    a, b = inputs.gemm_inputs(**spec)
    got, ok = run_gemm(ctx, a, b, "fp16", "fp16", M, N, K, False, True)
    assert ok
    rng = np.random.default_rng(5)
    rows, cols = np.sort(rng.choice(M, 96, replace=False)), np.sort(rng.choice(N, 512, replace=False))
    ref = gemm_oracle.gemm_sampled_fp64(a, b, "fp16", rows, cols, False, True)
    err = rel_frobenius(from_storage(got, "fp16")[np.ix_(rows, cols)], ref)
    assert err <= TOL["fp16"], err
    again, _ = run_gemm(ctx, a, b, "fp16", "fp16", M, N, K, False, True)
    assert np.array_equal(got.view(np.uint16), again.view(np.uint16))
    a2 = (a.astype(np.float32) * 2).astype(np.float16)
    doubled, _ = run_gemm(ctx, a2, b, "fp16", "fp16", M, N, K, False, True)
    normal = np.abs(got.astype(np.float32)) >= 2.0 ** -13  # doubling is not exact across fp16 subnormals
    assert normal.mean() > 0.99
    assert np.array_equal(doubled[normal], (got.astype(np.float32) * 2).astype(np.float16)[normal])
    # secondary cross-check of every element against the vendor GEMM (not authoritative)
    ta_, tb_ = to_device(a, "fp16"), to_device(b, "fp16")
    lib = (ta_.float() @ tb_.float().T).cpu().numpy()
    assert rel_frobenius(from_storage(got, "fp16"), lib) <= TOL["fp16"]


@pytest.mark.parametrize("tb,dtype_c", [(True, "bf16"), (False, "fp32")])
def test_tc_pair_wide_items_deep_k(ctx, tb, dtype_c):
    """K >= 8192 with several rounds of 256 x 512 items per CTA pair: both accumulators belong to one item whose
    halves share the A k-blocks.  Ragged M and N (the last item's second half lies wholly beyond N); the fp64
    oracle covers sampled rows, the first and the last 128 rows, over all columns."""
    import torch
    M, N, K = 4700, 8200, 8192
    a, b = inputs.gemm_inputs(M, N, K, "bf16", False, tb, 51, "normal_rsqrt_k")
    da, db = to_device(a, "bf16"), to_device(b, "bf16")
    dc = torch.full((M, N), float("nan"), dtype=torch.bfloat16 if dtype_c == "bf16" else torch.float32, device="cuda")
    desc = capi.gemm_desc(M, N, K, "bf16", dtype_c, False, tb, clear_accum=True)
    assert capi.load().frisk_b200_gemm_select(desc) == capi.ALGO_TCGEN05_PAIR
    stream = torch.cuda.current_stream().cuda_stream
    ctx.gemm(desc, da.data_ptr(), db.data_ptr(), dc.data_ptr(), stream=stream)
    ctx.check(stream)
    got = from_storage(to_host(dc, dtype_c), dtype_c)
    assert np.isfinite(got).all()
    rng = np.random.default_rng(52)
    rows = np.unique(np.concatenate([rng.choice(M, 64, replace=False), np.arange(128), np.arange(M - 128, M)]))
    a64 = from_storage(a, "bf16").astype(np.float64)[rows]
    b64 = from_storage(b, "bf16").astype(np.float64)
    ref = a64 @ (b64.T if tb else b64)
    err = rel_frobenius(got[rows], ref)
    assert err <= TOL["bf16"], err
    again = torch.full_like(dc, float("nan"))
    ctx.gemm(desc, da.data_ptr(), db.data_ptr(), again.data_ptr(), stream=stream)
    ctx.check(stream)
    assert torch.equal(dc, again)


def test_deepk_config(ctx):
    """bf16 GEMM M = N = 8192, K = 131072 at its own size (2048 k-blocks per tile, 1024 tiles on 74 CTA
    pairs, both tensor-memory accumulators).  The whole product is 17.6 TFLOP, out of reach for a
    CPU, so the fp64 oracle covers a sample: 64 random rows x 64 random columns with the full K
    extent plus two whole 256 x 256 blocks, one interior and one in the last tile row and column.
    The whole matrix is covered by a bit-identical rerun.  Contract:
    lib/Dialect/Frisk/IR/FriskOps.cpp:416-426, LegacyImportSemantics.cpp:26-44."""
    import torch
    spec = inputs.WORKLOADS["gemm_bf16_deepk"]
    M, N, K = spec["M"], spec["N"], spec["K"]
    rng = np.random.default_rng(6)
    rows = np.unique(np.concatenate([rng.choice(M, 64, replace=False), np.arange(2304, 2560), np.arange(M - 256, M)]))
    cols = np.unique(np.concatenate([rng.choice(N, 64, replace=False), np.arange(4352, 4608), np.arange(N - 256, N)]))
    dev = {"a": torch.empty(M, K, dtype=torch.bfloat16, device="cuda"),
           "b": torch.empty(N, K, dtype=torch.bfloat16, device="cuda")}
    keep = {"a": np.zeros((len(rows), K), np.uint16), "b": np.zeros((len(cols), K), np.uint16)}
    want = {"a": rows, "b": cols}
    # 2 x 2^30 values: the bulk is rounded to bf16 on the device (round-to-nearest-even, like the
    # host-side to_storage the sampled rows go through; the two are compared below)
    for name, r0, blk in inputs.gemm_inputs_streamed(**spec, chunk_rows=256, storage=False):
        dev[name][r0:r0 + blk.shape[0]].copy_(torch.from_numpy(blk).cuda().to(torch.bfloat16))
        sel = np.nonzero((want[name] >= r0) & (want[name] < r0 + blk.shape[0]))[0]
        keep[name][sel] = to_storage(blk[want[name][sel] - r0], "bf16")
    for name in ("a", "b"):
        idx = torch.from_numpy(want[name]).cuda()
        assert np.array_equal(to_host(dev[name][idx], "bf16"), keep[name])
    c = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    desc = capi.gemm_desc(M, N, K, "bf16", "bf16", False, True, clear_accum=True)
    assert capi.load().frisk_b200_gemm_select(desc) == capi.ALGO_TCGEN05_PAIR
    stream = torch.cuda.current_stream().cuda_stream
    ctx.gemm(desc, dev["a"].data_ptr(), dev["b"].data_ptr(), c.data_ptr(), stream=stream)
    ctx.check(stream)
    got = from_storage(to_host(c, "bf16"), "bf16")
    assert np.isfinite(got).all()
    a64 = from_storage(keep["a"], "bf16").astype(np.float64)
    b64 = from_storage(keep["b"], "bf16").astype(np.float64)
    ri, ci = {int(r): i for i, r in enumerate(rows)}, {int(c_): i for i, c_ in enumerate(cols)}

    def sample_err(rr, cc):
        ref = a64[[ri[int(r)] for r in rr]] @ b64[[ci[int(c_)] for c_ in cc]].T
        return rel_frobenius(got[np.ix_(rr, cc)], ref)

    errs = {"cross": sample_err(rows, cols),
            "interior_block": sample_err(np.arange(2304, 2560), np.arange(4352, 4608)),
            "last_block": sample_err(np.arange(M - 256, M), np.arange(N - 256, N))}
    assert max(errs.values()) <= TOL["bf16"], errs
    c2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.gemm(desc, dev["a"].data_ptr(), dev["b"].data_ptr(), c2.data_ptr(), stream=stream)
    ctx.check(stream)
    assert torch.equal(c.view(torch.int16), c2.view(torch.int16))


# ------------------------------------------------------------------ skinny
@pytest.mark.parametrize("algo", SKINNY_ALGOS)
def test_skinny_config(ctx, algo):
    spec = inputs.WORKLOADS["gemm_bf16_skinny"]
    err = check(ctx, spec["M"], spec["N"], spec["K"], "bf16", "bf16", False, True, spec["seed"], dist="act_weight",
                algo=algo)
    assert err < 4e-3


@pytest.mark.parametrize("algo", SKINNY_ALGOS)
@pytest.mark.parametrize("dtype", ["fp16", "bf16"])
def test_skinny_shapes(ctx, dtype, algo):
    # tiny, ragged in every extent, fewer tiles than SMs (a tile's K shared by many CTAs), one output shard of 8 GPUs
    for (M, N, K) in ((16, 64, 256), (1, 8, 8), (7, 100, 264), (16, 1000, 4096), (13, 2056, 9000 // 8 * 8),
                      (16, 3584, 8192), (3, 130, 72)):
        check(ctx, M, N, K, dtype, dtype, False, True, 31, algo=algo, dist="act_weight")


@pytest.mark.parametrize("algo", SKINNY_ALGOS)
def test_skinny_f32_out_accumulate_and_repeat(ctx, algo):
    check(ctx, 16, 512, 16384, "bf16", "fp32", False, True, 32, algo=algo, dist="act_weight")
    check(ctx, 5, 264, 2048, "fp16", "fp16", False, True, 33, accumulate=True, algo=algo)
    # the control words must be clean after every launch: identical bits on repeats
    a, b = inputs.gemm_inputs(16, 4096, 8192, "bf16", False, True, 34, "act_weight")
    first, _ = run_gemm(ctx, a, b, "bf16", "bf16", 16, 4096, 8192, False, True, algo=algo)
    for _ in range(3):
        again, ok = run_gemm(ctx, a, b, "bf16", "bf16", 16, 4096, 8192, False, True, algo=algo)
        assert ok and np.array_equal(first, again)


def test_skinny_matches_tcgen05_kernel(ctx):
    a, b = inputs.gemm_inputs(16, 1024, 2048, "bf16", False, True, 35, "act_weight")
    s, _ = run_gemm(ctx, a, b, "bf16", "fp32", 16, 1024, 2048, False, True, algo=capi.ALGO_SKINNY)
    t, _ = run_gemm(ctx, a, b, "bf16", "fp32", 16, 1024, 2048, False, True, algo=capi.ALGO_TCGEN05)
    assert rel_frobenius(s, t) < 1e-5


# ------------------------------------------------------------------ host-buffer entry + errors
def test_gemm_host_entry(ctx):
    a, b = inputs.gemm_inputs(256, 512, 128, "fp16", False, True, 41, "normal_rsqrt_k")
    c = np.zeros((256, 512), np.float16)
    desc = capi.gemm_desc(256, 512, 128, "fp16", "fp16", False, True)
    ctx.gemm_host(desc, a.ctypes.data, b.ctypes.data, c.ctypes.data)
    assert rel_frobenius(c, gemm_oracle.gemm_fp64(a, b, "fp16", False, True)) <= TOL["fp16"]


def test_gemm_host_entry_pipelined_panels(ctx):
    # large enough that the host entry moves A and C in row panels that overlap the kernels
    rng = np.random.default_rng(43)
    for (M, N, K, dt, acc) in ((4096, 1024, 512, "fp16", False), (3000, 1024, 520, "bf16", True),
                               (2048, 1024, 1024, "fp32", False)):
        a, b = inputs.gemm_inputs(M, N, K, dt, False, True, 44, "normal_rsqrt_k" if dt != "fp32" else "uniform")
        c0 = to_storage(rng.standard_normal((M, N), dtype=np.float32), dt) if acc else None
        c = c0.copy() if acc else np.zeros((M, N), a.dtype)
        desc = capi.gemm_desc(M, N, K, dt, dt, False, True, clear_accum=not acc)
        ctx.gemm_host(desc, a.ctypes.data, b.ctypes.data, c.ctypes.data)
        ref = gemm_oracle.gemm_fp64(a, b, dt, False, True, c0, dt)
        assert rel_frobenius(from_storage(c, dt), ref) <= TOL[dt], (M, N, K, dt)


def test_gemm_host_entry_short_last_panel_and_explicit_algo(ctx):
    """M just above a panel boundary: the 16-row remainder is merged into the panel before it and
    every panel runs the kernel chosen for the whole problem; an explicit algorithm is honoured."""
    M, N, K = 1040, 4096, 4096
    a, b = inputs.gemm_inputs(M, N, K, "fp16", False, True, 45, "normal_rsqrt_k")
    ref = gemm_oracle.gemm_fp64(a, b, "fp16", False, True)
    for algo in (capi.ALGO_AUTO, capi.ALGO_TCGEN05, capi.ALGO_TCGEN05_PAIR):
        c = np.full((M, N), np.nan, np.float16)
        desc = capi.gemm_desc(M, N, K, "fp16", "fp16", False, True, algo=algo)
        ctx.gemm_host(desc, a.ctypes.data, b.ctypes.data, c.ctypes.data)
        assert np.isfinite(c).all() and rel_frobenius(c, ref) <= TOL["fp16"], algo


def test_contract_errors_before_launch(ctx):
    import torch
    a = torch.zeros(128, 64, dtype=torch.float16, device="cuda")  # room for a shifted 64x64 view
    desc = capi.gemm_desc(64, 64, 64, "fp16", "fp16", False, True)
    with pytest.raises(ValueError, match="overlaps"):
        ctx.gemm(desc, a.data_ptr(), a.data_ptr(), a.data_ptr())
    c = torch.zeros(64, 64, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError, match="16-byte"):
        ctx.gemm(desc, a.data_ptr() + 2, a.data_ptr(), c.data_ptr())
    with pytest.raises(ValueError, match="legacy-gemm-type"):
        ctx.gemm(capi.gemm_desc(64, 64, 64, "fp32", "fp16"), a.data_ptr(), a.data_ptr(), c.data_ptr())
    with pytest.raises(ValueError, match="legacy-gemm-shape"):
        ctx.gemm(capi.gemm_desc(64, 0, 64, "fp16"), a.data_ptr(), a.data_ptr(), c.data_ptr())


def test_execute_bind_test_style(ctx):
    """Build the GEMM through the builders, then execute it (the flow the reference's
    bind_test stops short of)."""
    import torch

    import frisk_b200 as F
    from tests.test_frontend import build_bind_test_module
    mod = build_bind_test_module(clear_accum=True, with_side_ops=False, shape=(512, 512))
    a, b = inputs.gemm_inputs(512, 512, 512, "fp16", False, False, 42, "normal_rsqrt_k")
    ta, tb = to_device(a, "fp16"), to_device(b, "fp16")
    tc = torch.empty(512, 512, dtype=torch.float16, device="cuda")
    F.execute(mod, ta, tb, tc, torch.empty(512, dtype=torch.float16, device="cuda"))
    torch.cuda.synchronize()
    assert rel_frobenius(to_host(tc, "fp16"), gemm_oracle.gemm_fp64(a, b, "fp16")) <= TOL["fp16"]


def test_gemm_push_into_row_block_owners(ctx):
    """The fused split-K epilogue on one GPU: two "ranks" (K halves) store their fp32 products into
    their slots of two row-block owners (stand-ins for two GPUs' memories), then each owner sums
    its slots and rounds."""
    import torch
    M, N, K = 1024, 768, 1024
    a, b = inputs.gemm_inputs(M, N, K, "bf16", False, True, 61, "normal_rsqrt_k")
    rows = M // 2
    owners = [torch.full((2, rows, N), float("nan"), device="cuda") for _ in range(2)]  # [slot][rows][N] per owner
    desc = capi.gemm_desc(M, N, K // 2, "bf16", "fp32", False, True, clear_accum=True, algo=capi.ALGO_TCGEN05_PAIR)
    s = torch.cuda.current_stream().cuda_stream
    for rank in range(2):
        da = to_device(np.ascontiguousarray(a[:, rank * (K // 2):(rank + 1) * (K // 2)]), "bf16")
        db = to_device(np.ascontiguousarray(b[:, rank * (K // 2):(rank + 1) * (K // 2)]), "bf16")
        ctx.gemm_push(desc, da.data_ptr(), db.data_ptr(), [o[rank].data_ptr() for o in owners], rows, N, stream=s)
    ctx.check(s)
    ref = gemm_oracle.gemm_fp64(a, b, "bf16", False, True)
    got = torch.cat([o.sum(dim=0) for o in owners]).cpu().numpy()
    assert rel_frobenius(got, ref) <= 1e-5
    out = torch.empty(rows, N, dtype=torch.bfloat16, device="cuda")
    ctx.sum_slots(owners[1].data_ptr(), 2, rows * N, out.data_ptr(), rows * N, "bf16", stream=s)
    torch.cuda.synchronize()
    assert rel_frobenius(from_storage(to_host(out, "bf16"), "bf16"), ref[rows:]) <= TOL["bf16"]
    want = (owners[1][0] + owners[1][1]).to(torch.bfloat16)
    assert torch.equal(out, want)  # slot order, one rounding
    with pytest.raises(ValueError):
        ctx.gemm_push(desc, da.data_ptr(), db.data_ptr(), [owners[0][0].data_ptr()], M // 4, N, stream=s)  # rows not covered


def test_gemm_push_wide_items_deep_k(ctx):
    """The K-split push with K >= 32768 per rank and several rounds of 256 x 512 items per CTA pair (the shape class of
    the deep-K benchmark split over two or four GPUs): two K halves pushed into two row-block owners, ragged N."""
    import torch
    M, N, K = 4608, 8200, 65536
    a, b = inputs.gemm_inputs(M, N, K, "bf16", False, True, 65, "normal_rsqrt_k")
    rows = M // 2
    owners = [torch.full((2, rows, N), float("nan"), device="cuda") for _ in range(2)]
    desc = capi.gemm_desc(M, N, K // 2, "bf16", "fp32", False, True, clear_accum=True, algo=capi.ALGO_TCGEN05_PAIR)
    s = torch.cuda.current_stream().cuda_stream
    for rank in range(2):
        da = to_device(np.ascontiguousarray(a[:, rank * (K // 2):(rank + 1) * (K // 2)]), "bf16")
        db = to_device(np.ascontiguousarray(b[:, rank * (K // 2):(rank + 1) * (K // 2)]), "bf16")
        ctx.gemm_push(desc, da.data_ptr(), db.data_ptr(), [o[rank].data_ptr() for o in owners], rows, N, stream=s)
    ctx.check(s)
    got = torch.cat([o.sum(dim=0) for o in owners]).cpu().numpy()
    assert np.isfinite(got).all()
    rng = np.random.default_rng(66)
    pick = np.unique(np.concatenate([rng.choice(M, 48, replace=False), np.arange(32), np.arange(M - 32, M)]))
    ref = from_storage(a, "bf16").astype(np.float64)[pick] @ from_storage(b, "bf16").astype(np.float64).T
    assert rel_frobenius(got[pick], ref) <= 1e-4   # fp32 sums of 32768 products per rank, unrounded output


def test_gemm_push_more_tiles_than_cta_pairs(ctx):
    # 80 tiles on 74 CTA pairs, four owners: every tile is stored whole (no K halves in this mode)
    import torch
    M, N, K = 2048, 2560, 512
    a, b = inputs.gemm_inputs(M, N, K, "fp16", False, True, 63, "normal_rsqrt_k")
    da, db = to_device(a, "fp16"), to_device(b, "fp16")
    t = [torch.full((M // 4, N), float("nan"), device="cuda") for _ in range(4)]
    desc = capi.gemm_desc(M, N, K, "fp16", "fp32", False, True, clear_accum=True, algo=capi.ALGO_TCGEN05_PAIR)
    s = torch.cuda.current_stream().cuda_stream
    ctx.gemm_push(desc, da.data_ptr(), db.data_ptr(), [x.data_ptr() for x in t], M // 4, N, stream=s)
    ctx.check(s)
    ref = gemm_oracle.gemm_fp64(a, b, "fp16", False, True)
    assert rel_frobenius(torch.cat(t).cpu().numpy(), ref) <= 1e-5


def _push_worker(rank, world, port, out_dir):
    import os

    import torch
    import torch.distributed as dist

    from frisk_b200 import splitk
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        c = capi.Context(rank)
        M, N, K = 1024, 512, 2048
        a, b = inputs.gemm_inputs(M, N, K, "bf16", False, True, 62, "normal_rsqrt_k")
        kl = K // world
        da = to_device(np.ascontiguousarray(a[:, rank * kl:(rank + 1) * kl]), "bf16", f"cuda:{rank}")
        db = to_device(np.ascontiguousarray(b[:, rank * kl:(rank + 1) * kl]), "bf16", f"cuda:{rank}")
        op = splitk.SplitKGemmPush(M, N, K, world, rank, "bf16", c, dist.group.WORLD)
        for _ in range(3):
            out = op.run(da, db)
        torch.cuda.synchronize()
        ref = gemm_oracle.gemm_fp64(a, b, "bf16", False, True)[rank * (M // world):(rank + 1) * (M // world)]
        err = rel_frobenius(from_storage(to_host(out, "bf16"), "bf16"), ref)
        with open(os.path.join(out_dir, f"err{rank}.txt"), "w") as f:
            f.write(repr(err))
        dist.barrier()
        op.close()
        c.close()
    finally:
        dist.destroy_process_group()


def test_splitk_push_two_gpus(tmp_path):
    """Two ranks on two GPUs (skipped on a one-GPU box): each pushes its K half into the owners'
    buffers over peer mappings; leaves between steps only, NVLS off."""
    import socket

    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    mp.spawn(_push_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert float((tmp_path / f"err{r}.txt").read_text()) <= TOL["bf16"]


# ------------------------------------------------------------------ fill / row-reduce next to the gemm
def run_fused(ctx, M, N, K, dtype_ab, dtype_c, seed, *, fill=None, kind=None, clear=True, clear_accum=True,
              algo=capi.ALGO_AUTO, c_init=None, expect_fused=None):
    """-> (C storage, reduce storage or None, oracle C fp64, r_init)."""
    import torch
    a, b = inputs.gemm_inputs(M, N, K, dtype_ab, False, True, seed, "normal_rsqrt_k")
    ga, gb = Guarded(a.shape, dtype_ab, fill=a), Guarded(b.shape, dtype_ab, fill=b)
    gc = Guarded((M, N), dtype_c, fill=c_init)
    if c_init is None:
        gc.view.fill_(float("nan"))  # must not be read: neither with clear_accum nor with a fill
    rng = np.random.default_rng(seed + 7)
    r_init = to_storage(rng.standard_normal(M, dtype=np.float32), dtype_c)
    gr = Guarded((M,), dtype_c, fill=r_init)
    desc = capi.gemm_desc(M, N, K, dtype_ab, dtype_c, False, True, clear_accum=clear_accum, algo=algo)
    epi = capi.gemm_epilogue(fill=fill, reduce=kind, reduce_dst=gr.view.data_ptr() if kind else None,
                             reduce_clear=clear)
    if expect_fused is not None:
        assert capi.gemm_fused_select(desc, epi) == expect_fused
    s = torch.cuda.current_stream().cuda_stream
    ctx.gemm_fused(desc, epi, ga.view.data_ptr(), gb.view.data_ptr(), gc.view.data_ptr(), stream=s)
    ctx.check(s)
    assert gc.guards_intact() and gr.guards_intact()
    base = None
    if fill is not None and not clear_accum:
        base = np.broadcast_to(to_storage(np.float32(fill).reshape(1, 1), dtype_c), (M, N))
    elif not clear_accum:
        base = c_init
    ref = gemm_oracle.gemm_fp64(a, b, dtype_ab, False, True, base, dtype_c)
    return gc.host(), (gr.host() if kind else None), ref, r_init


def check_reduce(got_c, got_r, dtype_c, kind, clear, r_init):
    want = gemm_oracle.row_reduce(got_c, dtype_c, kind, None if clear else r_init)
    got = from_storage(got_r, dtype_c).astype(np.float64)
    if kind == "add":  # fp32 accumulation, one rounding to the element type
        assert np.all(np.abs(got - want) <= 2e-3 * np.abs(want) + 2e-2)
    else:              # exact: the extreme of the stored values
        assert np.array_equal(got, want)


@pytest.mark.parametrize("dtype_c", ["fp16", "fp32"])
@pytest.mark.parametrize("kind", ["max", "min", "add"])
def test_fused_row_reduce_in_pair_epilogue(ctx, kind, dtype_c):
    # 9 x 10 tiles on 74 pairs: whole tiles and a K-split tail wave; ragged N masks the last columns
    for N, clear in ((2560, True), (2496, False)):
        c, r, ref, r0 = run_fused(ctx, 2304, N, 512, "fp16", dtype_c, 70, kind=kind, clear=clear, expect_fused=1)
        assert rel_frobenius(from_storage(c, dtype_c), ref) <= TOL["fp16"]
        check_reduce(c, r, dtype_c, kind, clear, r0)


def test_fused_fill_replaces_the_read_of_c(ctx):
    # C holds NaN: a fused fill must not read it.  bf16 output, then with a reduction on top.
    c, _, ref, _ = run_fused(ctx, 2304, 2560, 256, "bf16", "bf16", 71, fill=0.75, clear_accum=False, expect_fused=1)
    assert rel_frobenius(from_storage(c, "bf16"), ref) <= TOL["bf16"]
    c, r, ref, r0 = run_fused(ctx, 2304, 2560, 256, "bf16", "bf16", 72, fill=-1.5, kind="max", clear_accum=False,
                              expect_fused=1)
    assert rel_frobenius(from_storage(c, "bf16"), ref) <= TOL["bf16"]
    check_reduce(c, r, "bf16", "max", True, r0)


def test_fill_and_reduce_composed_for_the_other_kernels(ctx):
    # one-CTA tcgen05 kernel, fp32 SIMT kernel, skinny kernel, and a reduction after an accumulate that reads C
    c, r, ref, r0 = run_fused(ctx, 384, 520, 192, "fp16", "fp16", 73, fill=0.25, kind="add", clear_accum=False,
                              clear=False, expect_fused=0)
    assert rel_frobenius(from_storage(c, "fp16"), ref) <= TOL["fp16"]
    check_reduce(c, r, "fp16", "add", False, r0)
    c, r, ref, r0 = run_fused(ctx, 130, 77, 51, "fp32", "fp32", 74, kind="min", expect_fused=0)
    assert rel_frobenius(c, ref) <= TOL["fp32"]
    check_reduce(c, r, "fp32", "min", True, r0)
    c, r, ref, r0 = run_fused(ctx, 8, 4096, 1024, "bf16", "bf16", 75, kind="max", expect_fused=0)
    assert rel_frobenius(from_storage(c, "bf16"), ref) <= TOL["bf16"]
    check_reduce(c, r, "bf16", "max", True, r0)
    rng = np.random.default_rng(76)
    c0 = to_storage(rng.standard_normal((2304, 2560), dtype=np.float32), "fp16")
    c, r, ref, r0 = run_fused(ctx, 2304, 2560, 256, "fp16", "fp16", 76, kind="max", clear_accum=False, c_init=c0,
                              expect_fused=0)
    assert rel_frobenius(from_storage(c, "fp16"), ref) <= TOL["fp16"]
    check_reduce(c, r, "fp16", "max", True, r0)


def test_execute_kernel_with_fill_and_reduce(ctx):
    """The builder flow end to end: fill C, gemm, reduce C along dim 1, run through ``execute``."""
    import torch

    import frisk_b200 as F
    from tests.test_frontend import build_fused_module
    M, N, K = 512, 384, 256
    a, b = inputs.gemm_inputs(M, N, K, "fp16", False, True, 77, "normal_rsqrt_k")
    ta, tb = to_device(a, "fp16"), to_device(b, "fp16")
    tc = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    tr = torch.zeros(M, dtype=torch.float16, device="cuda")
    F.execute(build_fused_module(fill=0.5, reduce="max"), ta, tb, tc, tr)
    torch.cuda.synchronize()
    base = np.full((M, N), np.float16(0.5))
    ref = gemm_oracle.gemm_fp64(a, b, "fp16", False, True, base, "fp16")
    got = to_host(tc, "fp16")
    assert rel_frobenius(from_storage(got, "fp16"), ref) <= TOL["fp16"]
    assert np.array_equal(from_storage(to_host(tr, "fp16"), "fp16").astype(np.float64),
                          gemm_oracle.row_reduce(got, "fp16", "max"))


def test_fused_epilogue_with_caller_workspace(ctx):
    """The caller may own the scratch of the fused path: the size the library states is enough, less is refused."""
    import torch
    M, N, K = 2304, 2560, 512
    a, b = inputs.gemm_inputs(M, N, K, "fp16", False, True, 78, "normal_rsqrt_k")
    da, db = to_device(a, "fp16"), to_device(b, "fp16")
    dc = torch.empty(M, N, dtype=torch.float16, device="cuda")
    dr = torch.empty(M, dtype=torch.float16, device="cuda")
    desc = capi.gemm_desc(M, N, K, "fp16", "fp16", False, True, clear_accum=True)
    epi = capi.gemm_epilogue(reduce="max", reduce_dst=dr.data_ptr())
    need = capi.gemm_fused_workspace_bytes(desc, epi)
    assert need > 0
    ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    ctx.gemm_fused(desc, epi, da.data_ptr(), db.data_ptr(), dc.data_ptr(), ws.data_ptr(), need, stream=s)
    ctx.check(s)
    got = to_host(dc, "fp16")
    assert rel_frobenius(from_storage(got, "fp16"), gemm_oracle.gemm_fp64(a, b, "fp16", False, True)) <= TOL["fp16"]
    assert np.array_equal(from_storage(to_host(dr, "fp16"), "fp16").astype(np.float64),
                          gemm_oracle.row_reduce(got, "fp16", "max"))
    with pytest.raises(ValueError):
        ctx.gemm_fused(desc, epi, da.data_ptr(), db.data_ptr(), dc.data_ptr(), ws.data_ptr(), need - 4096, stream=s)

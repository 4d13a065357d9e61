"""The CPU oracle against golden vectors made by the reference's own functions
(tests/golden/make_golden.py): this is what pins the oracle."""
import pathlib

import numpy as np
import pytest

from oracle import attention_oracle as ao
from oracle.numerics import bf16_bits_to_f32, f32_to_bf16_bits, rel_frobenius, round_to

GOLDEN = pathlib.Path(__file__).parent / "golden"
NAMES = ("random", "uniform-sparse-value", "last-key-dominant", "tail-uniform", "key-boundary",
         "neutral-extension")
EXACT = ("uniform-sparse-value", "last-key-dominant", "tail-uniform")


@pytest.fixture(scope="module")
def tiled():
    return np.load(GOLDEN / "attention_tiled_d64.npz")


def test_ordered_sum_bit_exact():
    g = np.load(GOLDEN / "ordered_sum.npz")
    for n in (1, 7, 64, 65, 129, 193, 513, 1025):
        got = ao.tree_sum_f32(g[f"n{n}/in"])
        assert np.array_equal(got.view(np.uint32), g[f"n{n}/out"].view(np.uint32)), n


@pytest.mark.parametrize("n", (64, 65, 130))
@pytest.mark.parametrize("name", NAMES)
def test_tiled_d64_matches_reference(tiled, name, n):
    key = f"{name}/n{n}"
    q, k, v = tiled[key + "/q"], tiled[key + "/k"], tiled[key + "/v"]
    strict = ao.attention_fwd(q, k, v, "fp16", 0.125, causal=False, mode="strict")
    fp64 = ao.attention_fwd(q, k, v, "fp16", 0.125, causal=False, mode="fp64")
    assert strict.dtype == np.float32 and fp64.dtype == np.float64
    if name in EXACT:
        # the reference returns closed-form answers for these; the restated numerics
        # must land inside the reference checker's own bound and, for the strict
        # mode, on the very same bits
        assert np.array_equal(strict.view(np.uint32), tiled[key + "/strict"].view(np.uint32))
        assert ao.within_reference_tolerance(fp64, tiled[key + "/fp64"], "fp64") <= 1.0
    else:
        assert np.array_equal(strict.view(np.uint32), tiled[key + "/strict"].view(np.uint32))
        # fp64 sums may associate differently inside BLAS: agree to a few ulps of fp64
        assert np.allclose(fp64, tiled[key + "/fp64"], rtol=1e-12, atol=1e-14)


def test_single_tile_cases_bit_exact():
    g = np.load(GOLDEN / "attention_tile_64x16.npz")
    names = sorted({k.split("/")[0] for k in g.files})
    assert len(names) == 15
    for name in names:
        got = ao.tile_reference(g[name + "/q"], g[name + "/k"], g[name + "/v"])
        assert np.array_equal(got.view(np.uint32), g[name + "/o"].view(np.uint32)), name


def test_cancel_property():
    # zero scores give uniform P; alternating +-1 values cancel exactly
    g = np.load(GOLDEN / "attention_tile_64x16.npz")
    assert not np.any(ao.tile_reference(g["cancelV/q"], g["cancelV/k"], g["cancelV/v"]))


def test_bf16_round_trip_and_rne():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 0.0], np.float32)
    b = f32_to_bf16_bits(x)
    back = bf16_bits_to_f32(b)
    assert back[0] == 1.0 and back[3] == -2.5
    # 1.00390625 = 1 + 2^-8 is a tie between 1.0 and 1+2^-7 -> even mantissa (1.0)
    assert back[1] == 1.0
    # 1.01171875 = 1 + 3*2^-8 ties to 1 + 2^-6 (even)
    assert back[2] == np.float32(1.015625)
    assert np.array_equal(f32_to_bf16_bits(back), b)
    rng = np.random.default_rng(0)
    y = rng.standard_normal(10000).astype(np.float32)
    err = np.abs(round_to(y, "bf16") - y) / np.abs(y)
    assert err.max() <= 2.0 ** -8


def test_causal_first_row_and_mask():
    rng = np.random.default_rng(1)
    q, k, v = (rng.standard_normal((1, 1, 70, 32)).astype(np.float16) for _ in range(3))
    o = ao.attention_fwd(q, k, v, "fp16", 32 ** -0.5, causal=True)
    # query 0 sees only key 0: output is exactly v[0]
    assert np.array_equal(o[0, 0, 0], v[0, 0, 0].astype(np.float64))
    # the last query sees everything: equals the non-causal answer
    full = ao.attention_fwd(q, k, v, "fp16", 32 ** -0.5, causal=False)
    assert np.array_equal(o[0, 0, -1], full[0, 0, -1])
    # changing a future key/value must not change earlier rows
    k2, v2 = k.copy(), v.copy()
    k2[..., 40:, :] = 7
    v2[..., 40:, :] = -3
    o2 = ao.attention_fwd(q, k2, v2, "fp16", 32 ** -0.5, causal=True)
    assert np.array_equal(o[0, 0, :40], o2[0, 0, :40])


def test_strict_and_fp64_agree_loosely():
    rng = np.random.default_rng(2)
    q, k, v = (f32_to_bf16_bits(rng.standard_normal((1, 2, 96, 128)).astype(np.float32)) for _ in range(3))
    a = ao.attention_fwd(q, k, v, "bf16", 128 ** -0.5, causal=True, mode="strict")
    b = ao.attention_fwd(q, k, v, "bf16", 128 ** -0.5, causal=True, mode="fp64")
    assert rel_frobenius(a, b) < 2e-3

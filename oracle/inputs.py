"""Seeded synthetic inputs for the five benchmark workloads (test infrastructure).

Generator: ``numpy.random.default_rng(seed)`` (PCG64), the generator the
reference's own harness uses (``benchmark/layout/execution/run_execution.py:67``,
``tail_attention_reference.py:156``).  Values are drawn as float32 in C order,
tensors in the order listed, from ONE generator per workload, scaled, then
rounded RNE to the storage type.  Multi-GPU shards are slices of these full
host tensors, so results do not depend on the GPU count.

Nothing here reproduces an external dataset: the reference names none, and the
shapes below are fully synthetic.
"""
import math

import numpy as np

from .numerics import to_storage

# name -> description of the workload (sizes as the benchmark states them)
WORKLOADS = {
    "gemm_f32_1024": dict(kind="gemm", M=1024, N=1024, K=1024, dtype_ab="fp32", dtype_c="fp32",
                          trans_a=False, trans_b=False, seed=0, dist="uniform"),
    "gemm_f16_4096_nt": dict(kind="gemm", M=4096, N=4096, K=4096, dtype_ab="fp16", dtype_c="fp16",
                             trans_a=False, trans_b=True, seed=1, dist="normal_rsqrt_k"),
    "gemm_bf16_skinny": dict(kind="gemm", M=16, N=28672, K=8192, dtype_ab="bf16", dtype_c="bf16",
                             trans_a=False, trans_b=True, seed=2, dist="act_weight"),
    "attn_bf16_causal": dict(kind="attention", B=8, H=32, S=4096, D=128, dtype="bf16",
                             causal=True, seed=3),
    "gemm_bf16_deepk": dict(kind="gemm", M=8192, N=8192, K=131072, dtype_ab="bf16", dtype_c="bf16",
                            trans_a=False, trans_b=True, seed=4, dist="normal_rsqrt_k"),
}

_CHUNK = 1 << 24


def _normal(rng, shape, scale):
    """standard_normal(float32) * scale, drawn in row chunks so that a huge
    tensor never needs a second full-size temporary.  Chunked draws consume the
    bit stream exactly like one large draw."""
    out = np.empty(shape, dtype=np.float32)
    flat = out.reshape(-1)
    for lo in range(0, flat.size, _CHUNK):
        hi = min(flat.size, lo + _CHUNK)
        flat[lo:hi] = rng.standard_normal(hi - lo, dtype=np.float32)
    if scale != 1.0:
        out *= np.float32(scale)
    return out


def gemm_inputs(M, N, K, dtype_ab, trans_a=False, trans_b=False, seed=0, dist="uniform", **_):
    """Return (A, B) in device storage form.  A is stored [M,K] (or [K,M] when
    ``trans_a``), B is stored [K,N] (or [N,K] when ``trans_b``): transposes are
    flags on the op, never strides (``LegacyImportSemantics.cpp:37-40``)."""
    rng = np.random.default_rng(seed)
    a_shape = (K, M) if trans_a else (M, K)
    b_shape = (N, K) if trans_b else (K, N)
    if dist == "uniform":
        a = rng.random(a_shape, dtype=np.float32) * np.float32(2) - np.float32(1)
        b = rng.random(b_shape, dtype=np.float32) * np.float32(2) - np.float32(1)
    elif dist == "normal_rsqrt_k":
        s = 1.0 / math.sqrt(K)
        a = _normal(rng, a_shape, s)
        b = _normal(rng, b_shape, s)
    elif dist == "act_weight":
        a = _normal(rng, a_shape, 1.0)
        b = _normal(rng, b_shape, 0.02)
    else:
        raise ValueError(f"unknown distribution {dist!r}")
    return to_storage(a, dtype_ab), to_storage(b, dtype_ab)


def gemm_inputs_streamed(M, N, K, dtype_ab, trans_a=False, trans_b=False, seed=0, dist="normal_rsqrt_k",
                         chunk_rows=128, storage=True, **_):
    """The same values as :func:`gemm_inputs`, yielded as ``(name, first_row, rows_in_storage_form)``
    row blocks of the A buffer and then of the B buffer, so that a tensor too large to hold
    twice on the host (the deep-K workload: 2 x 2 GiB) can be sent to the device piece by piece
    while the caller keeps only the rows its sampled check needs.  Row blocks of a normal
    draw consume the generator exactly like one large draw.  ``storage=False`` yields the scaled
    fp32 values before the rounding to ``dtype_ab`` (for callers that round on the device)."""
    if dist not in ("normal_rsqrt_k", "act_weight"):
        raise ValueError("streamed inputs exist for the normal distributions only")
    rng = np.random.default_rng(seed)
    a_shape = (K, M) if trans_a else (M, K)
    b_shape = (N, K) if trans_b else (K, N)
    scales = (1.0 / math.sqrt(K),) * 2 if dist == "normal_rsqrt_k" else (1.0, 0.02)
    for name, shape, scale in (("a", a_shape, scales[0]), ("b", b_shape, scales[1])):
        for r0 in range(0, shape[0], chunk_rows):
            rows = min(chunk_rows, shape[0] - r0)
            vals = _normal(rng, (rows, shape[1]), scale)
            yield name, r0, (to_storage(vals, dtype_ab) if storage else vals)


def attention_inputs(B, H, S, D, dtype="bf16", seed=3, **_):
    """Q, K, V as compact BHSD arrays in storage form, N(0,1), drawn in that order."""
    rng = np.random.default_rng(seed)
    return tuple(to_storage(_normal(rng, (B, H, S, D), 1.0), dtype) for _ in range(3))


def workload_inputs(name, **override):
    spec = dict(WORKLOADS[name])
    spec.update(override)
    if spec["kind"] == "gemm":
        return spec, gemm_inputs(**spec)
    return spec, attention_inputs(**spec)

"""CPU restatement of the ``frisk.gemm`` contract (test infrastructure).

PARITY UNPINNED: the reference executes no standalone GEMM and its tests hold
no GEMM result, so there is no golden vector to check this file against.  It
restates the op's documented contract instead:

* ``C <- (clear_accum ? 0 : C) + op(A) . op(B)``; A, B are read, C is written
  and, unless ``clear_accum``, also read
  (``lib/Dialect/Frisk/IR/FriskOps.cpp:416-426``).
* transposes are flags: effective A is MxK, effective B is KxN, ``trans_b``
  means the B buffer is NxK (``lib/Dialect/Frisk/IR/LegacyImportSemantics.cpp:37-44``).
* A and B share one element type; C has the same type or f32 for f16/bf16
  inputs (``LegacyImportSemantics.cpp:26-35``).
* products of the ROUNDED inputs are accumulated in at least fp32 and rounded
  once to the output type; the oracle accumulates in fp64.
"""
import numpy as np

from .numerics import from_storage, round_to


def validation_error(a_shape, b_shape, c_shape, dtype_ab_a, dtype_ab_b, dtype_c,
                     trans_a, trans_b, m, n, k):
    """String the reference would raise, or None
    (``LegacyImportSemantics.cpp:11-46``; same prefixes)."""
    if len(a_shape) != 2 or len(b_shape) != 2 or len(c_shape) != 2:
        return "legacy-gemm-shape: A, B, and C must have rank 2"
    if any(d < 0 for d in tuple(a_shape) + tuple(b_shape) + tuple(c_shape)):
        return "legacy-gemm-shape: A, B, and C must have static shapes"
    if m <= 0 or n <= 0 or k <= 0:
        return "legacy-gemm-shape: M, N, and K must be positive"
    if dtype_ab_a != dtype_ab_b:
        return "legacy-gemm-type: A and B must have the same element type"
    same = dtype_c == dtype_ab_a
    low_f32 = dtype_ab_a in ("fp16", "bf16") and dtype_c == "fp32"
    if not same and not low_f32:
        return "legacy-gemm-type: C must match A/B or be f32 for f16/bf16 inputs"
    a_m, a_k = (a_shape[1], a_shape[0]) if trans_a else (a_shape[0], a_shape[1])
    b_k, b_n = (b_shape[1], b_shape[0]) if trans_b else (b_shape[0], b_shape[1])
    if a_m != m or a_k != k or b_k != k or b_n != n:
        return "legacy-gemm-shape: effective A/B shapes must match M/N/K"
    if c_shape[0] != m or c_shape[1] != n:
        return "legacy-gemm-shape: C shape must be MxN"
    return None


def _effective(a_store, b_store, dtype_ab, trans_a, trans_b):
    a = from_storage(a_store, dtype_ab).astype(np.float64)
    b = from_storage(b_store, dtype_ab).astype(np.float64)
    return (a.T if trans_a else a), (b.T if trans_b else b)


def gemm_fp64(a_store, b_store, dtype_ab, trans_a=False, trans_b=False, c_init=None, dtype_c=None):
    """Full MxN product in fp64, NOT rounded to the output type.  ``c_init`` is the
    stored C for ``clear_accum=False``."""
    a, b = _effective(a_store, b_store, dtype_ab, trans_a, trans_b)
    out = a @ b
    if c_init is not None:
        out = out + from_storage(c_init, dtype_c).astype(np.float64)
    return out


def gemm_rounded(a_store, b_store, dtype_ab, dtype_c, trans_a=False, trans_b=False, c_init=None):
    """The value the op's output buffer holds: one rounding to ``dtype_c``."""
    return round_to(gemm_fp64(a_store, b_store, dtype_ab, trans_a, trans_b, c_init, dtype_c), dtype_c)


def gemm_sampled_fp64(a_store, b_store, dtype_ab, rows, cols, trans_a=False, trans_b=False):
    """fp64 products for the cross ``rows x cols`` with the full K extent — the form
    used where the whole product is out of reach for a CPU (deep-K workload)."""
    a = from_storage(a_store, dtype_ab)
    b = from_storage(b_store, dtype_ab)
    a_rows = (a[:, rows].T if trans_a else a[rows, :]).astype(np.float64)
    b_cols = (b[cols, :].T if trans_b else b[:, cols]).astype(np.float64)
    return a_rows @ b_cols


def gemm_f32_blas(a_store, b_store, dtype_ab, trans_a=False, trans_b=False):
    """fp32 BLAS product of the rounded inputs: the timed CPU baseline (all host
    threads), not a checker."""
    a = from_storage(a_store, dtype_ab)
    b = from_storage(b_store, dtype_ab)
    return (a.T if trans_a else a) @ (b.T if trans_b else b)


def row_reduce(c_storage, dtype_c, kind, dst_init=None):
    """``frisk.reduce`` of C along dim 1 (lib/Dialect/Frisk/IR/FriskOps.cpp:728-762): over the values
    of C as stored, combined in fp64 (exact for max/min), optionally with the destination's
    earlier contents (clear = false).  Returns fp64, not rounded."""
    c = from_storage(c_storage, dtype_c).astype(np.float64)
    if kind == "max":
        r = c.max(axis=1)
    elif kind == "min":
        r = c.min(axis=1)
    elif kind == "add":
        r = c.sum(axis=1)
    else:
        raise ValueError(f"unsupported reduce kind: {kind}. Supported: add, mul, min, max")
    if dst_init is not None:
        d = from_storage(dst_init, dtype_c).astype(np.float64)
        r = np.maximum(r, d) if kind == "max" else np.minimum(r, d) if kind == "min" else r + d
    return r

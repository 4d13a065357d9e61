"""Storage-type helpers for the CPU oracle (test infrastructure, not product).

numpy has no bfloat16, so 16-bit brain floats travel as ``uint16`` bit patterns
(the upper half of the IEEE fp32 word).  Rounding is round-to-nearest-even, the
conversion ``cvt.rn`` performs in the reference's emitted kernels
(``benchmark/layout/execution/tiled_attention.py:628-629``).
"""
import numpy as np

DTYPES = ("fp32", "fp16", "bf16")
ITEMSIZE = {"fp32": 4, "fp16": 2, "bf16": 2}


def f32_to_bf16_bits(x):
    """fp32 array -> uint16 bf16 bit patterns, RNE; NaN stays NaN."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    u = x.view(np.uint32)
    r = u >> np.uint32(16)              # one temporary, updated in place from here on
    r &= np.uint32(1)
    r += np.uint32(0x7FFF)
    r += u
    r >>= np.uint32(16)
    r = r.astype(np.uint16)
    nan = np.isnan(x)
    if nan.any():
        r = np.where(nan, np.uint16(0x7FC0), r)
    return r


def bf16_bits_to_f32(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    return (b.astype(np.uint32) << 16).view(np.float32)


def _f64_to_bf16_value(x):
    """fp64 -> nearest bf16 value (RNE), returned as fp32, with ONE rounding
    (going through fp32 first would round twice)."""
    x = np.asarray(x, dtype=np.float64)
    m, e = np.frexp(x)                       # x = m * 2**e, 0.5 <= |m| < 1
    normal = np.ldexp(np.rint(m * 256.0), e - 8)          # 8 significant bits
    tiny = np.ldexp(np.rint(np.ldexp(x, 133)), -133)      # bf16 subnormal quantum 2**-133
    out = np.where(np.abs(x) < 2.0 ** -126, tiny, normal)
    out = np.where(np.isfinite(x), out, x)
    with np.errstate(over="ignore"):
        out = np.where(np.abs(out) >= 2.0 ** 128, np.copysign(np.inf, x), out).astype(np.float32)
    return out


def round_to(x, dtype):
    """Round an fp32/fp64 array ONCE to ``dtype`` and return it widened to fp32."""
    x = np.asarray(x)
    if dtype == "fp32":
        return x.astype(np.float32)
    if dtype == "fp16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        if x.dtype == np.float64:
            return _f64_to_bf16_value(x)
        return bf16_bits_to_f32(f32_to_bf16_bits(x.astype(np.float32)))
    raise ValueError(f"unknown dtype {dtype!r}")


def to_storage(x, dtype):
    """fp32 values -> the array a device buffer of ``dtype`` holds
    (float32 / float16 / uint16-bits for bf16)."""
    if dtype == "fp32":
        return np.ascontiguousarray(x, dtype=np.float32)
    if dtype == "fp16":
        return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16)
    if dtype == "bf16":
        return f32_to_bf16_bits(x)
    raise ValueError(f"unknown dtype {dtype!r}")


def from_storage(a, dtype):
    """Inverse of :func:`to_storage`, widened to fp32."""
    if dtype == "fp32":
        return np.asarray(a, dtype=np.float32)
    if dtype == "fp16":
        return np.asarray(a, dtype=np.float16).astype(np.float32)
    if dtype == "bf16":
        return bf16_bits_to_f32(a)
    raise ValueError(f"unknown dtype {dtype!r}")


def rel_frobenius(got, ref):
    """||got - ref||_F / ||ref||_F evaluated in fp64."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.sqrt((ref * ref).sum())
    num = np.sqrt(((got - ref) ** 2).sum())
    if den == 0.0:
        return 0.0 if num == 0.0 else float("inf")
    return float(num / den)

"""CPU restatement of the reference's attention-forward numerics (test infrastructure).

PINNED against golden vectors produced by running the reference's own functions
(``tests/golden/make_golden.py`` -> ``tests/golden/attention_*.npz``).

Follows, per head (compact BHSD, ``tail_attention_reference.py:39-41``):

* ``fp64`` mode — ``tail_attention_reference.py:81-85,104-110``: fp64 dots, score
  times the fp32 scale, stable softmax in fp64, probabilities ROUNDED TO THE
  16-BIT INPUT TYPE, then P.V in fp64.
* ``strict`` mode — ``tail_attention_reference.py:74-78``: fp64 dot rounded to
  fp32, ``* scale`` in fp32, minus the row maximum, ``exp2(x * log2e_f32)`` in
  fp32, division by the fp32 row sum taken in the emitted kernel's fixed
  balanced-tree order (``:49-71``), P rounded to 16 bits, P.V in fp64 stored as
  fp32.
* single 64x16 tile — ``run_execution.py:59-64``: sequential fp32 accumulation
  over k, scale 0.25, fp32 ``exp``, fp32 row sum, P to fp16, sequential fp32 P.V.

Extensions the benchmark workloads need and the reference lacks (it has
key-prefix masking only, ``tiled_attention.py:421-430``): a causal mask
(key j visible to query i iff j <= i + S_kv - S_q), any head dimension, any
scale, bf16 probabilities.  With ``causal=False``, D=64, scale=0.125 and fp16
the functions reduce to the reference's.
"""
import numpy as np

from .numerics import from_storage, round_to

LOG2_E_F32 = np.array(0x3FB8AA3B, dtype=np.uint32).view(np.float32)[()]
# tolerances of the reference's own checker (tail_attention_reference.py:19)
REFERENCE_ERROR = dict(strict_atol=3e-5, strict_rtol=3e-4, fp64_atol=4e-5, fp64_rtol=4e-4)
_Q_CHUNK = 256


def tree_sum_f32(e):
    """Row sum of fp32 ``e`` (last axis) in the order the reference kernel uses:
    thread-lane L of a 4-lane row group owns column pairs (8j+2L, 8j+2L+1); each lane
    reduces its values (zero-padded to a power of two) by a balanced binary tree;
    lanes combine as (0+1)+(2+3).  Every add rounds to fp32."""
    e = np.asarray(e)
    if e.dtype != np.float32 or e.ndim == 0 or e.shape[-1] == 0:
        raise ValueError("expected a non-empty fp32 row")
    n = e.shape[-1]
    per_lane = []
    for lane in range(4):
        first = np.arange(2 * lane, n, 8)
        idx = np.stack([first, first + 1], axis=1).ravel()
        idx = idx[idx < n]
        if idx.size == 0:
            per_lane.append(np.zeros(e.shape[:-1], np.float32))
            continue
        width = 1
        while width < idx.size:
            width *= 2
        buf = np.zeros(e.shape[:-1] + (width,), np.float32)
        buf[..., :idx.size] = e[..., idx]
        while buf.shape[-1] > 1:
            buf = (buf[..., 0::2] + buf[..., 1::2]).astype(np.float32)
        per_lane.append(buf[..., 0])
    lo = (per_lane[0] + per_lane[1]).astype(np.float32)
    hi = (per_lane[2] + per_lane[3]).astype(np.float32)
    return (lo + hi).astype(np.float32)[..., None]


def _mask(s_q, s_kv, q_lo, q_hi):
    """True where key j is hidden from query i (bottom-right aligned causal)."""
    i = np.arange(q_lo, q_hi)[:, None] + (s_kv - s_q)
    j = np.arange(s_kv)[None, :]
    return j > i


def _p_fp64(dot, scale32, hidden, p_dtype):
    s = dot * np.float64(scale32)
    if hidden is not None:
        s = np.where(hidden, -np.inf, s)
    c = s - s.max(axis=-1, keepdims=True)
    e = np.exp(c)
    return round_to(e / e.sum(axis=-1, keepdims=True), p_dtype).astype(np.float64)


def _p_strict(dot, scale32, hidden, p_dtype):
    s = (dot.astype(np.float32) * scale32).astype(np.float32)
    if hidden is not None:
        s = np.where(hidden, np.float32(-np.inf), s)
    c = (s - s.max(axis=-1, keepdims=True)).astype(np.float32)
    e = np.exp2((c * LOG2_E_F32).astype(np.float32)).astype(np.float32)
    return round_to((e / tree_sum_f32(e)).astype(np.float32), p_dtype).astype(np.float64)


def attention_head(q, k, v, scale, causal=False, mode="fp64", p_dtype="fp16", rows=None):
    """One head: q [S_q,D], k/v [S_kv,D] widened fp32 -> O [len(rows) or S_q, D].
    fp64 for ``fp64`` mode, fp32 for ``strict``; the output is NOT rounded to a
    16-bit output type (the stricter comparison)."""
    s_q, s_kv = q.shape[0], k.shape[0]
    scale32 = np.float32(scale)
    kt = k.astype(np.float64).T
    vv = v.astype(np.float64)
    prob = _p_fp64 if mode == "fp64" else _p_strict
    sel = np.arange(s_q) if rows is None else np.asarray(rows)
    out = np.empty((len(sel), v.shape[1]), np.float64 if mode == "fp64" else np.float32)
    with np.errstate(under="ignore"):
        for lo in range(0, len(sel), _Q_CHUNK):
            r = sel[lo:lo + _Q_CHUNK]
            dot = q[r].astype(np.float64) @ kt
            hidden = None
            if causal:
                hidden = np.arange(s_kv)[None, :] > (r[:, None] + (s_kv - s_q))
            out[lo:lo + len(r)] = prob(dot, scale32, hidden, p_dtype) @ vv
    return out


def attention_fwd(q_store, k_store, v_store, dtype, scale, causal=False, mode="fp64", heads=None):
    """BHSD attention forward over storage-form arrays.  ``heads`` optionally
    restricts the work to a list of flat (b*H+h) indices (the sampled check used
    at full benchmark size); the result then has shape [len(heads), S_q, D]."""
    q = from_storage(q_store, dtype)
    k = from_storage(k_store, dtype)
    v = from_storage(v_store, dtype)
    b, h, s_q, d = q.shape
    s_kv = k.shape[2]
    qf, kf, vf = q.reshape(b * h, s_q, d), k.reshape(b * h, s_kv, d), v.reshape(b * h, s_kv, d)
    sel = range(b * h) if heads is None else heads
    out = np.stack([attention_head(qf[i], kf[i], vf[i], scale, causal, mode, dtype) for i in sel])
    return out.reshape(b, h, s_q, d) if heads is None else out


def tile_reference(q, k, v):
    """The 64x16 single-tile check: fp32 everywhere, k accumulated in index order."""
    q, k, v = (np.asarray(x).astype(np.float32) for x in (q, k, v))
    s = np.zeros((q.shape[0], k.shape[0]), np.float32)
    for t in range(q.shape[1]):
        s = (s + (q[:, t, None] * k[None, :, t]).astype(np.float32)).astype(np.float32)
    s = (s * np.float32(0.25)).astype(np.float32)
    e = np.exp((s - s.max(axis=1, keepdims=True)).astype(np.float32), dtype=np.float32)
    p = (e / e.sum(axis=1, keepdims=True, dtype=np.float32)).astype(np.float32)
    p = p.astype(np.float16).astype(np.float32)
    o = np.zeros((q.shape[0], v.shape[1]), np.float32)
    for t in range(k.shape[0]):
        o = (o + (p[:, t, None] * v[None, t, :]).astype(np.float32)).astype(np.float32)
    return o


def within_reference_tolerance(observed, ref, mode):
    """The reference checker's bound: |err| <= atol + rtol*|ref| for ``mode``."""
    err = np.abs(np.asarray(observed, np.float64) - np.asarray(ref, np.float64))
    bound = REFERENCE_ERROR[mode + "_atol"] + REFERENCE_ERROR[mode + "_rtol"] * np.abs(ref)
    return float((err / bound).max())

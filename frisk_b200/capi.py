"""ctypes binding of ``libfrisk_b200.so`` (the C ABI of ``include/frisk_b200.h``).

There is no CPU fallback: if the library is missing every call raises.  Error
codes become exceptions the way the reference's bindings raise them
(``ffi/ir.cpp:333-341``: ``std::invalid_argument`` -> ``ValueError`` with the
``legacy-gemm-shape`` / ``legacy-gemm-type`` prefixes); device or CUDA failures
become ``RuntimeError``.
"""
import ctypes
import os
import pathlib

F32, F16, BF16 = 0, 1, 2
ALGO_AUTO, ALGO_SIMT_F32, ALGO_TCGEN05, ALGO_SKINNY, ALGO_TCGEN05_PAIR, ALGO_F32_SPLIT = 0, 1, 2, 3, 4, 5
DTYPE_CODE = {"fp32": F32, "fp16": F16, "bf16": BF16}
DTYPE_NAME = {v: k for k, v in DTYPE_CODE.items()}
ITEMSIZE = {F32: 4, F16: 2, BF16: 2}

LIB_PATH = pathlib.Path(__file__).resolve().parent / "lib" / "libfrisk_b200.so"

# every symbol include/frisk_b200.h declares
EXPORTS = (
    "frisk_b200_ctx_create", "frisk_b200_ctx_destroy", "frisk_b200_last_status", "frisk_b200_last_cuda",
    "frisk_b200_strerror", "frisk_b200_version", "frisk_b200_gemm_validate", "frisk_b200_gemm_check_memrefs",
    "frisk_b200_gemm_select", "frisk_b200_gemm_workspace_bytes", "frisk_b200_gemm", "frisk_b200_gemm_host",
    "frisk_b200_attention_validate", "frisk_b200_attention_workspace_bytes", "frisk_b200_attention_fwd",
    "frisk_b200_attention_fwd_host", "frisk_b200_convert_f32", "frisk_b200_check",
    "frisk_b200_gemm_skinny_static", "frisk_b200_gemm_push", "frisk_b200_sum_slots",
    "frisk_b200_peer_buffer_create", "frisk_b200_peer_buffer_open", "frisk_b200_peer_buffer_close",
    "frisk_b200_gemm_fused_select", "frisk_b200_gemm_fused_workspace_bytes", "frisk_b200_gemm_fused",
)


class GemmDesc(ctypes.Structure):
    _fields_ = [("M", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
                ("trans_a", ctypes.c_int32), ("trans_b", ctypes.c_int32), ("clear_accum", ctypes.c_int32),
                ("dtype_ab", ctypes.c_int32), ("dtype_c", ctypes.c_int32),
                ("lda", ctypes.c_int64), ("ldb", ctypes.c_int64), ("ldc", ctypes.c_int64),
                ("policy", ctypes.c_int32), ("algo", ctypes.c_int32)]


class GemmEpilogue(ctypes.Structure):
    _fields_ = [("fill_enable", ctypes.c_int32), ("fill_value", ctypes.c_float), ("reduce_kind", ctypes.c_int32),
                ("reduce_clear", ctypes.c_int32), ("reduce_dst", ctypes.c_void_p)]


REDUCE_KIND = {None: 0, "max": 1, "min": 2, "add": 3}


def gemm_epilogue(fill=None, reduce=None, reduce_dst=None, reduce_clear=True):
    """``fill``: value C was filled with right before an accumulating gemm; ``reduce``: kind of the
    ``frisk.reduce`` along dim 1 right after it ('max' | 'min' | 'add'; 'mul' has no kernel)."""
    if reduce not in REDUCE_KIND:
        raise ValueError(f"frisk-b200: no kernel for reduce kind {reduce!r}")
    e = GemmEpilogue()
    e.fill_enable = 0 if fill is None else 1
    e.fill_value = 0.0 if fill is None else float(fill)
    e.reduce_kind = REDUCE_KIND[reduce]
    e.reduce_clear = 1 if reduce_clear else 0
    e.reduce_dst = reduce_dst
    return e


class AttnDesc(ctypes.Structure):
    _fields_ = [("B", ctypes.c_int32), ("H", ctypes.c_int32), ("S_q", ctypes.c_int32), ("S_kv", ctypes.c_int32),
                ("D", ctypes.c_int32), ("scale", ctypes.c_float), ("causal", ctypes.c_int32),
                ("dtype_in", ctypes.c_int32), ("dtype_out", ctypes.c_int32), ("normalize_p", ctypes.c_int32)]


_lib = None


def load():
    """Load the shared library (once).  Raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    path = pathlib.Path(os.environ.get("FRISK_B200_LIB", LIB_PATH))  # override: try a differently built library
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: build it with `python -m frisk_b200.build` "
            "(there is no CPU fallback for the GEMM / attention kernels)")
    lib = ctypes.CDLL(os.fspath(path))
    vp, sz, i32, i64 = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int32, ctypes.c_int64
    gd, ad, ge = ctypes.POINTER(GemmDesc), ctypes.POINTER(AttnDesc), ctypes.POINTER(GemmEpilogue)
    sig = {
        "frisk_b200_ctx_create": (ctypes.c_int, [ctypes.POINTER(vp), ctypes.c_int]),
        "frisk_b200_ctx_destroy": (ctypes.c_int, [vp]),
        "frisk_b200_last_status": (ctypes.c_int, [vp]),
        "frisk_b200_last_cuda": (ctypes.c_int, [vp]),
        "frisk_b200_strerror": (ctypes.c_char_p, [ctypes.c_int]),
        "frisk_b200_version": (ctypes.c_char_p, []),
        "frisk_b200_gemm_validate": (ctypes.c_int, [gd]),
        "frisk_b200_gemm_check_memrefs": (ctypes.c_int, [i32, ctypes.POINTER(i64), i32, i32, ctypes.POINTER(i64), i32,
                                                         i32, ctypes.POINTER(i64), i32, i32, i32, i64, i64, i64,
                                                         ctypes.POINTER(ctypes.c_char_p)]),
        "frisk_b200_gemm_select": (ctypes.c_int, [gd]),
        "frisk_b200_gemm_workspace_bytes": (sz, [gd]),
        "frisk_b200_gemm": (ctypes.c_int, [vp, gd, vp, vp, vp, vp, sz, vp]),
        "frisk_b200_gemm_host": (ctypes.c_int, [vp, gd, vp, vp, vp]),
        "frisk_b200_attention_validate": (ctypes.c_int, [ad]),
        "frisk_b200_attention_workspace_bytes": (sz, [ad]),
        "frisk_b200_attention_fwd": (ctypes.c_int, [vp, ad, vp, vp, vp, vp, vp, sz, vp]),
        "frisk_b200_attention_fwd_host": (ctypes.c_int, [vp, ad, vp, vp, vp, vp]),
        "frisk_b200_convert_f32": (ctypes.c_int, [vp, vp, vp, i64, i32, vp]),
        "frisk_b200_check": (ctypes.c_int, [vp, vp]),
        "frisk_b200_gemm_skinny_static": (ctypes.c_int, [ctypes.c_int, gd, vp, vp, vp, vp]),
        "frisk_b200_gemm_push": (ctypes.c_int, [vp, gd, vp, vp, ctypes.POINTER(vp), i32, i64, i64, vp]),
        "frisk_b200_sum_slots": (ctypes.c_int, [vp, vp, i32, i64, vp, i64, i32, vp]),
        "frisk_b200_peer_buffer_create": (ctypes.c_int, [vp, sz, ctypes.POINTER(vp), vp]),
        "frisk_b200_peer_buffer_open": (ctypes.c_int, [vp, vp, ctypes.POINTER(vp)]),
        "frisk_b200_peer_buffer_close": (ctypes.c_int, [vp, vp, i32]),
        "frisk_b200_gemm_fused_select": (ctypes.c_int, [gd, ge]),
        "frisk_b200_gemm_fused_workspace_bytes": (sz, [gd, ge]),
        "frisk_b200_gemm_fused": (ctypes.c_int, [vp, gd, ge, vp, vp, vp, vp, sz, vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def strerror(code):
    return load().frisk_b200_strerror(code).decode()


def raise_for(code, ctx=None):
    """0 -> None; negative (host contract) -> ValueError; positive -> RuntimeError."""
    if code == 0:
        return
    msg = strerror(code)
    if code < 0:
        raise ValueError(msg)
    detail = ""
    if ctx is not None:
        lib = load()
        detail = f" (device status 0x{lib.frisk_b200_last_status(ctx) & 0xffffffff:x}, cuda error {lib.frisk_b200_last_cuda(ctx)})"
    raise RuntimeError(msg + detail)


def gemm_desc(M, N, K, dtype_ab, dtype_c=None, trans_a=False, trans_b=False, clear_accum=True,
              lda=0, ldb=0, ldc=0, algo=ALGO_AUTO):
    code_ab = DTYPE_CODE[dtype_ab] if isinstance(dtype_ab, str) else dtype_ab
    code_c = code_ab if dtype_c is None else (DTYPE_CODE[dtype_c] if isinstance(dtype_c, str) else dtype_c)
    return GemmDesc(M, N, K, int(trans_a), int(trans_b), int(clear_accum), code_ab, code_c, lda, ldb, ldc, 0, algo)


def attn_desc(B, H, S_q, S_kv, D, scale, causal, dtype_in, dtype_out=None, normalize_p=False):
    code_in = DTYPE_CODE[dtype_in] if isinstance(dtype_in, str) else dtype_in
    code_out = code_in if dtype_out is None else (DTYPE_CODE[dtype_out] if isinstance(dtype_out, str) else dtype_out)
    return AttnDesc(B, H, S_q, S_kv, D, float(scale), int(bool(causal)), code_in, code_out, int(bool(normalize_p)))


class Context:
    """Owns a ``frisk_b200_ctx`` on one device."""

    def __init__(self, device=0):
        lib = load()
        h = ctypes.c_void_p()
        raise_for(lib.frisk_b200_ctx_create(ctypes.byref(h), device))
        self._h = h
        self.device = device

    @property
    def handle(self):
        if self._h is None:
            raise RuntimeError("context already destroyed")
        return self._h

    def close(self):
        if self._h is not None:
            load().frisk_b200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- raw pointer calls ---------------------------------------------------------
    def gemm(self, desc, a_ptr, b_ptr, c_ptr, ws_ptr=None, ws_bytes=0, stream=None):
        rc = load().frisk_b200_gemm(self.handle, ctypes.byref(desc), a_ptr, b_ptr, c_ptr, ws_ptr, ws_bytes, stream)
        raise_for(rc, self._h)

    def gemm_fused(self, desc, epi, a_ptr, b_ptr, c_ptr, ws_ptr=None, ws_bytes=0, stream=None):
        rc = load().frisk_b200_gemm_fused(self.handle, ctypes.byref(desc), ctypes.byref(epi), a_ptr, b_ptr, c_ptr,
                                          ws_ptr, ws_bytes, stream)
        raise_for(rc, self._h)

    def gemm_host(self, desc, a_ptr, b_ptr, c_ptr):
        raise_for(load().frisk_b200_gemm_host(self.handle, ctypes.byref(desc), a_ptr, b_ptr, c_ptr), self._h)

    def attention_fwd(self, desc, q, k, v, o, stream=None):
        rc = load().frisk_b200_attention_fwd(self.handle, ctypes.byref(desc), q, k, v, o, None, 0, stream)
        raise_for(rc, self._h)

    def attention_fwd_host(self, desc, q, k, v, o):
        raise_for(load().frisk_b200_attention_fwd_host(self.handle, ctypes.byref(desc), q, k, v, o), self._h)

    def convert_f32(self, src_ptr, dst_ptr, count, dtype, stream=None):
        code = DTYPE_CODE[dtype] if isinstance(dtype, str) else dtype
        raise_for(load().frisk_b200_convert_f32(self.handle, src_ptr, dst_ptr, count, code, stream), self._h)

    def gemm_push(self, desc, a_ptr, b_ptr, targets, rows_per_target, ld_target, stream=None):
        arr = (ctypes.c_void_p * len(targets))(*targets)
        rc = load().frisk_b200_gemm_push(self.handle, ctypes.byref(desc), a_ptr, b_ptr, arr, len(targets),
                                         rows_per_target, ld_target, stream)
        raise_for(rc, self._h)

    def sum_slots(self, slots_ptr, n_slots, slot_elems, dst_ptr, count, dtype, stream=None):
        code = DTYPE_CODE[dtype] if isinstance(dtype, str) else dtype
        raise_for(load().frisk_b200_sum_slots(self.handle, slots_ptr, n_slots, slot_elems, dst_ptr, count, code,
                                              stream), self._h)

    def peer_buffer_create(self, nbytes):
        """-> (device pointer, 64-byte handle) of a zeroed buffer other processes can map."""
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        raise_for(load().frisk_b200_peer_buffer_create(self.handle, nbytes, ctypes.byref(ptr), handle), self._h)
        return ptr.value, handle.raw

    def peer_buffer_open(self, handle):
        ptr = ctypes.c_void_p()
        buf = ctypes.create_string_buffer(handle, 64)
        raise_for(load().frisk_b200_peer_buffer_open(self.handle, buf, ctypes.byref(ptr)), self._h)
        return ptr.value

    def peer_buffer_close(self, ptr, owned):
        raise_for(load().frisk_b200_peer_buffer_close(self.handle, ptr, int(bool(owned))), self._h)

    def check(self, stream=None):
        raise_for(load().frisk_b200_check(self.handle, stream), self._h)


def gemm_fused_select(desc, epi):
    """1: fill / reduce run inside the GEMM epilogue; 0: composed from separate kernels.  Host-only."""
    rc = load().frisk_b200_gemm_fused_select(ctypes.byref(desc), ctypes.byref(epi))
    if rc < 0:
        raise_for(rc)
    return rc


def gemm_fused_workspace_bytes(desc, epi):
    return load().frisk_b200_gemm_fused_workspace_bytes(ctypes.byref(desc), ctypes.byref(epi))


def gemm_check_memrefs(a_shape, a_dtype, b_shape, b_dtype, c_shape, c_dtype, trans_a, trans_b, m, n, k):
    """Host-only contract check over memref shapes (no GPU needed).
    Returns (code, message-or-None); message is the reference's text."""
    def arr(shape):
        return (ctypes.c_int64 * max(1, len(shape)))(*shape)
    msg = ctypes.c_char_p()
    code = load().frisk_b200_gemm_check_memrefs(
        len(a_shape), arr(a_shape), a_dtype, len(b_shape), arr(b_shape), b_dtype,
        len(c_shape), arr(c_shape), c_dtype, int(trans_a), int(trans_b), m, n, k, ctypes.byref(msg))
    return code, (msg.value.decode() if msg.value else None)

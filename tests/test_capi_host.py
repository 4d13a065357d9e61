"""Host-only checks of the C ABI: the library loads, exports every symbol the header
declares, and its contract checks agree with the oracle's restatement of
LegacyImportSemantics.cpp:11-46.  No compute call is made here."""
import ctypes
import itertools
import pathlib
import re

import pytest

from frisk_b200 import capi
from oracle import gemm_oracle

HEADER = pathlib.Path(__file__).resolve().parents[1] / "include" / "frisk_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"\b(frisk_b200_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    lib = capi.load()
    names = declared_symbols()
    assert len(names) >= 18
    for name in names:
        assert getattr(lib, name) is not None
    assert set(names) == set(capi.EXPORTS)


def test_version_and_strerror():
    lib = capi.load()
    assert b"sm_100a" in lib.frisk_b200_version()
    assert capi.strerror(-1).startswith("legacy-gemm-shape")
    assert capi.strerror(-2).startswith("legacy-gemm-type")
    assert capi.strerror(0) == "ok"


def test_memref_contract_matches_oracle_restatement():
    names = {capi.F32: "fp32", capi.F16: "fp16", capi.BF16: "bf16"}
    shapes = [(64, 16), (16, 64), (64, 64), (8, 64), (64, 8)]
    n_bad = n_ok = 0
    for a, b, c in itertools.product(shapes, repeat=3):
        for ta, tb in itertools.product((0, 1), repeat=2):
            for da, db, dc in ((1, 1, 1), (1, 1, 0), (2, 2, 0), (1, 2, 0), (0, 0, 1), (0, 0, 0), (2, 2, 1)):
                m, k = (a[1], a[0]) if ta else a
                n = b[0] if tb else b[1]
                code, msg = capi.gemm_check_memrefs(a, da, b, db, c, dc, ta, tb, m, n, k)
                want = gemm_oracle.validation_error(a, b, c, names[da], names[db], names[dc], ta, tb, m, n, k)
                assert msg == want, (a, b, c, ta, tb, da, db, dc)
                assert (code == 0) == (want is None)
                n_bad += code != 0
                n_ok += code == 0
    assert n_bad > 100 and n_ok > 20


def test_rank_and_sign_checks():
    assert capi.gemm_check_memrefs((4,), 1, (4, 4), 1, (4, 4), 1, 0, 0, 4, 4, 4)[1].endswith("must have rank 2")
    assert capi.gemm_check_memrefs((4, -1), 1, (4, 4), 1, (4, 4), 1, 0, 0, 4, 4, 4)[1].endswith("static shapes")
    assert capi.gemm_check_memrefs((0, 4), 1, (4, 4), 1, (0, 4), 1, 0, 0, 0, 4, 4)[1].endswith("must be positive")


def test_kernel_selection_and_workspace():
    lib = capi.load()
    sel = lambda d: lib.frisk_b200_gemm_select(d)  # noqa: E731
    # fp32: the split-bf16 tensor-core path where it pays and the extents allow it, else the CUDA cores
    assert sel(capi.gemm_desc(1024, 1024, 1024, "fp32")) == capi.ALGO_F32_SPLIT
    assert sel(capi.gemm_desc(1024, 1024, 1024, "fp32", algo=capi.ALGO_SIMT_F32)) == capi.ALGO_SIMT_F32
    assert sel(capi.gemm_desc(1024, 1024, 1023, "fp32")) == capi.ALGO_SIMT_F32      # extents not multiples of 8
    assert sel(capi.gemm_desc(128, 1024, 1024, "fp32")) == capi.ALGO_SIMT_F32       # too small to pay for the passes
    assert sel(capi.gemm_desc(128, 1024, 1024, "fp32", algo=capi.ALGO_F32_SPLIT)) == capi.ALGO_F32_SPLIT
    assert sel(capi.gemm_desc(100, 77, 51, "fp32", algo=capi.ALGO_F32_SPLIT)) == -6
    assert sel(capi.gemm_desc(64, 64, 64, "fp16", algo=capi.ALGO_F32_SPLIT)) == -6
    assert sel(capi.gemm_desc(64, 64, 64, "fp32", algo=6)) == -7
    assert sel(capi.gemm_desc(4096, 4096, 4096, "fp16", trans_b=True)) == capi.ALGO_TCGEN05_PAIR
    assert sel(capi.gemm_desc(4096, 4096, 4096, "fp16")) == capi.ALGO_TCGEN05_PAIR
    # 16 tiles of 256x256: every tile as two K halves on 32 CTA pairs rather than 32 one-CTA tiles
    assert sel(capi.gemm_desc(1024, 1024, 4096, "fp16", trans_b=True)) == capi.ALGO_TCGEN05_PAIR
    assert sel(capi.gemm_desc(1024, 1024, 512, "fp16", trans_b=True)) == capi.ALGO_TCGEN05   # K too short to halve
    assert sel(capi.gemm_desc(2048, 1792, 4096, "fp16", trans_b=True)) == capi.ALGO_TCGEN05  # 56 tiles: one CTA each
    skinny = capi.gemm_desc(16, 28672, 8192, "bf16", trans_b=True)
    assert sel(skinny) == capi.ALGO_SKINNY
    assert lib.frisk_b200_gemm_workspace_bytes(skinny) > 0
    # the CTA-pair kernel may split the K extent of a partial last wave: scratch for its fp32 halves
    assert lib.frisk_b200_gemm_workspace_bytes(capi.gemm_desc(4096, 4096, 4096, "fp16", trans_b=True)) > 0
    assert lib.frisk_b200_gemm_workspace_bytes(capi.gemm_desc(1024, 1024, 4096, "fp16", trans_b=True)) > 0
    assert lib.frisk_b200_gemm_workspace_bytes(capi.gemm_desc(2048, 1792, 4096, "fp16", trans_b=True)) == 0
    assert lib.frisk_b200_gemm_workspace_bytes(capi.gemm_desc(1024, 1024, 1024, "fp32")) == 0
    assert sel(capi.gemm_desc(16, 64, 64, "bf16")) == capi.ALGO_TCGEN05  # weights not K-contiguous
    assert sel(capi.gemm_desc(64, 64, 60, "bf16", trans_b=True)) == -3   # 120-byte pitch
    assert sel(capi.gemm_desc(64, 64, 64, "fp32", "fp16")) == -2
    assert sel(capi.gemm_desc(0, 64, 64, "fp32")) == -1
    assert sel(capi.gemm_desc(64, 64, 64, "fp16", algo=capi.ALGO_SIMT_F32)) == -6
    # the decode kernel streams K through a ring, so no K is too deep for it; M > 16 is
    assert sel(capi.gemm_desc(16, 4096, 131072, "bf16", trans_b=True)) == capi.ALGO_SKINNY
    assert sel(capi.gemm_desc(17, 4096, 8192, "bf16", trans_b=True, algo=capi.ALGO_SKINNY)) == -6


def test_static_scratch_entry_host_side_refusals():
    """frisk_b200_gemm_skinny_static refuses before it touches the device: a problem it has no kernel
    for, one beyond its fixed scratch, and an output that overlaps an input."""
    lib = capi.load()
    call = lambda d, a, b, c: lib.frisk_b200_gemm_skinny_static(0, ctypes.byref(d), a, b, c, None)  # noqa: E731
    assert call(capi.gemm_desc(64, 4096, 8192, "bf16", trans_b=True), 0x1000, 0x2000, 0x3000) == -6
    huge = capi.gemm_desc(16, 200_000_000, 64, "bf16", trans_b=True)   # one ticket per 128 columns: > 8 MiB
    assert lib.frisk_b200_gemm_workspace_bytes(ctypes.byref(huge)) > 8 << 20
    assert call(huge, 0x1000, 0x2000, 0x3000) == -9
    d = capi.gemm_desc(16, 1024, 1024, "bf16", trans_b=True)
    a_bytes, b_bytes = 16 * 1024 * 2, 1024 * 1024 * 2
    base = 0x10000000
    assert call(d, base, base + a_bytes, base + a_bytes - 16) == -4        # C starts inside A
    assert call(d, base, base + a_bytes, base + a_bytes + b_bytes - 2) == -4  # C starts on B's last element
    assert "overlaps" in capi.strerror(-4)


def test_attention_validate():
    lib = capi.load()
    ok = capi.attn_desc(8, 32, 4096, 4096, 128, 128 ** -0.5, True, "bf16")
    assert lib.frisk_b200_attention_validate(ok) == 0
    assert lib.frisk_b200_attention_validate(capi.attn_desc(1, 1, 64, 64, 96, 0.1, False, "bf16")) == -8
    assert lib.frisk_b200_attention_validate(capi.attn_desc(1, 1, 64, 64, 64, 0.1, False, "fp32")) == -6
    assert lib.frisk_b200_attention_validate(capi.attn_desc(1, 1, 128, 64, 64, 0.1, True, "fp16")) == -8
    assert lib.frisk_b200_attention_validate(capi.attn_desc(1, 1, 64, 64, 64, 0.125, False, "fp16", "fp32")) == 0


def test_fused_epilogue_selection_and_workspace():
    """Host-only: when fill / reduce run inside the GEMM epilogue and how much scratch that takes."""
    big = capi.gemm_desc(4096, 4096, 4096, "fp16", "fp16", False, True, clear_accum=True)
    small = capi.gemm_desc(256, 256, 256, "fp16", "fp16", False, True, clear_accum=True)
    f32 = capi.gemm_desc(1024, 1024, 1024, "fp32", "fp32")
    red = capi.gemm_epilogue(reduce="max", reduce_dst=0x1000)
    assert capi.gemm_fused_select(big, red) == 1
    assert capi.gemm_fused_select(small, red) == 0
    assert capi.gemm_fused_select(f32, red) == 0
    acc = capi.gemm_desc(4096, 4096, 4096, "fp16", "fp16", False, True, clear_accum=False)
    assert capi.gemm_fused_select(acc, red) == 0                                        # C is read back
    assert capi.gemm_fused_select(acc, capi.gemm_epilogue(fill=1.0, reduce="add", reduce_dst=0x1000)) == 1
    assert capi.gemm_fused_select(acc, capi.gemm_epilogue(fill=1.0)) == 1
    base = capi.load().frisk_b200_gemm_workspace_bytes(ctypes.byref(big))
    assert capi.gemm_fused_workspace_bytes(big, red) == (base + 255) // 256 * 256 + 16 * 4096 * 4
    assert capi.gemm_fused_workspace_bytes(small, red) == 0
    with pytest.raises(ValueError):
        capi.gemm_epilogue(reduce="mul")                        # the reference's fourth kind has no kernel
    with pytest.raises(ValueError):
        capi.gemm_fused_select(big, capi.gemm_epilogue(reduce="max"))   # no destination
    with pytest.raises(ValueError):
        capi.gemm_fused_select(big, capi.gemm_epilogue(fill=float("nan")))

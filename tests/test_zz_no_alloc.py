"""The allocation-free skinny-GEMM entry point (frisk_b200_gemm_skinny_static).

It exists for callers that cannot allocate device memory at call time (all of HBM already
handed to a serving process's memory manager, or a loop that cannot afford the device-wide
synchronisation of cudaMalloc), so its split-K scratch is a fixed array inside the library.
The test calls it twice in a row through the C ABI, the second time with a different shape
so that stale partial sums of the first call lie where the second keeps its control words,
and requires the same bits as the ordinary entry point.  Collected last on purpose: a run
that stops at the first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest

from frisk_b200 import capi
from oracle import gemm_oracle, inputs
from oracle.numerics import from_storage, rel_frobenius
from tests.util import to_device, to_host

pytestmark = pytest.mark.gpu


def _both(ctx, M, N, K, dtype, seed):
    import torch
    lib = capi.load()
    a, b = inputs.gemm_inputs(M, N, K, dtype, False, True, seed, "act_weight")
    da, db = to_device(a, dtype), to_device(b, dtype)
    c_ref = torch.full((M, N), float("nan"), dtype=da.dtype, device="cuda")
    c_new = torch.full((M, N), float("nan"), dtype=da.dtype, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    desc = capi.gemm_desc(M, N, K, dtype, dtype, False, True, clear_accum=True, algo=capi.ALGO_SKINNY)
    ctx.gemm(desc, da.data_ptr(), db.data_ptr(), c_ref.data_ptr(), stream=stream)
    rc = lib.frisk_b200_gemm_skinny_static(0, ctypes.byref(desc), da.data_ptr(), db.data_ptr(), c_new.data_ptr(),
                                           stream)
    capi.raise_for(rc)
    torch.cuda.synchronize()
    ref, new = to_host(c_ref, dtype), to_host(c_new, dtype)
    assert np.isfinite(from_storage(new, dtype)).all()
    assert np.array_equal(ref, new)
    assert rel_frobenius(from_storage(new, dtype), gemm_oracle.gemm_fp64(a, b, dtype, False, True)) <= 5e-3


def test_static_scratch_entry_matches_ordinary_entry_twice():
    ctx = capi.Context(0)
    try:
        _both(ctx, 16, 1024, 8192, "bf16", 51)   # 8 tiles: every tile's K is shared by many CTAs
        _both(ctx, 13, 28672, 1024, "bf16", 52)  # 224 tiles: more tickets, lying over the first call's partial sums
        _both(ctx, 16, 1024, 8192, "bf16", 51)   # and back
    finally:
        ctx.close()


def test_static_scratch_entry_refuses_oversize_and_bad_layout():
    lib = capi.load()
    big = capi.gemm_desc(16, 200_000_000, 64, "bf16", "bf16", False, True)  # one ticket per 128 columns
    assert lib.frisk_b200_gemm_workspace_bytes(big) > 8 << 20
    assert lib.frisk_b200_gemm_skinny_static(0, ctypes.byref(big), 16, 16, 16, None) == -9
    assert "capacity" in capi.strerror(-9)
    wide = capi.gemm_desc(64, 1024, 1024, "bf16", "bf16", False, True)
    assert lib.frisk_b200_gemm_skinny_static(0, ctypes.byref(wide), 16, 16, 16, None) == -6


def test_static_scratch_entry_refuses_aliased_output_and_keeps_the_current_device():
    import torch
    lib = capi.load()
    M, N, K = 16, 1024, 1024
    x = torch.zeros(M * K + M * N, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
    desc = capi.gemm_desc(M, N, K, "bf16", "bf16", False, True)
    before = torch.cuda.current_device()
    # the output begins inside the activations: refused like the ordinary entry refuses it
    rc = lib.frisk_b200_gemm_skinny_static(0, ctypes.byref(desc), x.data_ptr(), w.data_ptr(), x.data_ptr() + 64, None)
    assert rc == -4
    rc = lib.frisk_b200_gemm_skinny_static(0, ctypes.byref(desc), x.data_ptr(), w.data_ptr(),
                                           x.data_ptr() + M * K * 2, torch.cuda.current_stream().cuda_stream)
    capi.raise_for(rc)
    torch.cuda.synchronize()
    assert torch.cuda.current_device() == before

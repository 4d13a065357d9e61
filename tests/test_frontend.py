"""The re-hosted builder surface: the flows of the reference's test/python/bind_test.py,
helper_test.py and legacy_normalization_test.py:82-88, minus what needs frisk-opt."""
import os

import pytest

import frisk_b200 as F


def build_bind_test_module(clear_accum=False, with_side_ops=True, dtype_name="f16", shape=(4096, 4096)):
    context = F.context()
    F.frisk.load_dialects(context)
    builder = F.builder(context)
    module = builder.create_module()
    module.context = context
    dtype = {"f16": builder.get_f16_ty, "bf16": builder.get_bf16_ty, "f32": builder.get_f32_ty}[dtype_name]()
    mem_type = builder.get_memref_ty(dtype, list(shape), F.AffineMap(), F.MemorySpace.GLOBAL)
    mem2_type = builder.get_memref_ty(dtype, [shape[0]], F.AffineMap(), F.MemorySpace.GLOBAL)
    kernel_type = builder.get_kernel_ty([mem_type, mem_type, mem_type, mem2_type])
    kernel = builder.create_kernel_op(module, "test_gemm", kernel_type)
    module.push_back(kernel)
    entry1 = kernel.add_entry_block()
    builder.set_insertion_point_to_start(entry1)
    parallel = builder.create_parallel_op([8, 8], 128)
    entry2 = parallel.add_entry_block()
    builder.set_insertion_point_to_start(entry2)
    args = [entry1.get_argument(i) for i in range(4)]
    builder.create_alloc_buffer_op([128, 32], "fp16", F.MemorySpace.SHARED, 1024)
    builder.create_alloc_buffer_op([32, 128], "fp16", F.MemorySpace.SHARED, 1024)
    builder.create_alloc_buffer_op([128, 128], "fp16", F.MemorySpace.LOCAL)

    def for_body(b, iv):
        if with_side_ops:
            builder.create_fill_op(args[0], 0.0, "fp16")
            builder.create_reduce_op(args[0], args[3], "max", 1, True)
            builder.create_copy_op(args[0], args[1], [iv, iv], [iv, iv])

        def block_body(b, ivs):
            assert len(ivs) == 2
            b.create_gemm_op(args[0], args[1], args[2], False, False, clear_accum)
        builder.create_block_op([128, 128], block_body)
    builder.create_for_op(0, 128, 1, for_body)
    return module


def test_bind_test_flow_prints_the_ops():
    text = str(build_bind_test_module())
    assert "frisk.kernel @test_gemm(memref<4096x4096xf16, 1>" in text
    assert "frisk.parallel (%arg4, %arg5) = (8, 8), threads = 128 {" in text
    assert "frisk.alloc_buffer {alignment = 1024 : i64} -> memref<128x32xf16, 3>" in text
    assert "-> memref<128x128xf16>" in text  # LOCAL = space 0 is elided
    assert "frisk.for %arg6 = 0 to 128 {" in text
    assert "frisk.block (%arg7, %arg8) to (128, 128) {" in text
    assert ("frisk.gemm(%arg0, %arg1, %arg2) {K = 4096 : i64, M = 4096 : i64, N = 4096 : i64, "
            "clear_accum = false, policy = #frisk<gemm_warp_policy Square>, transA = false, transB = false}") in text
    assert 'frisk.reduce %arg0, %arg3 {clear = true, dim = 1 : i64, kind = "max"}' in text
    assert "frisk.copy %arg0[%arg6, %arg6], %arg1[%arg6, %arg6]" in text


def test_helper_demo_flow():
    helper = F.create_session()
    f16 = helper.builder.get_f16_ty()
    a_ty = helper.memref_type((128, 64), f16, space=F.MemorySpace.SHARED)
    b_ty = helper.memref_type((64, 128), f16, space=F.MemorySpace.SHARED)
    c_ty = helper.memref_type((128, 128), f16, space=F.MemorySpace.LOCAL)
    kernel, entry = helper.new_kernel("helper_demo", [a_ty, b_ty, c_ty])
    args = [entry.get_argument(i) for i in range(3)]
    gemm = helper.create_gemm(args[0], args[1], args[2])
    assert gemm.get_matrix_A() is args[0] and gemm.get_matrix_C() is args[2]
    scratch = helper.alloc_buffer((32, 32), "fp16", space=F.MemorySpace.SHARED, alignment=64)
    assert "memref" in str(scratch.get_type())
    assert kernel.verify()
    assert helper.module.verify()
    assert helper.module.context is helper.context


def test_builder_rejects_effective_shape_mismatch():
    session = F.create_session()
    _, entry = session.new_kernel("bad", [session.memref_type([64, 16]), session.memref_type([8, 64]),
                                          session.memref_type([64, 64], "fp32")])
    with pytest.raises(ValueError, match="legacy-gemm-shape"):
        session.create_gemm(*(entry.get_argument(i) for i in range(3)))


def test_builder_type_contract():
    session = F.create_session()
    _, e = session.new_kernel("t", [session.memref_type([64, 16], "fp16"), session.memref_type([16, 64], "bf16"),
                                    session.memref_type([64, 64], "fp32"), session.memref_type([16, 64], "fp16"),
                                    session.memref_type([64, 64], "bf16")])
    with pytest.raises(ValueError, match="legacy-gemm-type: A and B must have the same element type"):
        session.create_gemm(e.get_argument(0), e.get_argument(1), e.get_argument(2))
    with pytest.raises(ValueError, match="legacy-gemm-type: C must match"):
        session.create_gemm(e.get_argument(0), e.get_argument(3), e.get_argument(4))
    # f16 x f16 -> f32 and f16 x f16 -> f16 are both in the contract
    session.create_gemm(e.get_argument(0), e.get_argument(3), e.get_argument(2))


def test_all_transposes_derive_mnk():
    for ta in (False, True):
        for tb in (False, True):
            s = F.create_session()
            a = [16, 64] if ta else [64, 16]
            b = [32, 16] if tb else [16, 32]
            _, e = s.new_kernel("g", [s.memref_type(a), s.memref_type(b), s.memref_type([64, 32], "fp32")])
            op = s.create_gemm(e.get_argument(0), e.get_argument(1), e.get_argument(2), trans_a=ta, trans_b=tb,
                               clear_accum=True, legacy_semantics="tensor_v1")
            assert (op.attrs["M"], op.attrs["N"], op.attrs["K"]) == (64, 32, 16)
            assert 'frisk.legacy_semantics = "tensor_v1"' in str(s.module)


def test_api_quirks():
    s = F.create_session()
    kernel, entry = s.new_kernel("k", [s.memref_type([8, 8])])
    # create_parallel_op must be the first thing built in the kernel body
    s.builder.create_alloc_buffer_op([8, 8], "fp16")
    with pytest.raises(ValueError, match="invalid parallel create"):
        s.builder.create_parallel_op([1], 128)
    # create_kernel_op returns the existing op for a known symbol
    again = s.builder.create_kernel_op(s.module, "k", s.builder.get_kernel_ty([]))
    assert again is kernel
    with pytest.raises(ValueError, match="invalid float type"):
        s.builder.create_alloc_buffer_op([8], "bf16")  # the string set has no bf16 in the reference either
    with pytest.raises(ValueError, match="alignment must be non-negative"):
        s.builder.create_alloc_buffer_op([8], "fp16", F.MemorySpace.SHARED, -1)
    with pytest.raises(IndexError):
        entry.get_argument(5)
    # thread-count whitelist and power-of-two alignment are verifier errors
    s2 = F.create_session()
    k2, e2 = s2.new_kernel("p", [])
    par = s2.builder.create_parallel_op([2], 96)
    par.add_entry_block()
    assert not k2.verify()
    s3 = F.create_session()
    k3, _ = s3.new_kernel("q", [])
    s3.builder.create_alloc_buffer_op([8], "fp16", F.MemorySpace.SHARED, 24)
    assert not k3.verify()


def test_gemm_plan_from_bind_test_nest():
    # an idempotent gemm (clear_accum) inside parallel/for/block resolves to one GEMM
    mod = build_bind_test_module(clear_accum=True, with_side_ops=False)
    desc, idx = F.gemm_plan(mod)
    assert (desc.M, desc.N, desc.K) == (4096, 4096, 4096)
    assert (desc.trans_a, desc.trans_b, desc.clear_accum) == (0, 0, 1)
    assert idx == (0, 1, 2)
    assert desc.dtype_ab == F.capi.F16 and desc.dtype_c == F.capi.F16
    # accumulate inside a 128-trip loop is not one GEMM; side-effecting neighbours are refused
    with pytest.raises(ValueError, match="multi-trip"):
        F.gemm_plan(build_bind_test_module(clear_accum=False, with_side_ops=False))
    with pytest.raises(ValueError, match="unsupported op frisk.fill"):
        F.gemm_plan(build_bind_test_module(clear_accum=True, with_side_ops=True))


def test_execute_refuses_cpu_tensors():
    import torch
    mod = build_bind_test_module(clear_accum=True, with_side_ops=False, shape=(128, 128))
    t = torch.zeros(128, 128, dtype=torch.float16)
    v = torch.zeros(128, dtype=torch.float16)
    with pytest.raises(ValueError, match="no CPU path"):
        F.execute(mod, t, t, t.clone(), v)


def build_fused_module(fill=None, reduce=None, clear=True, clear_accum=False, shape=(512, 384, 256), trips=1,
                       r_shape=None, r_type=None, dim=1):
    """kernel(A[M,K], B[N,K], C[M,N], r[M]): parallel { for { [fill C] gemm(A, B^T, C) [reduce C -> r] } }"""
    m, n, k = shape
    context = F.context()
    F.frisk.load_dialects(context)
    builder = F.builder(context)
    module = builder.create_module()
    module.context = context
    f16 = builder.get_f16_ty()
    types = [builder.get_memref_ty(f16, s, F.AffineMap(), F.MemorySpace.GLOBAL) for s in ([m, k], [n, k], [m, n])]
    r_elem = f16 if r_type is None else getattr(builder, f"get_{r_type}_ty")()
    types.append(builder.get_memref_ty(r_elem, [m] if r_shape is None else list(r_shape), F.AffineMap(),
                                       F.MemorySpace.GLOBAL))
    kernel = builder.create_kernel_op(module, "fused", builder.get_kernel_ty(types))
    module.push_back(kernel)
    entry = kernel.add_entry_block()
    builder.set_insertion_point_to_start(entry)
    par = builder.create_parallel_op([4, 4], 128)
    builder.set_insertion_point_to_start(par.add_entry_block())
    a, b, c, r = (entry.get_argument(i) for i in range(4))

    def body(bld, iv):
        if fill is not None:
            builder.create_fill_op(c, fill, "fp16")
        builder.create_gemm_op(a, b, c, False, True, clear_accum)
        if reduce is not None:
            builder.create_reduce_op(c, r, reduce, dim, clear)
    builder.create_for_op(0, trips, 1, body)
    return module


@pytest.mark.parametrize("kwargs,message", [
    (dict(r_shape=[8]), r"non-reduced dimension mismatch: source\[0\] = 512 vs destination\[0\] = 8"),
    (dict(r_type="f32"), "source and destination must have the same element type"),
    (dict(r_shape=[512, 1]), "destination rank must be one less than source rank. Got: 2 vs 2"),
    (dict(dim=2), "dimension 2 is out of range for source of rank 2"),
    (dict(dim=-1), "dimension -1 is out of range for source of rank 2"),
    (dict(reduce="xor"), "unsupported reduce kind: xor. Supported: add, mul, min, max"),
])
def test_reduce_verifier_rejects_what_the_reference_rejects(kwargs, message):
    """ReduceOp::verify (lib/Dialect/Frisk/IR/FriskOps.cpp:728-762): a destination whose rank, kept
    extents or element type disagree with the source never reaches a kernel."""
    kw = dict(reduce="max", clear_accum=True)
    kw.update(kwargs)
    mod = build_fused_module(**kw)
    assert not mod.verify()
    with pytest.raises(ValueError, match=message):
        F.ir._verify(mod)
    with pytest.raises(ValueError, match="does not verify"):
        F.fused_plan(mod)


def test_reduce_verifier_accepts_the_reduction_along_dim_0():
    # dim 0 of an M x N source keeps N: verifies, but has no kernel here
    mod = build_fused_module(reduce="max", clear_accum=True, dim=0, shape=(384, 384, 256))
    assert mod.verify()
    with pytest.raises(ValueError, match="unsupported op frisk.reduce"):
        F.fused_plan(mod)


def test_fused_plan_folds_fill_and_reduce_into_the_gemm():
    desc, idx, epi = F.fused_plan(build_fused_module(fill=0.5, reduce="max", clear=False))
    assert (desc.M, desc.N, desc.K, desc.trans_b, desc.clear_accum) == (512, 384, 256, 1, 0) and idx == (0, 1, 2)
    assert epi == {"fill": 0.5, "reduce": "max", "reduce_arg": 3, "reduce_clear": False}
    _, _, epi = F.fused_plan(build_fused_module(reduce="add", clear_accum=True))
    assert epi == {"fill": None, "reduce": "add", "reduce_arg": 3, "reduce_clear": True}
    assert F.fused_plan(build_fused_module(clear_accum=True))[2] is None
    with pytest.raises(ValueError, match="use fused_plan"):
        F.gemm_plan(build_fused_module(fill=1.0))
    with pytest.raises(ValueError, match="no kernel for reduce kind mul"):
        F.fused_plan(build_fused_module(reduce="mul", clear_accum=True))
    with pytest.raises(ValueError, match="multi-trip"):
        F.fused_plan(build_fused_module(fill=1.0, trips=3))
    # a fill or reduce that does not touch the gemm's C stays unsupported (the bind_test neighbours)
    with pytest.raises(ValueError, match="unsupported op frisk.fill"):
        F.fused_plan(build_bind_test_module(clear_accum=True, with_side_ops=True))


def _reference_dir():
    """FRISK_REFERENCE_DIR, else a checkout named `reference` beside this repository."""
    env = os.environ.get("FRISK_REFERENCE_DIR")
    if env:
        return env
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.path.join(os.path.dirname(repo), "reference")


REFERENCE_TESTS = os.path.join(_reference_dir(), "test", "python")


@pytest.mark.parametrize("script", ["bind_test.py", "helper_test.py", "map_expr_test.py", "test.py"])
def test_reference_builder_scripts_run_verbatim(script, capsys):
    """The reference's own builder scripts (`import frisk as F`), unmodified, against this
    package under the name `frisk`.  Skipped where the reference checkout is not present."""
    import runpy
    import sys
    path = os.path.join(REFERENCE_TESTS, script)
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    saved = sys.modules.get("frisk")
    sys.modules["frisk"] = F
    try:
        runpy.run_path(path, run_name="__main__")
    finally:
        if saved is None:
            sys.modules.pop("frisk", None)
        else:
            sys.modules["frisk"] = saved
    out = capsys.readouterr().out
    if script == "bind_test.py":
        assert "frisk.gemm" in out and "frisk.reduce" in out and "frisk.fill" in out
    if script == "map_expr_test.py":
        assert out.splitlines()[0] == "d0 * 5 + s0" and "(d0)[s0] -> ((d0 * 5 + s0) * 2)" in out


def test_affine_expressions_simplify_and_print_like_the_reference_binding():
    """ffi/ir.cpp:640-875 binds MLIR's AffineExpr / AffineMap; these are the documented construction-time
    simplifications and printer forms of those classes."""
    b = F.builder(F.context())
    d0, d1, s0 = b.get_affine_dim_expr(0), b.get_affine_dim_expr(1), b.get_affine_symbol_expr(0)
    c = b.get_affine_constant_expr
    assert str(d0 * c(5) + s0 + c(0)) == "d0 * 5 + s0"
    assert str(3 + d0 + 4) == "d0 + 7" and str((d0 * 2) * 3) == "d0 * 6"
    assert str(d0 - d1) == "d0 - d1" and str(d0 * 2 - s0 * 3) == "d0 * 2 - s0 * 3" and str(d0 - 3) == "d0 - 3"
    assert str((d0 + 1) * 2) == "(d0 + 1) * 2" and str(-(d0 + 1)) == "-(d0 + 1)"
    assert str((d0 + d1).floor_div(4)) == "(d0 + d1) floordiv 4" and (d0 * 8) % 4 == 0
    assert str((d0 * 8).floor_div(4)) == "d0 * 2" and str(d0.ceil_div(1)) == "d0"
    assert str(s0 * d0) == "d0 * s0" and str(d0 + d0) == "d0 * 2" and (d0 - d0) == 0
    assert c(7).floor_div(2) == 3 and c(-7).floor_div(2) == -4 and c(7).ceil_div(2) == 4 and c(-7) % 4 == 1
    with pytest.raises(ValueError):
        d0 * d1
    e = d0 * 5 + s0
    assert e.get_kind() == F.AffineExprKind.Add and str(e.get_kind()) == "AffineExprKind.Add"
    assert str(e.as_binary().get_lhs()) == "d0 * 5" and e.as_dim() is None and d1.as_dim().get_position() == 1
    assert e.is_pure_affine() and not e.is_symbolic_or_constant() and e.is_function_of_dim(0) and not e.is_function_of_dim(1)
    assert str(e.replace_dims_and_symbols([d1 + 1], [c(2)])) == "(d1 + 1) * 5 + 2"  # no flattening on construction
    m = F.AffineMap.get(2, 1, [d0 + s0, d1], None)
    assert str(m) == "(d0, d1)[s0] -> (d0 + s0, d1)" and m.get_num_inputs() == 3 and not m.is_identity()
    assert F.AffineMap.get_multi_dim_identity_map(2, None).is_identity()
    assert str(F.AffineMap.get_permutation_map([1, 0], None)) == "(d0, d1) -> (d1, d0)"
    assert F.AffineMap.get_permutation_map([1, 0], None).is_permutation()
    assert not F.AffineMap() and str(F.AffineMap()) == "<<NULL AFFINE MAP>>" and F.AffineMap.get(None).is_empty()
    assert F.AffineMap.get_constant_map(5, None).get_single_constant_result() == 5


# ------------------------------------------------------------------ the attention graph over frisk.mma
def build_attention_module(n_q=64, n_kv=64, d=64, dtype="f16", scale=0x3E000000, out="f32"):
    context = F.context()
    F.frisk.load_dialects(context)
    builder = F.builder(context)
    module = builder.create_module()
    module.context = context
    el = {"f16": builder.get_f16_ty, "bf16": builder.get_bf16_ty, "f32": builder.get_f32_ty}
    kernel = F.build_attention_kernel(builder, module, "attention_q64_full_kv", n_q, n_kv, d, el[dtype](), scale, el[out]())
    return module, kernel


def test_attention_graph_prints_the_reference_assembly():
    """The op lines of test/Transforms/attention-layout-tile-d64.mlir:44-61 in the ops' declared assembly formats
    (include/Dialect/Frisk/IR/FriskLayoutOps.td: reduce_tensor :29, mma :47, layout_view :73, tile_store :97)."""
    module, kernel = build_attention_module()
    assert module.verify()
    text = str(module)
    for line in (
        "frisk.kernel @attention_q64_full_kv(memref<64x64xf16, 1>, memref<64x64xf16, 1>, memref<64x64xf16, 1>, memref<64x64xf32, 1>) {",
        "= memref.alloc() {alignment = 1024 : i64} : memref<64x64xf16, 3>",
        "frisk.parallel (%arg4) = (1), threads = 128 {",
        "= frisk.layout_view %arg0 : memref<64x64xf16, 1> -> memref<64x64xf16, 1>",
        "= arith.constant dense<0.0> : tensor<64x64xf32>",
        "{k = 64 : i64, m = 64 : i64, n = 64 : i64, trans_b = true} : memref<64x64xf16, 3>, memref<64x64xf16, 3>, tensor<64x64xf32> -> tensor<64x64xf32>",
        "= arith.constant dense<0x3E000000> : tensor<64x64xf32>",
        '{dim = 1 : i64, kind = "max"} : tensor<64x64xf32> -> tensor<64xf32>',
        "outs(%14 : tensor<64x64xf32>) dimensions = [1]",
        '{dim = 1 : i64, kind = "sum"} : tensor<64x64xf32> -> tensor<64xf32>',
        "= arith.truncf %21 : tensor<64x64xf32> to tensor<64x64xf16>",
        "{k = 64 : i64, m = 64 : i64, n = 64 : i64} : tensor<64x64xf16>, memref<64x64xf16, 3>, tensor<64x64xf32> -> tensor<64x64xf32>",
        "frisk.tile_store %24, %25 : tensor<64x64xf32>, memref<64x64xf32, 1>",
    ):
        assert line in text, line


def test_attention_plan_resolves_the_graph():
    _, kernel = build_attention_module()
    spec, idx = F.attention_plan(kernel)
    assert spec == dict(S_q=64, S_kv=64, D=64, scale=0.125, dtype_in="fp16", dtype_out="fp32") and idx == (0, 1, 2, 3)
    _, kernel = build_attention_module(128, 512, 128, "bf16", 128 ** -0.5, "bf16")
    spec, _ = F.attention_plan(kernel)
    assert (spec["S_q"], spec["S_kv"], spec["D"], spec["dtype_in"], spec["dtype_out"]) == (128, 512, 128, "bf16", "bf16")
    assert abs(spec["scale"] - 128 ** -0.5) < 1e-7
    with pytest.raises(ValueError, match="head dimension"):
        F.attention_plan(build_attention_module(64, 64, 32)[1])
    import torch
    t = torch.zeros(64, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="no CPU path"):
        F.execute(build_attention_module()[0], t, t, t, torch.zeros(64, 64))


def test_tensor_op_verifiers_reject_what_the_reference_rejects():
    """MmaOp::verify, ReduceTensorOp::verify, TileStoreOp::verify (lib/Dialect/Frisk/IR/FriskLayoutOps.cpp:33-66,78-119,229-245)."""
    b = F.builder(F.context())
    ab = F.AttentionBuilder(b)
    f16, f32 = b.get_f16_ty(), b.get_f32_ty()
    shared = lambda shape, el=f16: ab.memref_alloc(el, shape).results[0]  # noqa: E731
    zero = lambda shape, el=f32: ab.constant(ab.tensor_ty(el, shape), 0.0).results[0]  # noqa: E731
    with pytest.raises(ValueError, match="mma-shape: matrix extents disagree with m/n/k and transpose"):
        ab.mma(shared([64, 64]), shared([32, 64]), zero([64, 64]))          # B is [k, n]: k = 32 != 64
    with pytest.raises(ValueError, match="mma-shape: incompatible input/accumulator element types"):
        ab.mma(shared([64, 64], f32), shared([64, 64], f32), zero([64, 64], f16))
    with pytest.raises(ValueError, match="mma-shape: incompatible input/accumulator element types"):
        ab.mma(shared([64, 64]), shared([64, 64], b.get_bf16_ty()), zero([64, 64]))
    with pytest.raises(ValueError, match="mma-shape: requires positive static rank-2 floating matrices"):
        ab.mma(shared([64, 64, 2]), shared([64, 64]), zero([64, 64]))
    ok = ab.mma(shared([64, 16]), shared([64, 16]), zero([64, 64]), trans_b=True)
    assert (ok.attrs["m"], ok.attrs["n"], ok.attrs["k"]) == (64, 64, 16)
    with pytest.raises(ValueError, match="reduce-shape: kind must be sum/max/min"):
        ab.reduce_tensor(zero([64, 64]), "add", 1)
    with pytest.raises(ValueError, match="reduce-shape: rank >= 2 and valid axis required"):
        ab.reduce_tensor(zero([64, 64]), "max", 2)
    with pytest.raises(ValueError, match="reduce-shape: requires static positive power-of-two extents"):
        ab.reduce_tensor(zero([64, 96]), "max", 1)
    with pytest.raises(ValueError, match="identical static shape and element type"):
        ab.tile_store(zero([64, 64]), shared([64, 64]))                    # f32 tensor into an f16 memref

"""The tensor-level ops of the attention graph, re-hosted without MLIR.

The reference states its attention kernels as MLIR text over ``frisk.mma``,
``frisk.reduce_tensor``, ``frisk.layout_view``, ``frisk.tile_load`` / ``frisk.tile_store``
(``include/Dialect/Frisk/IR/FriskLayoutOps.td:14-112``) and a handful of upstream ops
(``arith.constant / mulf / subf / divf / truncf``, ``math.exp``, ``tensor.empty``,
``linalg.broadcast``, ``memref.alloc``): ``test/Transforms/attention-layout-tile-d64.mlir:23-63``.
Its pybind surface has no builders for them (``ffi/ir.cpp`` stops at the memref ops), so the
``AttentionBuilder`` helpers below are an EXTENSION of the kept API: they build the same ops
with the verifiers of ``lib/Dialect/Frisk/IR/FriskLayoutOps.cpp:33-66,78-119,221-245`` and
print them in the ops' declared assembly formats.  ``attention_plan`` recognises the graph
(scores = Q.K^T, scale, row max, exp, row sum, divide, round to 16 bits, P.V, store) and
resolves it to the descriptor ``frisk_b200_attention_fwd`` takes; the division by the
COMPLETE row sum before the rounding is the library's ``normalize_p = 1`` mode.
"""
import struct

from . import ir
from .ir import MemorySpace, OpState, type as ir_type


def _is_pow2(n):
    return n > 0 and n & (n - 1) == 0


def _float_bits(ty):
    return {"f16": 16, "bf16": 16, "f32": 32, "f64": 64}.get(getattr(ty, "name", ""), 0)


def _shaped(ty):
    return ty.kind in ("memref", "tensor")


class MmaOp(OpState):
    """``frisk.mma``: result = init + op(A).op(B); A a tensor or memref, B a memref, accumulator at
    least as wide as the inputs (FriskLayoutOps.td:32-48)."""
    op_name = "frisk.mma"

    def verify_op(self):  # FriskLayoutOps.cpp:78-119
        a = self.attrs
        if a["m"] <= 0 or a["n"] <= 0 or a["k"] <= 0:
            raise ValueError("mma-shape: m/n/k must be positive signless i64")
        ta, tb, ti = (v.type for v in self.operands)
        tr = self.results[0].type
        for t in (ta, tb, ti, tr):
            if not _shaped(t) or len(t.shape) != 2 or any(e <= 0 for e in t.shape) or t.element.kind != "float":
                raise ValueError("mma-shape: requires positive static rank-2 floating matrices")
        if ta.element != tb.element or ti.element != tr.element or _float_bits(ti.element) < _float_bits(ta.element):
            raise ValueError("mma-shape: incompatible input/accumulator element types")
        ok = (ta.shape[1 if a["trans_a"] else 0] == a["m"] and ta.shape[0 if a["trans_a"] else 1] == a["k"] and
              tb.shape[1 if a["trans_b"] else 0] == a["k"] and tb.shape[0 if a["trans_b"] else 1] == a["n"] and
              list(ti.shape) == [a["m"], a["n"]] and list(tr.shape) == list(ti.shape))
        if not ok:
            raise ValueError("mma-shape: matrix extents disagree with m/n/k and transpose")

    def print_assembly(self, name):
        a, b, c = self.operands
        attrs = {k: v for k, v in self.attrs.items() if not (k in ("trans_a", "trans_b") and v is False)
                 and not (k == "policy" and v == ir.GemmWarpPolicy.Square)}
        return (f"{name(self.results[0])} = frisk.mma {name(a)}, {name(b)}, {name(c)}" + ir._attr_dict(attrs) +
                f" : {a.type}, {b.type}, {c.type} -> {self.results[0].type}")


class ReduceTensorOp(OpState):
    """``frisk.reduce_tensor``: one axis reduced with sum/max/min in the input type (FriskLayoutOps.td:14-30)."""
    op_name = "frisk.reduce_tensor"

    def verify_op(self):  # FriskLayoutOps.cpp:33-66
        src, dst = self.operands[0].type, self.results[0].type
        kind, dim = self.attrs["kind"], self.attrs["dim"]
        if kind not in ("sum", "max", "min"):
            raise ValueError("reduce-shape: kind must be sum/max/min")
        if len(src.shape) < 2 or len(dst.shape) != len(src.shape) - 1 or dim < 0 or dim >= len(src.shape):
            raise ValueError("reduce-shape: rank >= 2 and valid axis required")
        if getattr(src.element, "name", "") not in ("f16", "bf16", "f32") or src.element != dst.element:
            raise ValueError("reduce-shape: requires matching f16/bf16/f32 element types")
        for t in (src, dst):
            if any(not _is_pow2(e) for e in t.shape):
                raise ValueError("reduce-shape: requires static positive power-of-two extents")
        if list(dst.shape) != [e for i, e in enumerate(src.shape) if i != dim]:
            raise ValueError("reduce-shape: result must delete the reduction axis")

    def print_assembly(self, name):
        s = self.operands[0]
        return (f"{name(self.results[0])} = frisk.reduce_tensor {name(s)}" + ir._attr_dict(self.attrs) +
                f" : {s.type} -> {self.results[0].type}")


class LayoutViewOp(OpState):
    """``frisk.layout_view``: a fully aliasing view of a memref (FriskLayoutOps.td:50-74)."""
    op_name = "frisk.layout_view"

    def verify_op(self):
        s, r = self.operands[0].type, self.results[0].type
        if s.kind != "memref" or r.kind != "memref" or list(s.shape) != list(r.shape) or s.element != r.element:
            raise ValueError("layout_view requires a memref result of the source's shape and element type")

    def print_assembly(self, name):
        s = self.operands[0]
        return f"{name(self.results[0])} = frisk.layout_view {name(s)} : {s.type} -> {self.results[0].type}"


def _whole_tile(memref, tensor, message):  # FriskLayoutOps.cpp:157-177
    if list(memref.shape) != list(tensor.shape) or memref.element != tensor.element:
        raise ValueError(message)


class TileLoadOp(OpState):
    op_name = "frisk.tile_load"

    def verify_op(self):  # FriskLayoutOps.cpp:221-227
        _whole_tile(self.operands[0].type, self.results[0].type,
                    "source memref and result tensor must have identical static shape and element type")

    def print_assembly(self, name):
        s = self.operands[0]
        return f"{name(self.results[0])} = frisk.tile_load {name(s)} : {s.type} -> {self.results[0].type}"


class TileStoreOp(OpState):
    op_name = "frisk.tile_store"

    def verify_op(self):  # FriskLayoutOps.cpp:229-245
        _whole_tile(self.operands[1].type, self.operands[0].type,
                    "value tensor and target memref must have identical static shape and element type")

    def print_assembly(self, name):
        v, t = self.operands
        return f"frisk.tile_store {name(v)}, {name(t)} : {v.type}, {t.type}"


class UpstreamOp(OpState):
    """An op of an upstream dialect the attention graph uses (arith / math / tensor / linalg / memref):
    carried structurally, printed in MLIR's custom form for that op."""

    def __init__(self, name, operands=(), result_types=(), attrs=None):
        super().__init__(operands, result_types, attrs)
        self.op_name = name

    def verify_op(self):
        n = self.op_name
        if n in ("arith.mulf", "arith.subf", "arith.divf"):
            a, b = (v.type for v in self.operands)
            if a != b or a != self.results[0].type:
                raise ValueError(f"'{n}' op requires the same type for all operands and results")
        elif n == "arith.truncf":
            s, r = self.operands[0].type, self.results[0].type
            if list(s.shape) != list(r.shape) or _float_bits(r.element) >= _float_bits(s.element):
                raise ValueError("'arith.truncf' op result type must be narrower than the operand type")
        elif n == "linalg.broadcast":
            s, init = (v.type for v in self.operands)
            dims = self.attrs["dimensions"]
            kept = [e for i, e in enumerate(init.shape) if i not in dims]
            if list(s.shape) != kept or s.element != init.element:
                raise ValueError("'linalg.broadcast' op input shape must match the init shape without the added dimensions")

    def print_assembly(self, name):
        n, res = self.op_name, self.results
        if n == "arith.constant":
            return f"{name(res[0])} = arith.constant dense<{self.attrs['text']}> : {res[0].type}"
        if n == "tensor.empty":
            return f"{name(res[0])} = tensor.empty() : {res[0].type}"
        if n == "memref.alloc":
            return f"{name(res[0])} = memref.alloc()" + ir._attr_dict(self.attrs) + f" : {res[0].type}"
        if n == "linalg.broadcast":
            s, init = self.operands
            dims = ", ".join(str(d) for d in self.attrs["dimensions"])
            return (f"{name(res[0])} = linalg.broadcast ins({name(s)} : {s.type}) outs({name(init)} : {init.type}) "
                    f"dimensions = [{dims}]")
        if n == "arith.truncf":
            s = self.operands[0]
            return f"{name(res[0])} = arith.truncf {name(s)} : {s.type} to {res[0].type}"
        ops = ", ".join(name(v) for v in self.operands)
        return f"{name(res[0])} = {n} {ops} : {res[0].type}"


def splat_bits(value_or_bits):
    """(text, python float) of a dense splat: a float, or the 32-bit pattern MLIR prints as hex
    (``dense<0x3E000000>`` is 0.125 in attention-layout-tile-d64.mlir:45)."""
    if isinstance(value_or_bits, int):
        return f"0x{value_or_bits:08X}", struct.unpack("<f", struct.pack("<I", value_or_bits))[0]
    v = float(value_or_bits)
    return ("0.0" if v == 0.0 else repr(v)), v


class AttentionBuilder:
    """Builders for the ops above on top of ``ir.builder`` (an extension: see the module docstring)."""

    def __init__(self, builder):
        self.b = builder

    def tensor_ty(self, element, shape):
        return self.b.get_ranked_tensor_ty(element, [int(d) for d in shape])

    def memref_alloc(self, element, shape, space=MemorySpace.SHARED, alignment=0):
        ty = ir_type("memref", shape=[int(d) for d in shape], element=element, map=None, space=MemorySpace(space))
        attrs = {"alignment": int(alignment)} if alignment else {}
        return self.b._insert(UpstreamOp("memref.alloc", (), [ty], attrs))

    def layout_view(self, source):
        return self.b._insert(LayoutViewOp(operands=[source], result_types=[source.type]))

    def constant(self, tensor_type, value_or_bits):
        text, v = splat_bits(value_or_bits)
        return self.b._insert(UpstreamOp("arith.constant", (), [tensor_type], {"text": text, "_value": v}))

    def empty(self, tensor_type):
        return self.b._insert(UpstreamOp("tensor.empty", (), [tensor_type]))

    def mma(self, a, b, init, trans_a=False, trans_b=False):
        ta, tb = a.type, b.type
        m, k = (ta.shape[1], ta.shape[0]) if trans_a else (ta.shape[0], ta.shape[1])
        n = tb.shape[0] if trans_b else tb.shape[1]
        op = MmaOp(operands=[a, b, init], result_types=[self.tensor_ty(init.type.element, [m, n])],
                   attrs={"m": int(m), "n": int(n), "k": int(k), "trans_a": bool(trans_a), "trans_b": bool(trans_b),
                          "policy": ir.GemmWarpPolicy.Square})
        op.verify_op()
        return self.b._insert(op)

    def reduce_tensor(self, source, kind, dim):
        shape = [e for i, e in enumerate(source.type.shape) if i != dim]
        op = ReduceTensorOp(operands=[source], result_types=[self.tensor_ty(source.type.element, shape)],
                            attrs={"kind": str(kind), "dim": int(dim)})
        op.verify_op()
        return self.b._insert(op)

    def broadcast(self, source, init, dimensions):
        return self.b._insert(UpstreamOp("linalg.broadcast", [source, init], [init.type],
                                         {"dimensions": [int(d) for d in dimensions]}))

    def binary(self, name, lhs, rhs):
        return self.b._insert(UpstreamOp(name, [lhs, rhs], [lhs.type]))

    def exp(self, source):
        return self.b._insert(UpstreamOp("math.exp", [source], [source.type]))

    def truncf(self, source, element):
        return self.b._insert(UpstreamOp("arith.truncf", [source], [self.tensor_ty(element, source.type.shape)]))

    def tile_load(self, source):
        op = TileLoadOp(operands=[source], result_types=[self.tensor_ty(source.type.element, source.type.shape)])
        return self.b._insert(op)

    def tile_store(self, value, target):
        op = TileStoreOp(operands=[value, target])
        op.verify_op()
        return self.b._insert(op)


def build_attention_kernel(builder, module, name, n_q, n_kv, d, element, scale_bits_or_value, out_element=None,
                           threads=128):
    """The graph of test/Transforms/attention-layout-tile-d64.mlir:23-63 for a [n_q, d] query tile over n_kv keys:
    kernel(q, k, v, o) { shared copies; S = mma(q, k^T); S *= scale; P = softmax rows; o = mma(trunc(P), v) }."""
    ab = AttentionBuilder(builder)
    out_element = out_element or builder.get_f32_ty()
    f32 = builder.get_f32_ty()
    g = MemorySpace.GLOBAL
    types = [builder.get_memref_ty(element, [n_q, d], ir.AffineMap(), g), builder.get_memref_ty(element, [n_kv, d], ir.AffineMap(), g),
             builder.get_memref_ty(element, [n_kv, d], ir.AffineMap(), g), builder.get_memref_ty(out_element, [n_q, d], ir.AffineMap(), g)]
    kernel = builder.create_kernel_op(module, name, builder.get_kernel_ty(types))
    module.push_back(kernel)
    entry = kernel.add_entry_block()
    builder.set_insertion_point_to_start(entry)
    q, k, v, o = (entry.get_argument(i) for i in range(4))
    # (create_parallel_op insists on being the first op built in the kernel body, ffi/ir.cpp:363-370; the
    # staging buffers are then inserted in front of it, where the reference's text has them)
    par = builder.create_parallel_op([1], threads)
    builder.set_insertion_point_to_start(entry)
    qs, ks, vs = [ab.memref_alloc(element, t.type.shape, MemorySpace.SHARED, 1024).results[0] for t in (q, k, v)]
    builder.set_insertion_point_to_start(par.add_entry_block())
    views = []
    for glob, shared in ((q, qs), (k, ks), (v, vs)):
        gv, sv = ab.layout_view(glob).results[0], ab.layout_view(shared).results[0]
        builder.create_copy_op(gv, sv, [], [])
        views.append(sv)
    qv, kv, vv = views
    s_ty = ab.tensor_ty(f32, [n_q, n_kv])
    scores = ab.mma(qv, kv, ab.constant(s_ty, 0.0).results[0], trans_b=True).results[0]
    scaled = ab.binary("arith.mulf", scores, ab.constant(s_ty, scale_bits_or_value).results[0]).results[0]
    row_max = ab.reduce_tensor(scaled, "max", 1).results[0]
    centered = ab.binary("arith.subf", scaled, ab.broadcast(row_max, ab.empty(s_ty).results[0], [1]).results[0]).results[0]
    e = ab.exp(centered).results[0]
    row_sum = ab.reduce_tensor(e, "sum", 1).results[0]
    normalized = ab.binary("arith.divf", e, ab.broadcast(row_sum, ab.empty(s_ty).results[0], [1]).results[0]).results[0]
    p = ab.truncf(normalized, element).results[0]
    o_ty = ab.tensor_ty(f32, [n_q, d])
    result = ab.mma(p, vv, ab.constant(o_ty, 0.0).results[0]).results[0]
    if out_element != f32:
        result = ab.truncf(result, out_element).results[0]
    ab.tile_store(result, ab.layout_view(o).results[0])
    return kernel


# ------------------------------------------------------------------------ recognising the graph


def _ops_of(kernel):
    out = []

    def visit(op):
        for r in op.regions:
            for blk in r.blocks:
                for child in blk.operations:
                    out.append(child)
                    visit(child)
    visit(kernel)
    return out


def _fail(what):
    raise ValueError(f"frisk-b200-execute: not the attention graph: {what}")


def attention_plan(kernel):
    """Host-only.  Resolve a kernel that holds the attention graph to
    ``(dict(S_q, S_kv, D, scale, dtype_in, dtype_out), (iq, ik, iv, io))`` (argument indices), following the
    use-def chain back from the ``frisk.tile_store``; raises ValueError naming the first deviation."""
    ir._verify(kernel)
    ops = _ops_of(kernel)
    entry = kernel.regions[0].front()
    copies = [op for op in ops if isinstance(op, ir.CopyOp)]

    def strip_view(v):
        while not v.is_arg and isinstance(v.owner, LayoutViewOp):
            v = v.owner.operands[0]
        return v

    def root_arg(v):
        """The global kernel argument a (possibly staged) memref operand holds the data of."""
        v = strip_view(v)
        if not v.is_arg and isinstance(v.owner, UpstreamOp) and v.owner.op_name == "memref.alloc":
            src = [c for c in copies if strip_view(c.operands[1]) is v]
            if len(src) != 1:
                _fail("a staging buffer must be filled by exactly one frisk.copy")
            v = strip_view(src[0].operands[0])
        if not (v.is_arg and v.owner is entry) or v.type.space != MemorySpace.GLOBAL:
            _fail("matrix operands must come from global kernel arguments")
        return v

    def producer(v, cls=None, name=None):
        if v.is_arg:
            _fail("expected an op result, found a block argument")
        op = v.owner
        if cls is not None and not isinstance(op, cls):
            _fail(f"expected {cls.op_name}, found {op.op_name}")
        if name is not None and not (isinstance(op, UpstreamOp) and op.op_name == name):
            _fail(f"expected {name}, found {op.op_name}")
        return op

    def zero_init(v):
        c = producer(v, name="arith.constant")
        if c.attrs["_value"] != 0.0:
            _fail("an mma of the graph must start from a zero accumulator")

    def broadcast_of(v, kind):
        b = producer(v, name="linalg.broadcast")
        if b.attrs["dimensions"] != [1]:
            _fail("row statistics must be broadcast along dim 1")
        r = producer(b.operands[0], ReduceTensorOp)
        if r.attrs["kind"] != kind or r.attrs["dim"] != 1:
            _fail(f"expected a row {kind} (reduce_tensor along dim 1)")
        return r

    stores = [op for op in ops if isinstance(op, TileStoreOp)]
    if len(stores) != 1:
        _fail(f"expected one frisk.tile_store, found {len(stores)}")
    out_val, out_ref = stores[0].operands
    o_arg = root_arg(out_ref)
    if isinstance(out_val.owner, UpstreamOp) and out_val.owner.op_name == "arith.truncf":
        out_val = out_val.owner.operands[0]
    pv = producer(out_val, MmaOp)
    if pv.attrs["trans_a"] or pv.attrs["trans_b"]:
        _fail("P.V takes V as stored ([keys, d])")
    zero_init(pv.operands[2])
    v_arg = root_arg(pv.operands[1])
    trunc = producer(pv.operands[0], name="arith.truncf")
    div = producer(trunc.operands[0], name="arith.divf")
    e = producer(div.operands[0], name="math.exp")
    row_sum = broadcast_of(div.operands[1], "sum")
    if row_sum.operands[0] is not e.results[0]:
        _fail("the row sum must be taken over the exponentials")
    sub = producer(e.operands[0], name="arith.subf")
    row_max = broadcast_of(sub.operands[1], "max")
    scaled = sub.operands[0]
    if row_max.operands[0] is not scaled:
        _fail("the row maximum must be taken over the scaled scores")
    mul = producer(scaled, name="arith.mulf")
    lhs, rhs = mul.operands
    if isinstance(lhs.owner, UpstreamOp) and lhs.owner.op_name == "arith.constant":
        lhs, rhs = rhs, lhs
    scale = producer(rhs, name="arith.constant").attrs["_value"]
    qk = producer(lhs, MmaOp)
    if qk.attrs["trans_a"] or not qk.attrs["trans_b"]:
        _fail("the scores are Q.K^T (trans_b)")
    zero_init(qk.operands[2])
    q_arg, k_arg = root_arg(qk.operands[0]), root_arg(qk.operands[1])
    n_q, n_kv, d = qk.attrs["m"], qk.attrs["n"], qk.attrs["k"]
    if (pv.attrs["m"], pv.attrs["n"], pv.attrs["k"]) != (n_q, d, n_kv):
        _fail("the two mma shapes do not describe one attention tile")
    in_el, out_el = q_arg.type.element, o_arg.type.element
    if trunc.results[0].type.element != in_el or k_arg.type.element != in_el or v_arg.type.element != in_el:
        _fail("Q, K, V and the rounded probabilities must share one 16-bit element type")
    if in_el.name not in ("f16", "bf16") or out_el.name not in ("f32", in_el.name):
        _fail("inputs must be f16/bf16, the output that type or f32")
    if d not in (64, 128):
        _fail("head dimension must be 64 or 128")
    if not (scale > 0.0):
        _fail("the score scale must be positive")
    code = {"f16": "fp16", "bf16": "bf16", "f32": "fp32"}
    return (dict(S_q=n_q, S_kv=n_kv, D=d, scale=scale, dtype_in=code[in_el.name], dtype_out=code[out_el.name]),
            (q_arg.index, k_arg.index, v_arg.index, o_arg.index))

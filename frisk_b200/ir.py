"""MLIR-free re-host of the Frisk IR builder surface (``frisk_ffi.ir``).

The reference binds MLIR's C++ builder with pybind11 (``ffi/ir.cpp``); neither
MLIR nor the reference's fork of it exists on the machines this library runs on,
so the same Python surface is provided over a small self-contained IR: same
class and method names, same argument meaning, same exception types and message
prefixes, and op assembly printed the way the dialect's printers do
(``lib/Dialect/Frisk/IR/FriskOps.cpp:136-156,207-222,289-304,392-401,644-660``,
ODS formats in ``include/Dialect/Frisk/IR/FriskOps.td``).

Only what the GEMM / attention path needs is here: types, blocks, the structured
ops ``kernel/parallel/block/for``, ``alloc_buffer/copy/fill/reduce/gemm``.  The
affine-expression algebra of ``ffi/ir.cpp:640-875`` is reduced to the default,
identity and empty maps, which is what those ops use by default.
"""
import enum

from . import capi

# ------------------------------------------------------------------------ enums


class MemorySpace(enum.IntEnum):
    """include/Dialect/Frisk/IR/FriskEnums.td:6-8"""
    LOCAL = 0
    GLOBAL = 1
    SHARED = 3


GLOBAL, SHARED, LOCAL = MemorySpace.GLOBAL, MemorySpace.SHARED, MemorySpace.LOCAL


class GemmWarpPolicy(enum.IntEnum):
    """include/Dialect/Frisk/IR/FriskEnums.td:17-20"""
    Square = 0
    FullRow = 1
    FullCol = 2
    Auto = 3


_SUPPORTED_THREADS = (32, 64, 128, 256, 512, 1024)  # FriskOps.cpp:43-46

# ------------------------------------------------------------------------ types


class type:  # noqa: N801  (name kept from the reference binding)
    """A value type.  kind: 'float' | 'int' | 'index' | 'memref' | 'function' | 'tensor'."""

    def __init__(self, kind, **kw):
        self.kind = kind
        self.__dict__.update(kw)

    # predicates of the reference's ``type`` binding
    def is_f16(self):
        return self.kind == "float" and self.name == "f16"

    def is_bf16(self):
        return self.kind == "float" and self.name == "bf16"

    def is_f32(self):
        return self.kind == "float" and self.name == "f32"

    def is_f64(self):
        return self.kind == "float" and self.name == "f64"

    def is_memref(self):
        return self.kind == "memref"

    def get_shape(self):
        return list(self.shape)

    def get_element_type(self):
        return self.element

    def get_memory_space(self):
        return self.space

    def _key(self):
        if self.kind in ("float", "int"):
            return (self.kind, self.name)
        if self.kind == "index":
            return ("index",)
        if self.kind in ("memref", "tensor"):
            return (self.kind, tuple(self.shape), self.element._key(), getattr(self, "map", None) and str(self.map),
                    int(getattr(self, "space", 0)))
        return ("function", tuple(t._key() for t in self.inputs), tuple(t._key() for t in self.results))

    def __eq__(self, other):
        return isinstance(other, type) and self._key() == other._key()

    def __hash__(self):
        return hash(self._key())

    def __str__(self):
        if self.kind in ("float", "int"):
            return self.name
        if self.kind == "index":
            return "index"
        if self.kind in ("memref", "tensor"):
            dims = "x".join(["?" if d < 0 else str(d) for d in self.shape] + [str(self.element)])
            if self.kind == "tensor":
                return f"tensor<{dims}>"
            tail = ""
            if self.map is not None and not self.map.is_identity():
                tail += f", {self.map}"
            if int(self.space) != 0:
                tail += f", {int(self.space)}"
            return f"memref<{dims}{tail}>"
        ins = ", ".join(map(str, self.inputs))
        outs = ", ".join(map(str, self.results))
        return f"({ins}) -> ({outs})"

    __repr__ = __str__


_DTYPE_OF_FLOAT = {"f16": capi.F16, "bf16": capi.BF16, "f32": capi.F32}
_FLOAT_STRINGS = {"e4m3fn": "f8E4M3FN", "e5m2": "f8E5M2", "fp16": "f16", "fp32": "f32", "fp64": "f64"}


def _float_from_string(dtype):
    """The string dtypes ``create_alloc_buffer_op`` / ``create_fill_op`` accept
    (ffi/ir.cpp:398-411): no bf16 there in the reference either."""
    if dtype not in _FLOAT_STRINGS:
        raise ValueError("invalid float type")
    return type("float", name=_FLOAT_STRINGS[dtype])


from .affine import (AffineExpr, AffineExprKind, AffineMap, get_affine_binary_op_expr,  # noqa: E402,F401
                     get_affine_constant_expr, get_affine_constant_exprs, get_affine_dim_expr,
                     get_affine_symbol_expr)


# ------------------------------------------------------------------------ IR skeleton


class value:  # noqa: N801
    def __init__(self, ty, owner, index, is_arg):
        self.type, self.owner, self.index, self.is_arg = ty, owner, index, is_arg

    def get_type(self):
        return self.type

    def __str__(self):
        return f"<value {self.type}>"


class block:  # noqa: N801
    def __init__(self, arg_types=()):
        self.arguments = [value(t, self, i, True) for i, t in enumerate(arg_types)]
        self.operations = []
        self.parent_op = None

    def get_argument(self, idx):
        if idx >= len(self.arguments):
            raise IndexError("Block argument index out of range")
        return self.arguments[idx]

    def get_num_arguments(self):
        return len(self.arguments)

    def add_argument(self, ty):
        v = value(ty, self, len(self.arguments), True)
        self.arguments.append(v)
        return v


class region:  # noqa: N801
    def __init__(self, parent):
        self.blocks = []
        self.parent = parent

    def push_back(self, blk):
        blk.parent_op = self.parent
        self.blocks.append(blk)

    def empty(self):
        return not self.blocks

    def front(self):
        return self.blocks[0]


class OpState:
    """An operation: name, operands, results, attributes, regions."""
    op_name = "builtin.unknown"

    def __init__(self, operands=(), result_types=(), attrs=None, num_regions=0):
        self.operands = list(operands)
        self.results = [value(t, self, i, False) for i, t in enumerate(result_types)]
        self.attrs = dict(attrs or {})
        self.regions = [region(self) for _ in range(num_regions)]
        self.parent_block = None

    # -- reference OpState surface (ffi/ir.cpp:546-575)
    def set_attr(self, name, attr):
        self.attrs[name] = attr

    def get_num_results(self):
        return len(self.results)

    def get_result(self, idx=0):
        if idx >= len(self.results):
            raise IndexError("Op result index out of range")
        return self.results[idx]

    def get_region(self, idx):
        if idx >= len(self.regions):
            raise IndexError("Op region index out of range")
        return self.regions[idx]

    def get_name(self):
        return self.op_name

    def verify(self):
        try:
            _verify(self)
            return True
        except ValueError:
            return False

    def dump(self):
        print(str(self))

    def __str__(self):
        return _Printer().print_op(self)

    def walk(self, fn):
        for r in self.regions:
            for b in r.blocks:
                for op in list(b.operations):
                    op.walk(fn)
        fn(self)


class EndOp(OpState):
    op_name = "frisk.end"


class module(OpState):  # noqa: N801
    op_name = "builtin.module"

    def __init__(self):
        super().__init__(num_regions=1)
        self.regions[0].push_back(block())
        self.context = None

    def push_back(self, op):
        body = self.regions[0].front()
        if op.parent_block is body:
            return
        if op.parent_block is not None:
            op.parent_block.operations.remove(op)
        op.parent_block = body
        body.operations.append(op)

    def get_kernel(self, name):
        for op in self.regions[0].front().operations:
            if isinstance(op, KernelOp) and op.attrs["sym_name"] == name:
                return op
        return None

    def erase_kernel(self, name):
        k = self.get_kernel(name)
        if k is not None:
            self.regions[0].front().operations.remove(k)

    def has_function(self, name):
        return False

    def dump(self, log=""):
        if log:
            print(log)
        print(str(self))


class KernelOp(OpState):
    op_name = "frisk.kernel"

    def __init__(self, name, fn_type):
        super().__init__(attrs={"sym_name": name, "function_type": fn_type}, num_regions=1)

    @property
    def type(self):
        return self.attrs["function_type"]

    def get_num_arguments(self):
        return len(self.attrs["function_type"].inputs)

    def arg(self, idx):
        if idx >= self.get_num_arguments():
            raise IndexError("Kernel argument index out of range")
        return self.regions[0].front().get_argument(idx)

    def add_entry_block(self):
        blk = block(self.attrs["function_type"].inputs)
        self.regions[0].push_back(blk)
        blk.operations.append(_owned(EndOp(), blk))  # implicit terminator
        return blk


class ParallelOp(OpState):
    op_name = "frisk.parallel"

    def __init__(self, grid, threads):
        super().__init__(attrs={"ranges": list(grid), "threads": int(threads)}, num_regions=1)

    def get_grid(self):
        return list(self.attrs["ranges"])

    def get_thread_num(self):
        return self.attrs["threads"]

    def get_grid_dim(self):
        return len(self.attrs["ranges"])

    def get_ivs(self):
        return list(self.regions[0].front().arguments)

    def add_entry_block(self):
        blk = block([type("index")] * len(self.attrs["ranges"]))
        self.regions[0].push_back(blk)
        blk.operations.append(_owned(EndOp(), blk))
        return blk


class BlockOp(OpState):
    op_name = "frisk.block"

    def get_ivs(self):
        return list(self.regions[0].front().arguments)

    def get_block_ranges(self):
        return list(self.attrs["ranges"])

    def get_iteration_num(self):
        n = 1
        for r in self.attrs["ranges"]:
            n *= r
        return n

    def get_block_dim(self):
        return len(self.attrs["ranges"])


class ForOp(OpState):
    op_name = "frisk.for"

    def get_induction_var(self):
        return self.regions[0].front().arguments[0]

    def get_lower_bound(self):
        return self.attrs["lower"]

    def get_upper_bound(self):
        return self.attrs["upper"]

    def get_step(self):
        return self.attrs["step"]


class AllocBufferOp(OpState):
    op_name = "frisk.alloc_buffer"

    def get_alignment(self):
        return self.attrs["alignment"]

    def get_memroy_space(self):  # spelling kept from the reference binding
        return self.attrs["memorySpace"]

    def get_memref_ty(self):
        return self.results[0].type


class CopyOp(OpState):
    op_name = "frisk.copy"

    def get_src_memref(self):
        return self.operands[0]

    def get_dst_memref(self):
        return self.operands[1]

    def get_src_memref_ty(self):
        return self.operands[0].type

    def get_dst_memref_ty(self):
        return self.operands[1].type

    def get_src_affine_map(self):
        return self.attrs["srcMap"]

    def get_dst_affine_map(self):
        return self.attrs["dstMap"]

    def get_src_indices(self):
        return list(self.operands[2:2 + self.attrs["_nsrc"]])

    def get_dst_indices(self):
        return list(self.operands[2 + self.attrs["_nsrc"]:])

    def get_src_extents(self):
        return list(self.attrs["srcExtents"])

    def get_dst_extents(self):
        return list(self.attrs["dstExtents"])


class FillOp(OpState):
    op_name = "frisk.fill"

    def get_memref(self):
        return self.operands[0]


class ReduceOp(OpState):
    op_name = "frisk.reduce"

    def get_src_memref(self):
        return self.operands[0]

    def get_dst_memref(self):
        return self.operands[1]

    def get_reduce_dim(self):
        return self.attrs["dim"]


class GemmOp(OpState):
    op_name = "frisk.gemm"

    def get_matrix_A(self):
        return self.operands[0]

    def get_matrix_B(self):
        return self.operands[1]

    def get_matrix_C(self):
        return self.operands[2]

    def get_all_matrix(self):
        return list(self.operands)


def _owned(op, blk):
    op.parent_block = blk
    return op


# ------------------------------------------------------------------------ context / builder


class context:  # noqa: N801
    def __init__(self):
        self.dialects_loaded = False
        self.multithreading = True

    def disable_multithreading(self):
        self.multithreading = False


class _FriskNamespace:
    """``F.frisk``: dialect-level helpers and op classes (ffi/ir.cpp:35-136)."""
    GemmOp, KernelOp, ParallelOp, BlockOp, ForOp = GemmOp, KernelOp, ParallelOp, BlockOp, ForOp
    AllocBufferOp, CopyOp, FillOp, ReduceOp = AllocBufferOp, CopyOp, FillOp, ReduceOp

    @staticmethod
    def load_dialects(ctx):
        ctx.dialects_loaded = True


frisk = _FriskNamespace()


def _gemm_dtype(ty):
    if ty.kind == "memref" and ty.element.kind == "float":
        return _DTYPE_OF_FLOAT.get(ty.element.name, 100 + hash(ty.element.name) % 100)
    return -1


class builder:  # noqa: N801
    """``F.builder(ctx)``: the reference's ``OpBuilderWithLoc`` surface (ffi/ir.cpp:145-465)."""

    def __init__(self, ctx):
        self.context = ctx
        self._block = None
        self._pos = None  # index into block.operations where the next op goes

    # -- module / insertion point
    def create_module(self):
        return module()

    def set_insertion_point_to_start(self, blk):
        self._block, self._pos = blk, 0

    def set_insertion_point_to_end(self, blk):
        self._block, self._pos = blk, len(blk.operations)

    def set_insertion_point_after(self, op):
        blk = op.parent_block
        self._block, self._pos = blk, blk.operations.index(op) + 1

    def get_insertion_block(self):
        return self._block

    def get_insertion_point(self):
        return (self._block, self._pos)

    def restore_insertion_point(self, pt):
        self._block, self._pos = pt

    def new_block(self):
        return block()

    def _insert(self, op):
        if self._block is None:
            return op  # detached, as an MLIR builder without insertion point
        self._block.operations.insert(self._pos, _owned(op, self._block))
        self._pos += 1
        return op

    # -- types
    def get_bool_ty(self):
        return type("int", name="i8")

    def get_int64_ty(self):
        return type("int", name="i64")

    def get_f64_ty(self):
        return type("float", name="f64")

    def get_f16_ty(self):
        return type("float", name="f16")

    def get_bf16_ty(self):
        return type("float", name="bf16")

    def get_f32_ty(self):
        return type("float", name="f32")

    def get_ranked_tensor_ty(self, element, shape):
        return type("tensor", shape=list(shape), element=element)

    def get_memref_ty(self, elementType, shape, map=None, space=MemorySpace.GLOBAL):  # noqa: A002
        m = map if (map is not None and bool(map)) else None
        return type("memref", shape=[int(d) for d in shape], element=elementType, map=m, space=MemorySpace(space))

    def get_function_ty(self, in_types, out_types):
        return type("function", inputs=list(in_types), results=list(out_types))

    def get_kernel_ty(self, in_types):
        return type("function", inputs=list(in_types), results=[])

    # -- attrs / maps (the subset the structured ops use)
    def get_bool_attr(self, v):
        return bool(v)

    def get_int32_attr(self, v):
        return int(v)

    def get_float_attr(self, v, dtype):
        return (float(v), _float_from_string(dtype))

    # affine expressions (ffi/ir.cpp:303-308)
    def get_affine_dim_expr(self, position):
        return get_affine_dim_expr(position)

    def get_affine_symbol_expr(self, position):
        return get_affine_symbol_expr(position)

    def get_affine_constant_expr(self, value):
        return get_affine_constant_expr(value)

    def get_empty_affine_map(self):
        return AffineMap(empty=True)

    def get_multi_dim_identity_map(self, rank):
        return AffineMap(rank=rank)

    def get_dim_identity_map(self):
        return AffineMap(rank=1)

    # -- ops
    def create_kernel_op(self, mod, name, kernel_type):
        existing = mod.get_kernel(name)
        if existing is not None:
            return existing
        if not isinstance(kernel_type, type) or kernel_type.kind != "function":
            raise ValueError("invalid kernel function type")
        return self._insert(KernelOp(name, kernel_type))

    def create_parallel_op(self, grid, threads):
        blk = self._block
        if blk is None or len(blk.operations) != 1:
            raise ValueError("invalid parallel create")  # ffi/ir.cpp:363-370
        return self._insert(ParallelOp(grid, threads))

    def _structured(self, op, arg_types, body):
        blk = block(arg_types)
        op.regions[0].push_back(blk)
        saved = (self._block, self._pos)
        self._insert(op)
        after = (self._block, self._pos)
        self.set_insertion_point_to_start(blk)
        try:
            body(blk.arguments)
            self._insert(EndOp())
        finally:
            self._block, self._pos = after if saved[0] is not None else saved
        return op

    def create_block_op(self, block_range, py_func):
        op = BlockOp(attrs={"ranges": [int(r) for r in block_range]}, num_regions=1)
        return self._structured(op, [type("index")] * len(block_range), lambda ivs: py_func(self, list(ivs)))

    def create_for_op(self, lower, upper, step, py_func):
        op = ForOp(attrs={"lower": int(lower), "upper": int(upper), "step": int(step)}, num_regions=1)
        return self._structured(op, [type("index")], lambda ivs: py_func(self, ivs[0]))

    def create_alloc_buffer_op(self, shape, dtype, space=MemorySpace.GLOBAL, alignment=0):
        element = _float_from_string(dtype)
        if alignment < 0:
            raise ValueError("alignment must be non-negative")
        ty = type("memref", shape=[int(d) for d in shape], element=element, map=None, space=MemorySpace(space))
        return self._insert(AllocBufferOp(result_types=[ty], attrs={
            "shape": list(shape), "elementType": element, "alignment": int(alignment),
            "memorySpace": MemorySpace(space)}))

    def create_copy_op(self, src, dst, srcIndices, dstIndices, srcMap=None, dstMap=None,  # noqa: N803
                       srcExtents=(), dstExtents=()):
        have_maps = bool(srcMap) and bool(dstMap)
        if not have_maps and (bool(srcMap) or bool(dstMap) or srcExtents or dstExtents):
            raise RuntimeError("copy op map error.")
        if not have_maps:
            # FriskOps.cpp:553-567: empty indices denote a whole tile
            srcMap = AffineMap(empty=True) if not srcIndices else AffineMap(rank=len(src.type.shape))
            dstMap = AffineMap(empty=True) if not dstIndices else AffineMap(rank=len(dst.type.shape))
        if not srcExtents:
            d_ext = list(dst.type.shape)
            pad = len(src.type.shape) - len(d_ext)
            if pad < 0:
                raise ValueError("src rank must be >= dst rank")
            srcExtents, dstExtents = [1] * pad + d_ext, d_ext
        return self._insert(CopyOp(operands=[src, dst, *srcIndices, *dstIndices], attrs={
            "srcMap": srcMap, "dstMap": dstMap, "srcExtents": list(srcExtents), "dstExtents": list(dstExtents),
            "_nsrc": len(srcIndices)}))

    def create_fill_op(self, memref, v, dtype):
        return self._insert(FillOp(operands=[memref], attrs={"value": (float(v), _float_from_string(dtype))}))

    def create_reduce_op(self, src, dst, kind, dim, clear=True, legacy_semantics=None):
        op = ReduceOp(operands=[src, dst], attrs={"kind": str(kind), "dim": int(dim), "clear": bool(clear)})
        if legacy_semantics is not None:
            op.attrs["frisk.legacy_semantics"] = str(legacy_semantics)
        return self._insert(op)

    def create_gemm_op(self, A, B, C, transA=False, transB=False, clear_accum=False,  # noqa: N803
                       legacy_semantics=None):
        """ffi/ir.cpp:323-354: M, K from A and N from B honouring the transposes, then the
        contract check of LegacyImportSemantics.cpp:11-46 (done by the C library)."""
        a_ty, b_ty = A.type, B.type
        if (a_ty.kind != "memref" or b_ty.kind != "memref" or len(a_ty.shape) != 2 or len(b_ty.shape) != 2
                or min(a_ty.shape + b_ty.shape) < 0):
            raise ValueError("legacy-gemm-shape: A and B must be static rank-2 memrefs")
        m = a_ty.shape[1 if transA else 0]
        k = a_ty.shape[0 if transA else 1]
        n = b_ty.shape[0 if transB else 1]
        c_ty = C.type
        if c_ty.kind != "memref":
            raise ValueError("legacy-gemm-shape: A, B, and C must be memrefs")
        code, msg = capi.gemm_check_memrefs(a_ty.shape, _gemm_dtype(a_ty), b_ty.shape, _gemm_dtype(b_ty),
                                            c_ty.shape, _gemm_dtype(c_ty), transA, transB, m, n, k)
        if code:
            raise ValueError(msg)
        op = GemmOp(operands=[A, B, C], attrs={
            "transA": bool(transA), "transB": bool(transB), "M": m, "N": n, "K": k,
            "policy": GemmWarpPolicy.Square, "clear_accum": bool(clear_accum)})
        if legacy_semantics is not None:
            op.attrs["frisk.legacy_semantics"] = str(legacy_semantics)
        return self._insert(op)


# ------------------------------------------------------------------------ verification


def _verify(op):
    """Raise ValueError with the verifier message of the first failing op."""
    if isinstance(op, ParallelOp):  # FriskOps.cpp:224-234
        if op.attrs["threads"] not in _SUPPORTED_THREADS:
            raise ValueError("threads must be one of 32,64,128,256,512,1024")
        if not op.attrs["ranges"] or any(r <= 0 for r in op.attrs["ranges"]):
            raise ValueError("ranges must contain positive static extents")
        if op.regions[0].empty() or len(op.regions[0].front().arguments) != len(op.attrs["ranges"]):
            raise ValueError("range count must match the region induction arguments")
    elif isinstance(op, AllocBufferOp):  # FriskOps.cpp:481-489
        a = op.attrs["alignment"]
        if a < 0:
            raise ValueError("alignment must be non-negative")
        if a > 0 and a & (a - 1):
            raise ValueError("alignment must be a power of 2")
    elif isinstance(op, GemmOp):  # FriskOps.cpp:406-414
        if op.attrs["policy"] == GemmWarpPolicy.Auto:
            raise ValueError("Auto policy requires frisk.mma; legacy gemm has deterministic partitioning")
        a, b, c = (v.type for v in op.operands)
        code, msg = capi.gemm_check_memrefs(a.shape, _gemm_dtype(a), b.shape, _gemm_dtype(b), c.shape,
                                            _gemm_dtype(c), op.attrs["transA"], op.attrs["transB"],
                                            op.attrs["M"], op.attrs["N"], op.attrs["K"])
        if code:
            raise ValueError(msg)
    elif isinstance(op, FillOp):  # FriskOps.cpp:684-699
        if op.operands[0].type.element != op.attrs["value"][1]:
            raise ValueError(f"value type {op.attrs['value'][1]} does not match memref element type "
                             f"{op.operands[0].type.element}")
    elif isinstance(op, ReduceOp):  # FriskOps.cpp:728-762
        src, dst = op.operands[0].type, op.operands[1].type
        kind, dim = op.attrs["kind"], op.attrs["dim"]
        if src.kind != "memref" or dst.kind != "memref":
            raise ValueError("source and destination must be memref types")
        if dim < 0 or dim >= len(src.shape):
            raise ValueError(f"dimension {dim} is out of range for source of rank {len(src.shape)}")
        if kind not in ("add", "mul", "min", "max"):
            raise ValueError(f"unsupported reduce kind: {kind}. Supported: add, mul, min, max")
        if len(src.shape) != len(dst.shape) + 1:
            raise ValueError("destination rank must be one less than source rank. Got: "
                             f"{len(dst.shape)} vs {len(src.shape)}")
        kept = [i for i in range(len(src.shape)) if i != dim]
        for j, i in enumerate(kept):
            if src.shape[i] != dst.shape[j]:
                raise ValueError(f"non-reduced dimension mismatch: source[{i}] = {src.shape[i]} vs "
                                 f"destination[{j}] = {dst.shape[j]}")
        if src.element != dst.element:
            raise ValueError("source and destination must have the same element type")
    elif hasattr(op, "verify_op"):  # the tensor-level ops (tensor_ops.py) carry their own verifiers
        op.verify_op()
    elif isinstance(op, CopyOp):  # FriskOps.cpp:662-679
        if len(op.get_src_indices()) != op.attrs["srcMap"].get_num_inputs():
            raise ValueError("source index count does not match the source map")
        if len(op.get_dst_indices()) != op.attrs["dstMap"].get_num_inputs():
            raise ValueError("destination index count does not match the destination map")
    for r in op.regions:
        for b in r.blocks:
            for child in b.operations:
                _verify(child)


# ------------------------------------------------------------------------ printing


def _attr_text(v):
    if isinstance(v, bool):
        return "true" if v else "false"
    if isinstance(v, GemmWarpPolicy):
        return f"#frisk<gemm_warp_policy {v.name}>"
    if isinstance(v, MemorySpace):
        return f"#frisk<memory_space {v.name.capitalize()}>"
    if isinstance(v, int):
        return f"{v} : i64"
    if isinstance(v, str):
        return f'"{v}"'
    if isinstance(v, (list, tuple)) and len(v) == 2 and isinstance(v[1], type):
        return f"{v[0]:e} : {v[1]}"
    if isinstance(v, (list, tuple)):
        return "array<i64: " + ", ".join(str(int(x)) for x in v) + ">" if v else "array<i64>"
    return str(v)


def _attr_dict(attrs, elided=()):
    items = [(k, v) for k, v in sorted(attrs.items()) if k not in elided and not k.startswith("_")]
    if not items:
        return ""
    return " {" + ", ".join(f"{k} = {_attr_text(v)}" for k, v in items) + "}"


class _Printer:
    def __init__(self):
        self.names = {}
        self.n_arg = 0
        self.n_val = 0

    def name(self, v):
        if id(v) not in self.names:
            if v.is_arg:
                self.names[id(v)] = f"%arg{self.n_arg}"
                self.n_arg += 1
            else:
                self.names[id(v)] = f"%{self.n_val}"
                self.n_val += 1
        return self.names[id(v)]

    def _number(self, op):
        for r in op.regions:
            for b in r.blocks:
                for a in b.arguments:
                    self.name(a)
                for child in b.operations:
                    for res in child.results:
                        self.name(res)
                    self._number(child)

    def print_op(self, op):
        self._number(op)
        return "\n".join(self._op(op, 0))

    def _region(self, blk, indent, entry_args, terminators):
        lines = []
        pad = "  " * (indent + 1)
        if entry_args and blk.arguments:
            args = ", ".join(f"{self.name(a)}: {a.type}" for a in blk.arguments)
            lines.append("  " * indent + f"^bb0({args}):")
        for child in blk.operations:
            if isinstance(child, EndOp) and not terminators:
                continue
            lines += self._op(child, indent + 1)
        del pad
        return lines

    def _op(self, op, indent):
        pad = "  " * indent
        n = self.name
        if isinstance(op, module):
            body = self._region(op.regions[0].front(), indent, False, True)
            return [pad + "module {"] + body + [pad + "}"]
        if isinstance(op, KernelOp):
            ft = op.attrs["function_type"]
            head = f'{pad}frisk.kernel @{op.attrs["sym_name"]}(' + ", ".join(map(str, ft.inputs)) + ") {"
            body = self._region(op.regions[0].front(), indent, True, True) if not op.regions[0].empty() else []
            extra = _attr_dict(op.attrs, ("sym_name", "function_type"))
            return [head] + body + [pad + "}" + extra]
        if isinstance(op, ParallelOp):
            blk = op.regions[0].front()
            head = (f"{pad}frisk.parallel (" + ", ".join(n(a) for a in blk.arguments) + ") = (" +
                    ", ".join(map(str, op.attrs["ranges"])) + f"), threads = {op.attrs['threads']} {{")
            return [head] + self._region(blk, indent, False, True) + [pad + "}"]
        if isinstance(op, BlockOp):
            blk = op.regions[0].front()
            head = (f"{pad}frisk.block (" + ", ".join(n(a) for a in blk.arguments) + ") to (" +
                    ", ".join(map(str, op.attrs["ranges"])) + ") {")
            return [head] + self._region(blk, indent, False, False) + [pad + "}"]
        if isinstance(op, ForOp):
            blk = op.regions[0].front()
            step = f" step = {op.attrs['step']}" if op.attrs["step"] > 1 else ""
            head = f"{pad}frisk.for {n(blk.arguments[0])} = {op.attrs['lower']} to {op.attrs['upper']}{step} {{"
            return [head] + self._region(blk, indent, False, False) + [pad + "}"]
        if isinstance(op, AllocBufferOp):
            attrs = {k: v for k, v in op.attrs.items() if not (k == "alignment" and v == 0)}
            return [f"{pad}{n(op.results[0])} = frisk.alloc_buffer" +
                    _attr_dict(attrs, ("shape", "elementType", "memorySpace")) + f" -> {op.results[0].type}"]
        if isinstance(op, CopyOp):
            src_i = ", ".join(n(v) for v in op.get_src_indices())
            dst_i = ", ".join(n(v) for v in op.get_dst_indices())
            return [f"{pad}frisk.copy {n(op.operands[0])}[{src_i}], {n(op.operands[1])}[{dst_i}]" +
                    _attr_dict(op.attrs, ("srcMap", "dstMap")) +
                    f" : {op.operands[0].type}, {op.operands[1].type}"]
        if isinstance(op, FillOp):
            return [f"{pad}frisk.fill {n(op.operands[0])}" + _attr_dict(op.attrs) + f" : {op.operands[0].type}"]
        if isinstance(op, ReduceOp):
            return [f"{pad}frisk.reduce {n(op.operands[0])}, {n(op.operands[1])}" + _attr_dict(op.attrs) +
                    f" : {op.operands[0].type}, {op.operands[1].type}"]
        if isinstance(op, GemmOp):
            ops = ", ".join(n(v) for v in op.operands)
            tys = ", ".join(str(v.type) for v in op.operands)
            return [f"{pad}frisk.gemm({ops})" + _attr_dict(op.attrs) + f" : {tys}"]
        if isinstance(op, EndOp):
            return [pad + "frisk.end"]
        if hasattr(op, "print_assembly"):
            return [pad + op.print_assembly(n)]
        return [pad + f'"{op.op_name}"()' + _attr_dict(op.attrs)]

"""``FriskHelper`` / ``create_context`` / ``create_session``: the convenience layer of
``python/frisk/common/utils.py:18-181`` over the re-hosted builders, same names and
keyword arguments."""
from dataclasses import dataclass
from typing import Sequence, Tuple

from . import ir

__all__ = ["create_context", "create_session", "FriskHelper"]


def create_context(*, load_dialects=True, disable_multithreading=True):
    ctx = ir.context()
    if disable_multithreading:
        ctx.disable_multithreading()
    if load_dialects:
        ir.frisk.load_dialects(ctx)
    return ctx


def create_session(*, load_dialects=True, disable_multithreading=True):
    return FriskHelper.create(load_dialects=load_dialects, disable_multithreading=disable_multithreading)


@dataclass
class FriskHelper:
    context: ir.context
    builder: ir.builder
    module: ir.module

    @classmethod
    def create(cls, *, load_dialects=True, disable_multithreading=True):
        ctx = create_context(load_dialects=load_dialects, disable_multithreading=disable_multithreading)
        b = ir.builder(ctx)
        m = b.create_module()
        m.context = ctx
        return cls(ctx, b, m)

    def memref_type(self, shape, dtype="fp16", *, space=ir.MemorySpace.GLOBAL, layout=None):
        element = self._as_type(dtype)
        return self.builder.get_memref_ty(element, [int(d) for d in shape],
                                          layout if layout is not None else ir.AffineMap(), space)

    def new_kernel(self, name: str, arg_types: Sequence[ir.type]) -> Tuple[ir.KernelOp, ir.block]:
        kernel = self.builder.create_kernel_op(self.module, name, self.builder.get_kernel_ty(list(arg_types)))
        self.module.push_back(kernel)
        entry = kernel.add_entry_block()
        self.builder.set_insertion_point_to_start(entry)
        return kernel, entry

    def alloc_buffer(self, shape, dtype="fp16", *, space=ir.MemorySpace.LOCAL, alignment=0):
        op = self.builder.create_alloc_buffer_op(list(shape), self._as_dtype_str(dtype), space, alignment)
        return op.get_result(0)

    def create_gemm(self, A, B, C, *, trans_a=False, trans_b=False, clear_accum=False,  # noqa: N803
                    legacy_semantics=None):
        return self.builder.create_gemm_op(A, B, C, trans_a, trans_b, clear_accum, legacy_semantics)

    def create_reduce(self, src, dst, kind, dim, *, clear=True, legacy_semantics=None):
        return self.builder.create_reduce_op(src, dst, kind, dim, clear, legacy_semantics)

    def ensure_insertion_block(self):
        blk = self.builder.get_insertion_block()
        if blk is not None:
            return blk
        blk = self.builder.new_block()
        self.module.get_region(0).push_back(blk)
        self.builder.set_insertion_point_to_start(blk)
        return blk

    def dump(self, msg=None):
        if msg:
            print(msg)
        print(self.module)

    def _as_type(self, dtype):
        if isinstance(dtype, ir.type):
            return dtype
        key = dtype.lower()
        table = {"fp16": self.builder.get_f16_ty, "bf16": self.builder.get_bf16_ty, "fp32": self.builder.get_f32_ty,
                 "fp64": self.builder.get_f64_ty, "int64": self.builder.get_int64_ty}
        if key not in table:
            raise ValueError(f"Unsupported dtype '{dtype}'.")
        return table[key]()

    def _as_dtype_str(self, dtype):
        if isinstance(dtype, str):
            return dtype
        if dtype.is_f16():
            return "fp16"
        if dtype.is_f32():
            return "fp32"
        if dtype.is_f64():
            return "fp64"
        raise ValueError("Unsupported MLIR type for allocation helper.")

"""frisk_b200: B200 (sm_100a) GEMM and attention kernels behind the Frisk builder API.

``import frisk_b200 as F`` offers what ``import frisk as F`` offers for the GEMM /
attention path (``python/frisk/__init__.py:1-4``): the builder classes of
``frisk_ffi.ir`` and the ``FriskHelper`` conveniences, plus ``execute`` /
``attention_forward``, which run on the GPU through ``libfrisk_b200``.
"""
from . import capi, ir, packet, tensor_ops
from .execute import attention_forward, attention_geometry, execute, fused_plan, gemm, gemm_plan
from .helper import FriskHelper, create_context, create_session
from .affine import (AffineBinaryOpExpr, AffineConstantExpr, AffineDimExpr, AffineExpr, AffineExprKind,
                     AffineSymbolExpr, get_affine_binary_op_expr, get_affine_constant_expr, get_affine_constant_exprs,
                     get_affine_dim_expr, get_affine_symbol_expr)
from .ir import (AffineMap, AllocBufferOp, BlockOp, CopyOp, FillOp, ForOp, GemmOp, GemmWarpPolicy, KernelOp,
                 MemorySpace, OpState, ParallelOp, ReduceOp, block, builder, context, frisk, module, type, value)

from .tensor_ops import (AttentionBuilder, LayoutViewOp, MmaOp, ReduceTensorOp, TileLoadOp, TileStoreOp, attention_plan,
                         build_attention_kernel)

GLOBAL, SHARED, LOCAL = MemorySpace.GLOBAL, MemorySpace.SHARED, MemorySpace.LOCAL

__all__ = [name for name in globals() if not name.startswith("_")]

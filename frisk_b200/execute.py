"""``execute``: the run entry the reference lacks.

The reference's ``bind_test`` builds a GEMM through the builders and prints it
(``test/python/bind_test.py:64-66``); its NVIDIA lowering reaches a GPU only through
export -> PTX emission -> Triton -> ``cuLaunchKernel``
(``benchmark/layout/execution/run_execution.py:23-31,84``).  Here the kernel op is
pattern-matched on the host and dispatched through the C ABI of ``libfrisk_b200``:

* a kernel whose only computation is one ``frisk.gemm`` over its global memref
  arguments, possibly nested in ``frisk.parallel`` / ``frisk.block`` / ``frisk.for``
  (tile shapes there are scheduling hints; the hand-written kernels fix their own),
  optionally with a ``frisk.fill`` of C before it and a ``frisk.reduce`` of C along dim 1
  after it, which run inside the GEMM's epilogue;
* a kernel that holds the attention graph of
  ``test/Transforms/attention-layout-tile-d64.mlir:23-63`` over ``frisk.mma`` /
  ``frisk.reduce_tensor`` (``tensor_ops.attention_plan``): one [N_q, D] query tile over N_kv keys,
  run by the attention kernel in its normalised mode (the graph divides by the complete row sum
  before it rounds the probabilities);
* the batched attention forward, entered through :func:`attention_forward` with the
  launch contract of ``tiled_attention.py:28-61`` (compact BHSD, spec dict B/H/N/D).

Device memory, streams and process groups come from torch; the arithmetic does not.
"""
import math

from . import capi, ir, tensor_ops

_TORCH_DTYPE = None


def _torch():
    import torch
    global _TORCH_DTYPE
    if _TORCH_DTYPE is None:
        _TORCH_DTYPE = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
    return torch


_contexts = {}


def context_for(device_index):
    """One library context per device, created on first use."""
    ctx = _contexts.get(device_index)
    if ctx is None:
        ctx = capi.Context(device_index)
        _contexts[device_index] = ctx
    return ctx


def _stream_ptr(stream, device):
    torch = _torch()
    s = stream if stream is not None else torch.cuda.current_stream(device)
    return s.cuda_stream if hasattr(s, "cuda_stream") else int(s)


def _find_gemm(kernel):
    """Return (gemm_op, enclosing_ops, fill_op or None, reduce_op or None) or raise ValueError naming
    what is unsupported.  Besides the structural ops, the kernel may hold a ``frisk.fill`` of the
    gemm's C before the gemm and a ``frisk.reduce`` of C along dim 1 after it, in program order
    (the neighbours ``test/python/bind_test.py:44-53`` gives a gemm); they become the GEMM's epilogue."""
    found, order = [], []

    def visit(op, chain):
        for r in op.regions:
            for b in r.blocks:
                for child in b.operations:
                    if isinstance(child, ir.GemmOp):
                        found.append((child, chain))
                        order.append(child)
                    elif isinstance(child, (ir.FillOp, ir.ReduceOp)):
                        order.append(child)
                    elif isinstance(child, (ir.ParallelOp, ir.BlockOp, ir.ForOp)):
                        visit(child, chain + [child])
                    elif isinstance(child, (ir.AllocBufferOp, ir.EndOp)):
                        continue
                    else:
                        order.append(child)

    visit(kernel, [])
    if len(found) != 1:
        raise ValueError(f"frisk-b200-execute: expected exactly one frisk.gemm, found {len(found)}")
    gemm, chain = found[0]
    c_val = gemm.operands[2]
    at = order.index(gemm)
    fill = reduce = None
    for pos, op in enumerate(order):  # the first offender in program order is the one reported
        if op is gemm:
            continue
        if isinstance(op, ir.FillOp) and op.operands[0] is c_val and pos < at and fill is None:
            fill = op
        elif isinstance(op, ir.ReduceOp) and op.operands[0] is c_val and pos > at and reduce is None \
                and op.attrs["dim"] == 1:
            reduce = op
        else:
            raise ValueError(f"frisk-b200-execute: unsupported op {op.op_name} in an executed kernel"
                             " (besides the gemm: one fill of its C before it, one reduce of its C along dim 1 after it)")
    return gemm, chain, fill, reduce


def _kernel_of(module_or_kernel, name=None):
    if isinstance(module_or_kernel, ir.KernelOp):
        return module_or_kernel
    kernels = [op for op in module_or_kernel.regions[0].front().operations if isinstance(op, ir.KernelOp)]
    if name is not None:
        kernels = [k for k in kernels if k.attrs["sym_name"] == name]
    if len(kernels) != 1:
        raise ValueError(f"frisk-b200-execute: expected one kernel, found {len(kernels)}")
    return kernels[0]


def fused_plan(module_or_kernel, name=None, algo=capi.ALGO_AUTO):
    """Host-only: resolve the kernel to (descriptor, (ia, ib, ic), epilogue) where the indices name
    the kernel arguments bound to A, B and C and ``epilogue`` is None or a dict with ``fill``
    (value or None), ``reduce`` (kind or None), ``reduce_arg`` (argument index) and ``reduce_clear``."""
    kernel = _kernel_of(module_or_kernel, name)
    try:
        ir._verify(kernel)
    except ValueError as e:
        raise ValueError(f"frisk-b200-execute: kernel does not verify: {e}") from None
    gemm, chain, fill, reduce = _find_gemm(kernel)
    entry = kernel.regions[0].front()
    idx = []
    for v in gemm.operands:
        if not (v.is_arg and v.owner is entry):
            raise ValueError("frisk-b200-execute: gemm operands must be kernel arguments")
        if v.type.space != ir.MemorySpace.GLOBAL:
            raise ValueError("frisk-b200-execute: gemm operands must be global memrefs")
        idx.append(v.index)
    a = gemm.attrs
    side = fill is not None or reduce is not None
    if not a["clear_accum"] or side:
        trips = 1
        for op in chain:
            if isinstance(op, ir.ForOp):
                trips *= max(0, -(-(op.attrs["upper"] - op.attrs["lower"]) // max(1, op.attrs["step"])))
        if trips != 1:
            raise ValueError("frisk-b200-execute: an accumulating gemm inside a multi-trip frisk.for is not a single GEMM")
    ta, tc = gemm.operands[0].type, gemm.operands[2].type
    code = {"f16": capi.F16, "bf16": capi.BF16, "f32": capi.F32}
    if ta.element.name not in code or tc.element.name not in code:
        raise ValueError("legacy-gemm-type: no B200 kernel for this element type")
    desc = capi.gemm_desc(a["M"], a["N"], a["K"], code[ta.element.name], code[tc.element.name],
                          a["transA"], a["transB"], a["clear_accum"], algo=algo)
    desc.policy = int(a["policy"])
    epilogue = None
    if side:
        epilogue = {"fill": None, "reduce": None, "reduce_arg": None, "reduce_clear": True}
        if fill is not None:
            epilogue["fill"] = fill.attrs["value"][0]
        if reduce is not None:
            dst = reduce.operands[1]
            if not (dst.is_arg and dst.owner is entry) or dst.type.space != ir.MemorySpace.GLOBAL:
                raise ValueError("frisk-b200-execute: the reduce destination must be a global kernel argument")
            if reduce.attrs["kind"] not in ("max", "min", "add"):
                raise ValueError(f"frisk-b200-execute: no kernel for reduce kind {reduce.attrs['kind']}")
            # the row-reduction kernels write M elements of C's element type (the verifier has
            # already required exactly that of the destination memref; checked again because an
            # undersized buffer here would be a device-side out-of-bounds write)
            if list(dst.type.shape) != [a["M"]] or dst.type.element != tc.element:
                raise ValueError("frisk-b200-execute: the reduce destination must be memref<M x element type of C>")
            epilogue.update(reduce=reduce.attrs["kind"], reduce_arg=dst.index, reduce_clear=bool(reduce.attrs["clear"]))
    return desc, tuple(idx), epilogue


def gemm_plan(module_or_kernel, name=None, algo=capi.ALGO_AUTO):
    """Host-only: resolve a kernel whose only computation is one gemm to (descriptor, (ia, ib, ic))."""
    desc, idx, epilogue = fused_plan(module_or_kernel, name, algo)
    if epilogue is not None:
        raise ValueError("frisk-b200-execute: the kernel holds a fill or reduce next to its gemm: use fused_plan")
    return desc, idx


def execute(module_or_kernel, *tensors, stream=None, name=None, algo=capi.ALGO_AUTO):
    """Run the kernel on CUDA tensors bound positionally to its memref arguments."""
    torch = _torch()
    kernel = _kernel_of(module_or_kernel, name)
    attention = any(isinstance(op, tensor_ops.MmaOp) for op in tensor_ops._ops_of(kernel))
    if attention:
        spec, arg_idx = tensor_ops.attention_plan(kernel)
    else:
        desc, (ia, ib, ic), epilogue = fused_plan(kernel, algo=algo)
    arg_types = kernel.attrs["function_type"].inputs
    if len(tensors) != len(arg_types):
        raise ValueError(f"frisk-b200-execute: kernel takes {len(arg_types)} tensors, got {len(tensors)}")
    for t, ty in zip(tensors, arg_types):
        if t is None:
            continue
        if not t.is_cuda:
            raise ValueError("frisk-b200-execute: tensors must live on a CUDA device (there is no CPU path)")
        if list(t.shape) != list(ty.shape) or not t.is_contiguous():
            raise ValueError(f"frisk-b200-execute: tensor of shape {list(t.shape)} does not match {ty}")
        want = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}.get(ty.element.name)
        if t.dtype != want:
            raise ValueError(f"frisk-b200-execute: tensor dtype {t.dtype} does not match {ty}")
    if attention:
        q, k, v, o = (tensors[i] for i in arg_idx)
        adesc = capi.attn_desc(1, 1, spec["S_q"], spec["S_kv"], spec["D"], spec["scale"], False, spec["dtype_in"],
                               spec["dtype_out"], normalize_p=True)
        ctx = context_for(o.device.index or 0)
        ctx.attention_fwd(adesc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                          stream=_stream_ptr(stream, o.device))
        return o
    a, b, c = tensors[ia], tensors[ib], tensors[ic]
    dev = c.device.index or 0
    ctx = context_for(dev)
    if epilogue is None:
        ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=_stream_ptr(stream, c.device))
    else:
        dst = tensors[epilogue["reduce_arg"]] if epilogue["reduce"] else None
        epi = capi.gemm_epilogue(fill=epilogue["fill"], reduce=epilogue["reduce"],
                                 reduce_dst=dst.data_ptr() if dst is not None else None,
                                 reduce_clear=epilogue["reduce_clear"])
        ctx.gemm_fused(desc, epi, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=_stream_ptr(stream, c.device))
    return c


def gemm(a, b, c, *, trans_a=False, trans_b=False, clear_accum=True, algo=capi.ALGO_AUTO, stream=None):
    """Direct GEMM on CUDA tensors (the op ``create_gemm_op`` describes), bypassing IR."""
    torch = _torch()
    code = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
    m = a.shape[1] if trans_a else a.shape[0]
    k = a.shape[0] if trans_a else a.shape[1]
    n = b.shape[0] if trans_b else b.shape[1]
    rc, msg = capi.gemm_check_memrefs(list(a.shape), code.get(a.dtype, -1), list(b.shape), code.get(b.dtype, -2),
                                      list(c.shape), code.get(c.dtype, -3), trans_a, trans_b, m, n, k)
    if rc:
        raise ValueError(msg)
    for t in (a, b, c):
        if not t.is_cuda or t.stride(-1) != 1:
            raise ValueError("frisk-b200-execute: operands must be row-major CUDA tensors")
    desc = capi.gemm_desc(m, n, k, code[a.dtype], code[c.dtype], trans_a, trans_b, clear_accum,
                          lda=a.stride(0), ldb=b.stride(0), ldc=c.stride(0), algo=algo)
    ctx = context_for(c.device.index or 0)
    ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=_stream_ptr(stream, c.device))
    return c


def attention_geometry(spec):
    """Validate a launch spec dict (B, H, N, D [, N_kv]) the way
    ``tail_attention_reference.geometry`` does for its envelope, for ours."""
    keys = {"B", "H", "N", "D"}
    if not isinstance(spec, dict) or not keys <= set(spec) or any(not isinstance(spec[k], int) for k in keys):
        raise ValueError("expected integer B/H/N/D")
    if min(spec["B"], spec["H"], spec["N"]) <= 0 or spec["D"] not in (64, 128):
        raise ValueError("shape outside the attention launch contract")
    return spec["B"], spec["H"], spec["N"], spec["D"]


def attention_forward(spec, q, k, v, out, *, scale=None, causal=False, normalize_p=False, stream=None):
    """O = softmax(scale * Q K^T [+causal]) V on compact BHSD CUDA tensors.
    ``normalize_p`` selects the reference's two-pass semantics (P divided by the whole row sum
    before it is rounded to 16 bits, ``tiled_attention.py:697-698``) instead of the single pass."""
    torch = _torch()
    b, h, n, d = attention_geometry(spec)
    n_kv = int(spec.get("N_kv", n))
    code = {torch.float32: capi.F32, torch.float16: capi.F16, torch.bfloat16: capi.BF16}
    for t, s in ((q, n), (k, n_kv), (v, n_kv), (out, n)):
        if not t.is_cuda or not t.is_contiguous() or list(t.shape) != [b, h, s, d]:
            raise ValueError("attention operands must be compact BHSD CUDA tensors")
    if k.dtype != q.dtype or v.dtype != q.dtype or q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("attention inputs must share one 16-bit float type")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    desc = capi.attn_desc(b, h, n, n_kv, d, scale, causal, code[q.dtype], code[out.dtype], normalize_p)
    ctx = context_for(out.device.index or 0)
    ctx.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                      stream=_stream_ptr(stream, out.device))
    return out

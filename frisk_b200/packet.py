"""Front door for the reference's execution packets.

``frisk-opt -frisk-export-execution`` serialises a kernel whose layouts have been selected into a
JSON packet (``lib/Conversion/FriskLayoutToGPU/ExportExecution.cpp:46-296``):

    {"schema_version": 1 | 2,
     "values":     [{"id", "type", ["distributed": {...}], ["storage": {...}]}, ...],
     "operations": [{"name", "operands": [ids], "results": [ids], "attrs": {...},
                     ["execution" | "redistribution" | "fibers"]}, ...]}      (pre-order walk)

and the reference's adapter turns that into PTX (``benchmark/layout/execution/backend.py``).  Here the
packet is read back into the re-hosted IR (``tensor_ops``), recognised as the attention graph, and run
by ``frisk_b200_attention_fwd``.  The per-thread layout tables of the packet (``distributed``,
``execution``, ``fibers``, ``redistribution``) describe HOW the reference's generated kernel would
place values in registers; the hand-written kernel has its own fixed placement, so they are not
consumed.  What IS checked is the part of the ``frisk.mma_contract`` that names shared-memory operand
images, because that is where the two designs must agree: K-major 128-byte swizzle for Q and K,
MN-major 128-byte swizzle for V (``benchmark/layout/execution/tiled_attention.py:174-183``) are the
images this library's TMA loads write.  A packet that asks for anything else is refused.
"""
import json
import re
import struct

from . import ir, tensor_ops
from .ir import MemorySpace

_ALLOWED_OPS = (  # the pass's own preflight list (ExportExecution.cpp:88-90) plus its two f32 elementwise ops
    "builtin.module", "frisk.kernel", "frisk.parallel", "frisk.end", "frisk.storage_contract", "frisk.layout_view",
    "memref.alloc", "frisk.copy", "frisk.mma", "frisk.reduce_tensor", "frisk.tile_load", "frisk.tile_store",
    "frisk.convert_layout", "arith.constant", "arith.mulf", "arith.subf", "arith.divf", "arith.truncf", "math.exp",
    "tensor.empty", "linalg.broadcast", "linalg.yield", "arith.addf", "math.rsqrt")
_TYPE = re.compile(r"^(memref|tensor)<((?:\d+x)+)(f16|bf16|f32)\s*(?:,\s*(.*))?>$", re.S)
_SPLAT = re.compile(r"dense<\s*([^>]+?)\s*>")


def _reject(code, why):
    raise ValueError(f"[frisk-b200-packet code={code}] {why}")


def parse_type(text):
    """'memref<64x64xf16, 3>' / 'tensor<64x64xf32, #frisk.distributed<...>>' / 'index' -> ir.type."""
    text = text.strip()
    if text == "index":
        return ir.type("index")
    m = _TYPE.match(text)
    if not m:
        _reject("value-type", f"unsupported value type {text!r}")
    kind, dims, el, rest = m.groups()
    shape = [int(d) for d in dims.rstrip("x").split("x")]
    element = ir.type("float", name=el)
    if kind == "tensor":
        return ir.type("tensor", shape=shape, element=element)  # the encoding (if any) is not consumed
    space = 0
    if rest:
        last = rest.split(",")[-1].strip()
        if last.isdigit():
            space = int(last)
    return ir.type("memref", shape=shape, element=element, map=None, space=MemorySpace(space))


def _splat(attr_text):
    """Value of a dense f32 splat, hexadecimal payloads included (backend.py:16-27)."""
    m = _SPLAT.search(attr_text if isinstance(attr_text, str) else "")
    if not m:
        _reject("constant", "constant must be a dense scalar splat")
    token = m.group(1)
    if re.fullmatch(r"0[xX][0-9a-fA-F]{8}", token):
        bits = int(token, 16)
        return f"0x{bits:08X}", struct.unpack("<f", struct.pack("<I", bits))[0]
    try:
        v = float(token)
    except ValueError:
        _reject("constant", f"unsupported splat literal {token!r}")
    return ("0.0" if v == 0.0 else token), v


def check_schema(packet):
    """Structural checks the adapter relies on before it walks the operations."""
    if not isinstance(packet, dict) or packet.get("schema_version") not in (1, 2):
        _reject("schema", "schema_version must be 1 or 2")
    values, ops = packet.get("values"), packet.get("operations")
    if not isinstance(values, list) or not isinstance(ops, list) or not values or not ops:
        _reject("schema", "values and operations must be non-empty lists")
    ids = set()
    for v in values:
        if not isinstance(v, dict) or type(v.get("id")) is not int or not isinstance(v.get("type"), str):
            _reject("schema", "every value needs an integer id and a type string")
        if v["id"] in ids:
            _reject("schema", f"value id {v['id']} appears twice")
        ids.add(v["id"])
    for o in ops:
        if not isinstance(o, dict) or set(("name", "operands", "results", "attrs")) - set(o):
            _reject("schema", "every operation needs name, operands, results and attrs")
        if o["name"] not in _ALLOWED_OPS:
            _reject("unsupported-operation", f"unsupported execution operation {o['name']}")
        for i in list(o["operands"]) + list(o["results"]):
            if i not in ids:
                _reject("schema", f"operation {o['name']} names unknown value {i}")
    return ids


def check_mma_contract(op, which):
    """The shared-memory operand images a ``frisk.mma_contract`` asks for must be the ones this library's
    kernels use.  `which` is 'qk' (SS form, both operands K-major) or 'pv' (RS form, V MN-major)."""
    c = op["attrs"].get("frisk.mma_contract")
    if c is None:
        return  # a packet exported before instruction selection carries no contract: nothing to disagree with
    if not isinstance(c, dict) or c.get("version") != 1:
        _reject("mma-contract", "expected a version-1 frisk.mma_contract")
    if c.get("accumulator_type") != "f32" or c.get("input_type") not in ("f16", "bf16"):
        _reject("mma-contract", "kernels accumulate f16/bf16 products in f32")
    want_form, want_major = ("ss", "k") if which == "qk" else ("rs", "mn")
    if c.get("form") != want_form:
        _reject("mma-contract", f"the {which} product runs in {want_form.upper()} form here, the packet asks for {c.get('form')!r}")
    b = c.get("b_descriptor", {})
    if b.get("major") != want_major or b.get("swizzle") != 128:
        _reject("mma-contract", f"the B operand of the {which} product is {want_major}-major with 128-byte swizzle here")
    if which == "qk":
        a = c.get("a_descriptor", {})
        if a.get("major") != "k" or a.get("swizzle") != 128:
            _reject("mma-contract", "Q is staged K-major with 128-byte swizzle here")
    for d in (c.get("a_descriptor"), c.get("b_descriptor")):
        if d is not None and (d.get("leading", 0) % 16 or d.get("stride", 0) % 16):
            _reject("mma-contract", "descriptor offsets must be multiples of 16 bytes")


def to_kernel(packet):
    """Rebuild the kernel op of a packet in the re-hosted IR; returns (module, kernel)."""
    if isinstance(packet, (str, bytes)):
        packet = json.loads(packet)
    check_schema(packet)
    types = {v["id"]: parse_type(v["type"]) for v in packet["values"]}
    produced = {i for o in packet["operations"] for i in o["results"]}
    arg_ids = sorted(i for i, t in types.items() if i not in produced and t.kind == "memref")
    b = ir.builder(ir.context())
    module = b.create_module()
    kernels = [o for o in packet["operations"] if o["name"] == "frisk.kernel"]
    parallels = [o for o in packet["operations"] if o["name"] == "frisk.parallel"]
    if len(kernels) != 1 or len(parallels) != 1:
        _reject("target-envelope", "requires one kernel holding one parallel")  # ExportExecution.cpp:95
    name = kernels[0]["attrs"].get("sym_name", "frisk_execution")
    kernel = b.create_kernel_op(module, name, b.get_kernel_ty([types[i] for i in arg_ids]))
    module.push_back(kernel)
    entry = kernel.add_entry_block()
    val = {i: entry.get_argument(n) for n, i in enumerate(arg_ids)}
    b.set_insertion_point_to_start(entry)
    pa = parallels[0]["attrs"]
    ranges, threads = pa.get("ranges", [1]), pa.get("threads", 128)
    par = b.create_parallel_op(list(ranges), int(threads))
    body = par.add_entry_block()
    seen_parallel = False
    qk_seen = False
    for o in packet["operations"]:
        n, a = o["name"], o["attrs"]
        if n in ("builtin.module", "frisk.kernel", "frisk.end", "frisk.storage_contract", "linalg.yield"):
            continue
        if n == "frisk.parallel":
            seen_parallel = True
            b.set_insertion_point_to_start(body)
            continue
        if not seen_parallel:
            b.set_insertion_point_to_start(entry)  # allocations in front of the parallel
            b._pos = entry.operations.index(par)
        ins = [val[i] for i in o["operands"]]
        outs = [types[i] for i in o["results"]]
        if n == "memref.alloc":
            op = tensor_ops.UpstreamOp(n, (), outs, {"alignment": int(a["alignment"])} if "alignment" in a else {})
        elif n == "frisk.layout_view":
            op = tensor_ops.LayoutViewOp(operands=ins, result_types=outs)
        elif n == "frisk.convert_layout":
            val[o["results"][0]] = ins[0]  # a change of register placement only
            continue
        elif n == "frisk.copy":
            op = b.create_copy_op(ins[0], ins[1], [], [])
            continue
        elif n == "arith.constant":
            text, v = _splat(a.get("value"))
            op = tensor_ops.UpstreamOp(n, (), outs, {"text": text, "_value": v})
        elif n == "frisk.mma":
            check_mma_contract(o, "pv" if qk_seen else "qk")
            qk_seen = True
            op = tensor_ops.MmaOp(operands=ins, result_types=outs, attrs={
                "m": int(a["m"]), "n": int(a["n"]), "k": int(a["k"]), "trans_a": bool(a.get("trans_a", 0)),
                "trans_b": bool(a.get("trans_b", 0)), "policy": ir.GemmWarpPolicy.Square})
        elif n == "frisk.reduce_tensor":
            op = tensor_ops.ReduceTensorOp(operands=ins, result_types=outs, attrs={"kind": a["kind"], "dim": int(a["dim"])})
        elif n == "linalg.broadcast":
            op = tensor_ops.UpstreamOp(n, ins, outs, {"dimensions": [int(d) for d in a.get("dimensions", [])]})
        elif n == "frisk.tile_store":
            op = tensor_ops.TileStoreOp(operands=ins)
        elif n == "frisk.tile_load":
            op = tensor_ops.TileLoadOp(operands=ins, result_types=outs)
        else:  # arith.mulf / subf / divf / truncf / addf, math.exp / rsqrt, tensor.empty
            op = tensor_ops.UpstreamOp(n, ins, outs)
        b._insert(op)
        for i, r in zip(o["results"], op.results):
            val[i] = r
    return module, kernel


def plan(packet):
    """Host-only: (attention spec, argument indices) of a packet, or ValueError saying why it is refused."""
    _, kernel = to_kernel(packet)
    return tensor_ops.attention_plan(kernel)


def export(module, contracts=True):
    """Serialise a kernel built with ``tensor_ops`` the way the pass does for the op subset used here (names,
    operand / result ids in pre-order, attributes as JSON).  The layout proofs of a real packet (``distributed``,
    ``execution``, ``fibers``) are products of the reference's solver and are NOT reproduced.  `contracts` adds
    the ``frisk.mma_contract`` of the reference's D64 tile (tiled_attention.py:155-183) to the two mma ops."""
    ids, values, operations = {}, [], []

    def vid(v):
        if id(v) not in ids:
            ids[id(v)] = len(ids)
            values.append({"id": ids[id(v)], "type": str(v.type)})
        return ids[id(v)]

    n_mma = [0]

    def attrs_of(op):
        if isinstance(op, ir.KernelOp):
            return {"sym_name": op.attrs["sym_name"], "function_type": str(op.attrs["function_type"])}
        if isinstance(op, ir.ParallelOp):
            return {"ranges": list(op.attrs["ranges"]), "threads": op.attrs["threads"]}
        if isinstance(op, tensor_ops.MmaOp):
            a = {k: (int(v) if isinstance(v, bool) else v) for k, v in op.attrs.items() if k != "policy"}
            a = {k: v for k, v in a.items() if not (k.startswith("trans") and not v)}
            if contracts:
                k_major = {"major": "k", "swizzle": 128, "leading": 16, "stride": 1024, "entries": []}
                mn_major = {"major": "mn", "swizzle": 128, "leading": 1024, "stride": 1024, "entries": []}
                first = n_mma[0] == 0
                el = op.operands[1].type.element.name
                c = {"version": 1, "target": "sm_90a", "form": "ss" if first else "rs", "input_type": el,
                     "accumulator_type": "f32", "atom": [64, min(256, op.attrs["n"]), 16], "grid": [1, 1],
                     "repeats": [1, 1, op.attrs["k"] // 16], "packing": "none" if first else "f16x2-low-high",
                     "b_descriptor": k_major if first else mn_major}
                if first:
                    c["a_descriptor"] = dict(k_major)
                a["frisk.mma_contract"] = c
            n_mma[0] += 1
            return a
        if isinstance(op, tensor_ops.UpstreamOp) and op.op_name == "arith.constant":
            return {"value": f"dense<{op.attrs['text']}> : {op.results[0].type}"}
        return {k: v for k, v in op.attrs.items() if not k.startswith("_") and isinstance(v, (int, str, list))}

    def walk(op):
        for r in op.regions:
            for blk in r.blocks:
                for a in blk.arguments:
                    vid(a)
        operations.append({"name": "builtin.module" if isinstance(op, ir.module) else op.op_name,
                           "operands": [vid(v) for v in op.operands], "results": [vid(v) for v in op.results],
                           "attrs": attrs_of(op)})
        for r in op.regions:
            for blk in r.blocks:
                for child in blk.operations:
                    walk(child)

    walk(module)
    return {"schema_version": 1, "values": values, "operations": operations}


def execute(packet, q, k, v, o, stream=None):
    """Run a packet on CUDA tensors bound to its four global roots (query, keys, values, output)."""
    from .execute import execute as run_module   # the package attribute `execute` is that function, not the module
    module, _ = to_kernel(packet)
    return run_module(module, q, k, v, o, stream=stream)

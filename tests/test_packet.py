"""The execution-packet front door: the JSON the reference's export pass writes
(lib/Conversion/FriskLayoutToGPU/ExportExecution.cpp:46-296) read back into the re-hosted IR and resolved to
the attention kernel.  No packet is stored in the reference tree (its tests make them with frisk-opt at run
time), so the packets here are built from the same graph; where the reference checkout is present its own
adapter code (benchmark/layout/execution/backend.py:16-27,31-85,132-138) is asked to accept them."""
import copy
import json
import os
import sys

import pytest

import frisk_b200 as F
from frisk_b200 import packet
from tests.test_frontend import _reference_dir, build_attention_module


def make_packet(**kw):
    module, _ = build_attention_module(**kw)
    return packet.export(module), module


def test_packet_round_trip_and_plan():
    pk, module = make_packet()
    assert pk["schema_version"] == 1 and pk["operations"][0]["name"] == "builtin.module"
    names = [o["name"] for o in pk["operations"]]
    assert names.count("frisk.mma") == 2 and names.count("frisk.reduce_tensor") == 2 and "frisk.tile_store" in names
    rebuilt, kernel = packet.to_kernel(json.dumps(pk))
    assert str(rebuilt) == str(module)                       # same op assembly after the round trip
    spec, idx = packet.plan(pk)
    assert spec == dict(S_q=64, S_kv=64, D=64, scale=0.125, dtype_in="fp16", dtype_out="fp32") and idx == (0, 1, 2, 3)
    big, _ = make_packet(n_q=128, n_kv=1024, d=128, dtype="bf16", scale=128 ** -0.5, out="bf16")
    assert packet.plan(big)[0]["S_kv"] == 1024


def test_packet_refusals():
    pk, _ = make_packet()
    bad = copy.deepcopy(pk)
    bad["schema_version"] = 3
    with pytest.raises(ValueError, match="code=schema"):
        packet.plan(bad)
    bad = copy.deepcopy(pk)
    bad["operations"].append({"name": "gpu.launch", "operands": [], "results": [], "attrs": {}})
    with pytest.raises(ValueError, match="code=unsupported-operation"):
        packet.plan(bad)
    bad = copy.deepcopy(pk)
    bad["operations"][5]["operands"] = [999]
    with pytest.raises(ValueError, match="unknown value 999"):
        packet.plan(bad)
    # the shared-memory images the contract names must be the ones the kernels use
    mma = [i for i, o in enumerate(pk["operations"]) if o["name"] == "frisk.mma"]
    bad = copy.deepcopy(pk)
    bad["operations"][mma[0]]["attrs"]["frisk.mma_contract"]["b_descriptor"]["swizzle"] = 64
    with pytest.raises(ValueError, match="code=mma-contract.*128-byte swizzle"):
        packet.plan(bad)
    bad = copy.deepcopy(pk)
    bad["operations"][mma[1]]["attrs"]["frisk.mma_contract"]["b_descriptor"]["major"] = "k"
    with pytest.raises(ValueError, match="mn-major"):
        packet.plan(bad)
    bad = copy.deepcopy(pk)
    bad["operations"][mma[0]]["attrs"]["frisk.mma_contract"]["form"] = "rs"
    with pytest.raises(ValueError, match="SS form"):
        packet.plan(bad)
    # a graph that is not attention: the row sum taken over the scores instead of the exponentials
    bad = copy.deepcopy(pk)
    sums = [o for o in bad["operations"] if o["name"] == "frisk.reduce_tensor" and o["attrs"]["kind"] == "sum"]
    maxs = [o for o in bad["operations"] if o["name"] == "frisk.reduce_tensor" and o["attrs"]["kind"] == "max"]
    sums[0]["operands"] = list(maxs[0]["operands"])
    with pytest.raises(ValueError, match="not the attention graph"):
        packet.plan(bad)


def test_packet_without_contracts_is_accepted():
    module, _ = build_attention_module()
    pk = packet.export(module, contracts=False)
    assert all("frisk.mma_contract" not in o["attrs"] for o in pk["operations"])
    assert packet.plan(pk)[0]["D"] == 64


def test_reference_adapter_accepts_the_packet():
    """The reference's own adapter code on the packet: its splat decoder, the constructor checks of its emitter
    and its descriptor-field check.  Skipped where the reference checkout is not present."""
    exec_dir = os.path.join(_reference_dir(), "benchmark", "layout", "execution")
    if not os.path.exists(os.path.join(exec_dir, "backend.py")):
        pytest.skip("reference checkout not present")
    pk, _ = make_packet()
    sys.path.insert(0, exec_dir)   # the adapter imports its sibling modules by bare name, some of them lazily
    try:
        import backend
        em = backend.Emitter(pk)
    finally:
        sys.path.remove(exec_dir)
    consts = [o for o in pk["operations"] if o["name"] == "arith.constant"]
    assert [backend.splat_f32_bits(o["attrs"]["value"]) for o in consts] == [0, 0x3E000000, 0]
    assert sorted(em.v) == list(range(len(pk["values"])))
    for o in pk["operations"]:
        if o["name"] == "frisk.mma":
            c = o["attrs"]["frisk.mma_contract"]
            for key in ("a_descriptor", "b_descriptor"):
                if key in c:
                    assert set(c[key]) == {"entries", "leading", "major", "stride", "swizzle"}   # backend.py:133
            required = {"accumulator_type", "atom", "b_descriptor", "form", "grid", "input_type", "packing", "repeats",
                        "target", "version"} | ({"a_descriptor"} if c["form"] == "ss" else set())
            assert set(c) == required                                                           # backend.py:385-386

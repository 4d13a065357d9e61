"""Regenerate the golden attention vectors from the reference's OWN code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It imports ``benchmark/layout/execution/tail_attention_reference.py`` and
executes the ``reference()`` function of ``run_execution.py`` (lines 59-64; the
script itself cannot be imported because it runs a compile at import time, so
only that function's source lines are executed), then writes

* ``attention_tiled_d64.npz``  — inputs of every registered fixture
  (``tail_attention_reference.NAMES``) at several key counts with the
  reference's ``strict`` and ``fp64`` outputs,
* ``attention_tile_64x16.npz`` — the single-tile cases of
  ``run_execution.py:65-68`` with the reference output,
* ``ordered_sum.npz``          — ``ordered_sum`` on seeded rows.

The committed ``.npz`` files are what the tests read; the reference checkout is
not needed to run them.
"""
import importlib.util
import pathlib
import sys

import numpy as np

HERE = pathlib.Path(__file__).resolve().parent
LENGTHS = (64, 65, 130)
B, H = 1, 2


def load_tail(ref_root):
    path = ref_root / "benchmark/layout/execution/tail_attention_reference.py"
    spec = importlib.util.spec_from_file_location("tail_attention_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def load_tile_reference(ref_root):
    lines = (ref_root / "benchmark/layout/execution/run_execution.py").read_text().splitlines()
    start = next(i for i, l in enumerate(lines) if l.startswith("def reference(q,k,v)"))
    end = next(i for i in range(start + 1, len(lines)) if not lines[i].startswith(" "))
    scope = {"np": np}
    exec("\n".join(lines[start:end]), scope)
    return scope["reference"]


def main():
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref_root = pathlib.Path(sys.argv[1])
    tail = load_tail(ref_root)

    tiled = {}
    for n in LENGTHS:
        spec = dict(B=B, H=H, N=n, D=64, q_block=64, kv_block=64)
        for name in tail.NAMES:
            q, k, v = tail.inputs(spec, name)
            refs = tail.references((q, k, v), name)
            key = f"{name}/n{n}"
            tiled[key + "/q"], tiled[key + "/k"], tiled[key + "/v"] = q, k, v
            tiled[key + "/strict"] = refs["strict"].astype(np.float32)
            tiled[key + "/fp64"] = refs["fp64"].astype(np.float64)
    np.savez_compressed(HERE / "attention_tiled_d64.npz", **tiled)

    reference = load_tile_reference(ref_root)
    cases = []
    for seed in range(10):
        rng = np.random.default_rng(seed)
        cases.append(("seed%d" % seed, *[rng.uniform(-1, 1, (64, 16)).astype(np.float16) for _ in range(3)]))
    z = np.zeros((64, 16), np.float16)
    one = np.ones_like(z)
    coord = np.linspace(-1, 1, 1024).reshape(64, 16).astype(np.float16)
    hot = z.copy()
    hot[13, 7] = 1
    cancel = np.tile(np.array([1, -1], np.float16)[:, None], (32, 16))
    cases += [("zeroQK", z, z, coord), ("constant", one, one, one), ("signedcoords", coord, -coord, coord),
              ("onehotV", coord, coord, hot), ("cancelV", z, z, cancel)]
    tile = {}
    for name, q, k, v in cases:
        tile[name + "/q"], tile[name + "/k"], tile[name + "/v"] = q, k, v
        tile[name + "/o"] = reference(q, k, v)
    np.savez_compressed(HERE / "attention_tile_64x16.npz", **tile)

    sums = {}
    rng = np.random.default_rng(4)
    for n in (1, 7, 64, 65, 129, 193, 513, 1025):
        row = rng.random((3, n), dtype=np.float32)
        sums[f"n{n}/in"] = row
        sums[f"n{n}/out"] = tail.ordered_sum(row)
    np.savez_compressed(HERE / "ordered_sum.npz", **sums)
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()

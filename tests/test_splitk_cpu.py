"""Host-side logic of the K-split GEMM on CPU: partitioning, row ownership and the
exchange step, run as two gloo ranks.  The GEMM and the fp32->16-bit conversion are
test doubles here (torch CPU ops); on a GPU they are the library's kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from frisk_b200 import splitk


def test_plan_and_ownership():
    plan = splitk.make_plan(8192, 8192, 131072, 8, 3, panels=4)
    assert plan.k_local == 16384 and plan.k_lo == 3 * 16384
    assert plan.panel_rows == 2048 and plan.block_rows == 256
    rows = splitk.owned_rows(plan)
    assert rows[0] == (3 * 256, 4 * 256) and rows[3] == (3 * 2048 + 768, 3 * 2048 + 1024)
    # every row has exactly one owner
    seen = np.zeros(8192, int)
    for r in range(8):
        for lo, hi in splitk.owned_rows(plan, r):
            seen[lo:hi] += 1
    assert (seen == 1).all()
    with pytest.raises(ValueError):
        splitk.make_plan(64, 64, 100, 8, 0)      # K does not split into 16-byte slices
    with pytest.raises(ValueError):
        splitk.make_plan(30, 64, 128, 4, 0)      # rows do not split across ranks
    assert splitk.make_plan(96, 64, 128, 2, 0, panels=4).panels == 4
    assert splitk.make_plan(100, 64, 128, 2, 0, panels=4).panels == 2  # falls back to a panel count that divides


def _worker(rank, world, port, M, N, K, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        a = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16()
        b = torch.randn(N, K, generator=g).bfloat16()
        plan = splitk.make_plan(M, N, K, world, rank, panels=2)
        a_shard = a[:, plan.k_lo:plan.k_lo + plan.k_local].contiguous()
        b_shard = b[:, plan.k_lo:plan.k_lo + plan.k_local].contiguous()

        def gemm_fn(ap, bp, c):
            c.copy_(ap.float() @ bp.float().T)

        def convert_fn(src, dst):
            dst.copy_(src)

        op = splitk.SplitKGemm(plan, "bf16", device=torch.device("cpu"), group=dist.group.WORLD,
                               gemm_fn=gemm_fn, convert_fn=convert_fn)
        out = op.run(a_shard, b_shard)
        full = (a.float() @ b.float().T)
        for p, (lo, hi) in enumerate(splitk.owned_rows(plan)):
            assert torch.allclose(out[p].float(), full[lo:hi], rtol=2e-2, atol=2e-2)
        torch.save(out, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_exchange(tmp_path):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    M, N, K = 64, 48, 256
    mp.spawn(_worker, args=(2, port, M, N, K, str(tmp_path)), nprocs=2, join=True)
    outs = [torch.load(tmp_path / f"rank{r}.pt") for r in range(2)]
    g = torch.Generator().manual_seed(1)
    a = (torch.randn(M, K, generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, K, generator=g).bfloat16()
    full = torch.empty(M, N)
    for r in range(2):
        plan = splitk.make_plan(M, N, K, 2, r, panels=2)
        for p, (lo, hi) in enumerate(splitk.owned_rows(plan)):
            full[lo:hi] = outs[r][p].float()
    ref = a.double() @ b.double().T
    err = ((full.double() - ref).norm() / ref.norm()).item()
    assert err <= 5e-3


def test_push_slot_addresses_do_not_overlap():
    """Host logic of the fused path: g ranks x g owners, every (owner, rank) slot distinct and inside the owner's buffer."""
    from frisk_b200 import splitk
    g, slot_elems = 8, 1024 * 8192
    bases = [0x7000_0000_0000 + o * (1 << 32) for o in range(g)]
    seen = set()
    for rank in range(g):
        addrs = splitk.slot_addresses(bases, rank, slot_elems)
        assert len(addrs) == g
        for owner, a in enumerate(addrs):
            assert a % 16 == 0 and bases[owner] <= a and a + slot_elems * 4 <= bases[owner] + g * slot_elems * 4
            assert (owner, a) not in seen
            seen.add((owner, a))
    assert len(seen) == g * g

"""Deep-K GEMM split across GPUs: C = A . B^T with K divided among the ranks.

Each rank holds the K-slice ``[k_lo, k_hi)`` of A ([M, K/g]) and of B ([N, K/g], K
contiguous) and computes an fp32 partial product with the tcgen05 GEMM (an fp32 C for
16-bit inputs is inside the ``frisk.gemm`` contract,
``lib/Dialect/Frisk/IR/LegacyImportSemantics.cpp:26-35``).  The partials are summed with one
exchange step, a reduce-scatter over row blocks, and each rank rounds the rows it owns to
the 16-bit output type.  The reference has no multi-GPU path; this is new work.

To overlap the exchange with the arithmetic the M extent is cut into ``panels`` row panels:
while panel p's reduce-scatter runs on a communication stream, panel p+1's GEMM runs on the
compute stream (events order them; the host never waits).  Rank r therefore owns, in every
panel, the r-th block of ``M / (panels * g)`` rows: see :func:`owned_rows`.

torch.distributed supplies the process group and the collective; the arithmetic is the
library's kernels.
"""
from dataclasses import dataclass

from . import capi


@dataclass(frozen=True)
class SplitKPlan:
    M: int
    N: int
    K: int
    world: int
    rank: int
    panels: int

    @property
    def k_lo(self):
        return self.rank * self.k_local

    @property
    def k_local(self):
        return self.K // self.world

    @property
    def panel_rows(self):
        return self.M // self.panels

    @property
    def block_rows(self):
        return self.panel_rows // self.world


def make_plan(M, N, K, world, rank, panels=4):
    """Validate the partition: K splits evenly into 16-byte-aligned slices, every panel splits
    evenly into one row block per rank."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("split-k: bad rank/world")
    if K % world or (K // world) % 8:
        raise ValueError("split-k: K must divide into slices of a multiple of 8 elements")
    panels = max(1, int(panels))
    while panels > 1 and (M % panels or (M // panels) % world):
        panels -= 1
    if M % panels or (M // panels) % world:
        raise ValueError("split-k: M must divide into one row block per rank")
    return SplitKPlan(M, N, K, world, rank, panels)


def owned_rows(plan, rank=None):
    """Global row ranges [(lo, hi), ...] whose final values end on ``rank`` (one per panel)."""
    r = plan.rank if rank is None else rank
    return [(p * plan.panel_rows + r * plan.block_rows, p * plan.panel_rows + (r + 1) * plan.block_rows)
            for p in range(plan.panels)]


def _reduce_scatter(out, inp, group):
    """Sum ``inp`` ([world*rows, N]) over the group; ``out`` ([rows, N]) receives this rank's block."""
    import torch.distributed as dist
    if dist.get_backend(group) == "gloo":  # CPU test path: gloo has no reduce_scatter_tensor
        dist.all_reduce(inp, group=group)
        r = dist.get_rank(group)
        out.copy_(inp[r * out.shape[0]:(r + 1) * out.shape[0]])
    else:
        dist.reduce_scatter_tensor(out, inp, group=group)


class SplitKGemm:
    """Reusable state (fp32 partial buffers, streams, events) for one problem size."""

    def __init__(self, plan, dtype="bf16", device=None, ctx=None, group=None, gemm_fn=None, convert_fn=None):
        import torch
        self.plan, self.dtype, self.group = plan, dtype, group
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.on_gpu = self.device.type == "cuda"
        if self.on_gpu and ctx is None:
            raise ValueError("split-k: a library context is required on a CUDA device")
        self.ctx = ctx
        self._gemm_fn, self._convert_fn = gemm_fn, convert_fn
        out_dtype = {"bf16": torch.bfloat16, "fp16": torch.float16}[dtype]
        # two partial buffers so that panel p+1 can be computed while panel p is in flight
        self.partial = [torch.empty(plan.panel_rows, plan.N, dtype=torch.float32, device=self.device)
                        for _ in range(min(2, plan.panels))]
        self.reduced = torch.empty(plan.panels, plan.block_rows, plan.N, dtype=torch.float32, device=self.device)
        self.out = torch.empty(plan.panels, plan.block_rows, plan.N, dtype=out_dtype, device=self.device)
        if self.on_gpu:
            self.comm_stream = torch.cuda.Stream(self.device)
            self.ev_gemm = [torch.cuda.Event() for _ in range(plan.panels)]
            self.ev_comm = [torch.cuda.Event() for _ in range(plan.panels)]
            self.desc = capi.gemm_desc(plan.panel_rows, plan.N, plan.k_local, dtype, "fp32", False, True,
                                       clear_accum=True, algo=capi.ALGO_AUTO)

    def _gemm(self, a_panel, b, c, stream):
        if self._gemm_fn is not None:
            return self._gemm_fn(a_panel, b, c)
        self.ctx.gemm(self.desc, a_panel.data_ptr(), b.data_ptr(), c.data_ptr(), stream=stream.cuda_stream)

    def _convert(self, src, dst, stream):
        if self._convert_fn is not None:
            return self._convert_fn(src, dst)
        self.ctx.convert_f32(src.data_ptr(), dst.data_ptr(), src.numel(), self.dtype, stream=stream.cuda_stream)

    def run(self, a_shard, b_shard):
        """a_shard [M, K/g], b_shard [N, K/g] (both K-contiguous).  Returns ``self.out``
        ([panels, block_rows, N]): the rows :func:`owned_rows` lists, in that order."""
        plan = self.plan
        if tuple(a_shard.shape) != (plan.M, plan.k_local) or tuple(b_shard.shape) != (plan.N, plan.k_local):
            raise ValueError("split-k: shard shapes do not match the plan")
        if not self.on_gpu:
            for p in range(plan.panels):
                part = self.partial[p % len(self.partial)]
                self._gemm(a_shard[p * plan.panel_rows:(p + 1) * plan.panel_rows], b_shard, part, None)
                _reduce_scatter(self.reduced[p], part, self.group)
                self._convert(self.reduced[p], self.out[p], None)
            return self.out
        import torch
        compute = torch.cuda.current_stream(self.device)
        for p in range(plan.panels):
            part = self.partial[p % len(self.partial)]
            if p >= len(self.partial):
                compute.wait_event(self.ev_comm[p - len(self.partial)])  # the buffer's last exchange is done
            self._gemm(a_shard[p * plan.panel_rows:(p + 1) * plan.panel_rows], b_shard, part, compute)
            self.ev_gemm[p].record(compute)
            with torch.cuda.stream(self.comm_stream):
                self.comm_stream.wait_event(self.ev_gemm[p])
                _reduce_scatter(self.reduced[p], part, self.group)
                self._convert(self.reduced[p], self.out[p], self.comm_stream)
                self.ev_comm[p].record(self.comm_stream)
        compute.wait_event(self.ev_comm[plan.panels - 1])
        for p in range(max(0, plan.panels - len(self.partial)), plan.panels - 1):
            compute.wait_event(self.ev_comm[p])
        return self.out


def slot_addresses(owner_bases, rank, slot_elems):
    """Where rank ``rank`` stores its partial rows: every owner's buffer holds one fp32 slot of
    ``slot_elems`` elements per rank, in rank order; the result is this rank's slot at every owner."""
    return [int(base) + rank * slot_elems * 4 for base in owner_bases]


class SplitKGemmPush:
    """The same K-split product with the exchange FUSED into the GEMM: the epilogue of the
    tcgen05 kernel stores every finished fp32 tile straight into the memory of the GPU that owns
    its rows (``frisk_b200_gemm_push``: 16-byte stores over NVLink to buffers mapped with
    cudaIpc), so the transfer overlaps the arithmetic tile by tile and no SM is taken away by a
    collective kernel.  Rank r owns rows ``[r*M/g, (r+1)*M/g)`` and holds one slot of that many
    rows per rank; rank s writes only slot s, everywhere.

    Per call: push; a one-element all-reduce on the stream as the cross-GPU barrier (every rank's
    stores are then complete); sum this rank's g slots in slot order and round them
    (``frisk_b200_sum_slots``) -- the result does not depend on timing.  Two sets of slots
    alternate, so a rank that is already pushing call i+1 can never overwrite a slot its peer has
    not yet summed for call i."""

    def __init__(self, M, N, K, world, rank, dtype, ctx, group=None):
        import torch
        import torch.distributed as dist
        if M % world or K % world or (K // world) % 8 or world > 8:
            raise ValueError("split-k push: M and K must divide by the number of ranks (<= 8)")
        self.M, self.N, self.k_local, self.world, self.rank = M, N, K // world, world, rank
        self.rows = M // world
        self.slot_elems = self.rows * N
        self.ctx, self.group, self.dtype = ctx, group, dtype
        self.device = torch.device("cuda", torch.cuda.current_device())
        self.own, self.mapped, self.targets = [], [], []
        for _ in range(2):
            ptr, handle = ctx.peer_buffer_create(world * self.slot_elems * 4)
            handles = [None] * world
            if world > 1:
                dist.all_gather_object(handles, handle, group=group)
            else:
                handles = [handle]
            bases = [ptr if r == rank else ctx.peer_buffer_open(handles[r]) for r in range(world)]
            self.own.append(ptr)
            self.mapped.append(bases)
            self.targets.append(slot_addresses(bases, rank, self.slot_elems))
        self.out = torch.empty(self.rows, N, dtype={"bf16": torch.bfloat16, "fp16": torch.float16}[dtype],
                               device=self.device)
        self.token = torch.zeros(1, device=self.device)
        self.desc = capi.gemm_desc(M, N, self.k_local, dtype, "fp32", False, True, clear_accum=True,
                                   algo=capi.ALGO_TCGEN05_PAIR)
        self.calls = 0

    def run(self, a_shard, b_shard):
        """a_shard [M, K/g], b_shard [N, K/g] (K-contiguous).  Returns this rank's rows [M/g, N]."""
        import torch
        import torch.distributed as dist
        if tuple(a_shard.shape) != (self.M, self.k_local) or tuple(b_shard.shape) != (self.N, self.k_local):
            raise ValueError("split-k push: shard shapes do not match")
        buf = self.calls & 1
        self.calls += 1
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self.ctx.gemm_push(self.desc, a_shard.data_ptr(), b_shard.data_ptr(), self.targets[buf], self.rows, self.N,
                           stream=stream)
        if self.world > 1:
            dist.all_reduce(self.token, group=self.group)  # stream-ordered barrier across the GPUs
        self.ctx.sum_slots(self.own[buf], self.world, self.slot_elems, self.out.data_ptr(), self.slot_elems, self.dtype,
                           stream=stream)
        return self.out

    def close(self):
        for buf in range(len(self.mapped)):
            for r, ptr in enumerate(self.mapped[buf]):
                self.ctx.peer_buffer_close(ptr, owned=(r == self.rank))
        self.mapped, self.targets = [], []

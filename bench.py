#!/usr/bin/env python
"""Benchmark of the GEMM / attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  The headline workload is the fp16 GEMM M=N=K=4096, A row-major,
B column-major (NT), fp32 accumulation, fp16 output, on the tcgen05 kernel.  A "step" is
one pass of that GEMM.  With N > 1 (launched by torchrun, one rank per GPU) every rank
runs the same per-GPU problem on its own M-row shard of a 4096*N x 4096 x 4096 product
(independent output tiles, no collective): weak scaling.

Timing: CUDA events on the launching stream around every step, W >= 3 warm-up steps,
inputs rotate through buffer sets larger than L2 so no step finds its operands cached,
barrier + synchronize on both sides of the timed region, max over ranks.

Keys beyond the basic contract: `e2e` (same GEMM through the host-buffer C-ABI entry
point, pinned host memory, copies inside the timed region), `roofline`, `cpu_baseline`
(the numpy oracle on the host cores), `clocks`, `gpu_launches`, and `secondary` (the other
benchmark workloads, kernel-only, for information).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "TFLOP/s (% of B200 dense peak) for GEMM & attention at 1/2/4/8 GPUs"
NOMINAL_TENSOR_TFLOPS = 2250.0
NOMINAL_HBM_GBS = 8000.0
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
L2_BYTES = 126 * 1024 * 1024


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/ (one file per kernel and workload).
NCU_TRAFFIC = {"gemm_tcgen05_f16_4096": 101886464, "gemm_skinny_bf16_16x28672x8192": 479246080}


def ncu_traffic(key):
    return NCU_TRAFFIC.get(key)


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML (read-only queries) every few
    milliseconds while the timed region runs; falls back to one nvidia-smi query if NVML is
    not importable."""

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.samples = []
        self.stop_flag = False
        self.thread = None
        self.nvml = None
        self.handle = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if self.gpu < len(ids) and ids[self.gpu].isdigit():
                    index = int(ids[self.gpu])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nvml = None
            return
        self.thread = threading.Thread(target=self._poll, daemon=True)
        self.thread.start()

    def _poll(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                reasons = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle) if hasattr(
                    n, "nvmlDeviceGetCurrentClocksEventReasons") else n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                power = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                self.samples.append((time.time(), sm, reasons, power))
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self, t0, t1):
        self.stop_flag = True
        if self.nvml is None:
            return self._smi_once()
        if self.thread is not None:
            self.thread.join(timeout=1)
        n = self.nvml
        rows = [s for s in self.samples if t0 <= s[0] <= t1] or self.samples[-3:]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(r[1] for r in rows)
        bits = 0
        for r in rows:
            bits |= r[2]
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "hw_power_brake_slowdown": 0x80}
        reasons = [k for k, v in names.items() if bits & v]
        try:
            mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        except Exception:
            mx = None
        return {"sm_mhz": float(sm[len(sm) // 2]), "sm_min_mhz": float(sm[0]), "sm_max_mhz": float(mx) if mx else None,
                "reasons": reasons, "samples": len(rows), "power_w_max": round(max(r[3] for r in rows), 1),
                "source": "nvml, 2 ms polling inside the timed region"}

    def _smi_once(self):
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=clocks.sm,clocks.max.sm",
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
            a, b = [float(x) for x in out.strip().split(",")]
            return {"sm_mhz": a, "sm_max_mhz": b, "reasons": [], "samples": 1, "source": "nvidia-smi after the run"}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source"]}


# ----------------------------------------------------------------------------- helpers
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def time_steps(fn, steps, warmup, torch, dist, world):
    """fn(i) launches step i on the current stream.  Returns (total ms max over ranks, per-step ms list)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall0 = time.time()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for i in range(steps):
        evs[i][0].record()
        fn(warmup + i)
        evs[i][1].record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_wall1 = time.time()
    per = [a.elapsed_time(b) for a, b in evs]
    total = float(sum(per))
    if world > 1:
        t = torch.tensor([total], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    return total, per, (t_wall0, t_wall1)


def gemm_sets(torch, M, N, K, dtype, trans_b, scale_a, scale_b, out_dtype=None, min_bytes=2.5 * L2_BYTES):
    """Enough (A, B, C) sets that a rotation through them exceeds L2 several times over."""
    item = torch.finfo(dtype).bits // 8
    per_set = (M * K + N * K + M * N) * item
    n = max(2, int(math.ceil(min_bytes / per_set)))
    n = min(n, 8)
    sets = []
    for _ in range(n):
        a = (torch.randn(M, K, device="cuda", dtype=torch.float32) * scale_a).to(dtype)
        b = (torch.randn((N, K) if trans_b else (K, N), device="cuda", dtype=torch.float32) * scale_b).to(dtype)
        c = torch.empty(M, N, device="cuda", dtype=out_dtype or dtype)
        sets.append((a, b, c))
    return sets


# ----------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    from frisk_b200 import capi

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = capi.Context(local)
    stream = torch.cuda.current_stream().cuda_stream
    peaks, peak_kind = measured_peaks()

    M = N = K = 4096
    sets = gemm_sets(torch, M, N, K, torch.float16, True, 1.0 / math.sqrt(K), 1.0)
    desc = capi.gemm_desc(M, N, K, "fp16", "fp16", False, True, clear_accum=True)
    flop = 2.0 * M * N * K

    def step(i):
        a, b, c = sets[i % len(sets)]
        ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=stream)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    total_ms, per, wall = time_steps(step, args.steps, args.warmup, torch, dist, world)
    ctx.check(stream)
    clocks = sampler.stop(*wall) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = world * flop * args.steps / (total_ms * 1e-3) / 1e12
    kernel_ms = sum(per) / len(per)
    achieved = flop / (kernel_ms * 1e-3) / 1e12

    # ---- end to end through the host-buffer C-ABI entry (pinned host memory)
    ha = (torch.randn(M, K) / math.sqrt(K)).to(torch.float16).pin_memory()
    hb = torch.randn(N, K).to(torch.float16).pin_memory()
    hc = torch.empty(M, N, dtype=torch.float16).pin_memory()
    e2e_steps = max(1, min(args.steps, 10))
    for _ in range(2):
        ctx.gemm_host(desc, ha.data_ptr(), hb.data_ptr(), hc.data_ptr())
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ctx.gemm_host(desc, ha.data_ptr(), hb.data_ptr(), hc.data_ptr())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = world * flop * e2e_steps / e2e_s / 1e12
    checksum = float(hc[:8, :8].float().abs().sum())

    splitk_res = sharded_res = None
    if world > 1 and not args.no_secondary:
        # the short sharded workloads first: the deep-K products that follow leave the GPUs power-capped
        sharded_res = sharded_secondary(ctx, torch, dist, world, stream, peaks)
        splitk_res = splitk_secondary(ctx, torch, dist, world, rank, peaks)

    out = None
    if rank == 0:
        out = {
            "metric": METRIC, "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
            "data": "synthetic",
            "config": {"workload": "fp16 GEMM M=N=K=4096 per GPU, A row-major, B column-major (NT), "
                                   "fp32 accumulate, fp16 out",
                       "sharding": "independent M-row shards, one 4096x4096x4096 product per GPU, no collective",
                       "kernel": "gemm_tcgen05_2cta (tcgen05.mma cta_group::2 256x256x16 per CTA pair, TMEM accumulators, TMA 6-stage ring, no multicast)",
                       "l2": f"inputs rotate through {len(sets)} operand sets "
                             f"({len(sets) * 3 * M * N * 2 / 2**20:.0f} MiB > 126 MiB L2)",
                       "pct_of_nominal_dense_peak": round(100 * value / world / NOMINAL_TENSOR_TFLOPS, 2)},
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 2,
                    "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps, "checksum": checksum},
            "gpu_launches": args.steps,
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": round(achieved, 2), "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 4),
                         "traffic": ncu_traffic("gemm_tcgen05_f16_4096"), "peak_source": peak_kind + " (burst)",
                         "frac_of_nominal": round(achieved / NOMINAL_TENSOR_TFLOPS, 4)},
        }
        if world == 1:
            out["cpu_baseline"] = cpu_baseline_gemm(M, N, K)
            if not args.no_secondary:
                out["secondary"] = secondary(ctx, torch, stream, peaks, args)
        if splitk_res is not None:
            out["secondary"] = {"gemm_bf16_deepk_splitk": splitk_res}
            out["secondary"].update(sharded_res or {})
        print(json.dumps(out), flush=True)
    ctx.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


def sharded_secondary(ctx, torch, dist, world, stream, peaks):
    """The two workloads that shard without communication, strong-scaled over the ranks: the skinny GEMM
    with N/g columns of W per GPU (X replicated) and the causal attention with 256/g (batch, head) pairs
    per GPU.  Time = max over ranks; throughput = the whole workload over that time."""
    from frisk_b200 import capi
    res = {}
    try:
        M, N, K = 16, 28672, 8192
        n_local = N // world
        sets = gemm_sets(torch, M, n_local, K, torch.bfloat16, True, 1.0, 0.02, min_bytes=2.5 * L2_BYTES)
        desc = capi.gemm_desc(M, n_local, K, "bf16", "bf16", False, True)
        total, _, _ = time_steps(lambda i: ctx.gemm(desc, *(t.data_ptr() for t in sets[i % len(sets)]), stream=stream),
                                 10, 3, torch, dist, world)
        ms = total / 10
        byts = (N * K + world * M * K + M * N) * 2
        res["gemm_bf16_skinny_sharded"] = {"ms": round(ms, 5), "gbs": round(byts / ms / 1e6, 1), "n_gpus": world,
                                           "columns_per_gpu": n_local,
                                           "per_gpu_frac_of_measured_hbm": round(byts / ms / 1e6 / world / peaks["hbm_gbs"], 4)}
        del sets
    except Exception as e:  # noqa: BLE001
        res["gemm_bf16_skinny_sharded"] = {"error": str(e)}
    try:
        B, H, S, D = 8, 32, 4096, 128
        heads = B * H // world
        q, k, v = (torch.randn(1, heads, S, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        o = torch.empty_like(q)
        desc = capi.attn_desc(1, heads, S, S, D, 1.0 / math.sqrt(D), True, "bf16", "bf16")
        total, _, _ = time_steps(lambda i: ctx.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                                             stream=stream), 5, 3, torch, dist, world)
        ms = total / 5
        fl = 4.0 * B * H * S * S * D / 2
        res["attn_bf16_causal_sharded"] = {"ms": round(ms, 5), "tflops": round(fl / ms / 1e9, 2), "n_gpus": world,
                                           "heads_per_gpu": heads,
                                           "per_gpu_frac_of_nominal": round(fl / ms / 1e9 / world / NOMINAL_TENSOR_TFLOPS, 4)}
    except Exception as e:  # noqa: BLE001
        res["attn_bf16_causal_sharded"] = {"error": str(e)}
    return res


def splitk_secondary(ctx, torch, dist, world, rank, peaks):
    """bf16 GEMM M=N=8192, K=131072 with K split across the ranks, two ways: (fused) the tcgen05
    epilogue stores each fp32 tile into its slot in the row owner's memory over NVLink; (nccl) fp32 partials,
    NCCL reduce-scatter pipelined over row panels, local rounding to bf16."""
    from frisk_b200 import splitk
    M, N, K = 8192, 8192, 131072
    res = {"n_gpus": world}

    def line(ms, exchange):
        tf = 2.0 * M * N * K / ms / 1e9
        return {"ms": round(ms, 4), "tflops": round(tf, 2),
                "per_gpu_frac_of_measured_sustained": round(tf / world / peaks["bf16_tflops_sustained"], 4),
                "exchange": exchange}
    sent = (world - 1) / world * M * N * 4 / 1e6
    try:
        k_local = K // world
        a = torch.randn(M, k_local, device="cuda", dtype=torch.bfloat16) * (1 / math.sqrt(K))
        b = torch.randn(N, k_local, device="cuda", dtype=torch.bfloat16)
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}
    try:
        op = splitk.SplitKGemmPush(M, N, K, world, rank, "bf16", ctx, dist.group.WORLD)
        total, per, _ = time_steps(lambda i: op.run(a, b), 5, 3, torch, dist, world)
        ctx.check(torch.cuda.current_stream().cuda_stream)
        res["fused_push"] = line(total / 5, "epilogue 16-byte stores into this rank's slot in the owners' memory, slots summed in rank order, %.1f MB sent per GPU" % sent)
        dist.barrier()
        op.close()
    except Exception as e:  # noqa: BLE001
        res["fused_push"] = {"error": str(e)}
    try:
        plan = splitk.make_plan(M, N, K, world, rank, panels=4)
        op = splitk.SplitKGemm(plan, "bf16", ctx=ctx, group=dist.group.WORLD)
        total, per, _ = time_steps(lambda i: op.run(a, b), 5, 3, torch, dist, world)
        res["nccl"] = line(total / 5, "NCCL reduce_scatter of fp32 partials over %d row panels, %.1f MB sent per GPU"
                           % (plan.panels, sent))
    except Exception as e:  # noqa: BLE001
        res["nccl"] = {"error": str(e)}
    return res


def secondary(ctx, torch, stream, peaks, args):
    """The other benchmark workloads, kernel-only, a few steps each."""
    from frisk_b200 import capi
    res = {}
    steps, warm = max(3, min(args.steps, 10)), 3

    def timed(fn):
        total, per, _ = time_steps(fn, steps, warm, torch, None, 1)
        ctx.check(stream)
        return total / steps

    # fp32 GEMM 1024^3 (12 MiB of operands: rotate 32 sets to stay ahead of L2)
    try:
        M = 1024
        sets = gemm_sets(torch, M, M, M, torch.float32, False, 1.0, 1.0, min_bytes=3 * L2_BYTES)
        sets = sets + gemm_sets(torch, M, M, M, torch.float32, False, 1.0, 1.0, min_bytes=3 * L2_BYTES)
        desc = capi.gemm_desc(M, M, M, "fp32", "fp32")
        ms = timed(lambda i: ctx.gemm(desc, *(t.data_ptr() for t in sets[i % len(sets)]), stream=stream))
        res["gemm_f32_1024"] = {"ms": round(ms, 5), "tflops": round(2.0 * M ** 3 / ms / 1e9, 2)}
    except Exception as e:  # noqa: BLE001
        res["gemm_f32_1024"] = {"error": str(e)}
    # skinny bf16 16 x 28672 x 8192 (470 MB of weights: larger than L2 by itself)
    try:
        M, N, K = 16, 28672, 8192
        sets = gemm_sets(torch, M, N, K, torch.bfloat16, True, 1.0, 0.02, min_bytes=1)
        desc = capi.gemm_desc(M, N, K, "bf16", "bf16", False, True)
        ms = timed(lambda i: ctx.gemm(desc, *(t.data_ptr() for t in sets[i % len(sets)]), stream=stream))
        byts = (N * K + M * K + M * N) * 2
        res["gemm_bf16_skinny"] = {"ms": round(ms, 5), "gbs": round(byts / ms / 1e6, 1),
                                   "frac_of_measured_hbm": round(byts / ms / 1e6 / peaks["hbm_gbs"], 4),
                                   "frac_of_nominal_hbm": round(byts / ms / 1e6 / NOMINAL_HBM_GBS, 4)}
    except Exception as e:  # noqa: BLE001
        res["gemm_bf16_skinny"] = {"error": str(e)}
    # causal attention B=8 H=32 S=4096 D=128 bf16
    try:
        B, H, S, D = 8, 32, 4096, 128
        q, k, v = (torch.randn(B, H, S, D, device="cuda", dtype=torch.bfloat16) for _ in range(3))
        o = torch.empty_like(q)
        desc = capi.attn_desc(B, H, S, S, D, 1.0 / math.sqrt(D), True, "bf16", "bf16")
        ms = timed(lambda i: ctx.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                                               stream=stream))
        fl = 4.0 * B * H * S * S * D / 2
        res["attn_bf16_causal"] = {"ms": round(ms, 5), "tflops": round(fl / ms / 1e9, 2),
                                   "frac_of_nominal": round(fl / ms / 1e9 / NOMINAL_TENSOR_TFLOPS, 4)}
        del q, k, v, o
    except Exception as e:  # noqa: BLE001
        res["attn_bf16_causal"] = {"error": str(e)}
    # deep-K bf16 8192 x 8192 x 131072 (single GPU: whole K)
    try:
        M, N, K = 8192, 8192, 131072
        a = (torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * (1 / math.sqrt(K)))
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        c = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        desc = capi.gemm_desc(M, N, K, "bf16", "bf16", False, True)
        total, per, _ = time_steps(lambda i: ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=stream),
                                   3, 1, torch, None, 1)
        ctx.check(stream)
        ms = total / 3
        res["gemm_bf16_deepk"] = {"ms": round(ms, 4), "tflops": round(2.0 * M * N * K / ms / 1e9, 2),
                                  "frac_of_measured_sustained": round(2.0 * M * N * K / ms / 1e9 /
                                                                      peaks["bf16_tflops_sustained"], 4)}
        del a, b, c
    except Exception as e:  # noqa: BLE001
        res["gemm_bf16_deepk"] = {"error": str(e)}
    return res


# ----------------------------------------------------------------------------- CPU arm
def cpu_gemm_sample(M, N, K, rows, seed=1):
    """fp32 BLAS product of `rows` rows of the rounded fp16 operands on all host threads."""
    import numpy as np

    from oracle import gemm_oracle
    rng = np.random.default_rng(seed)
    a = (rng.standard_normal((rows, K), dtype=np.float32) / np.float32(math.sqrt(K))).astype(np.float16)
    b = rng.standard_normal((N, K), dtype=np.float32).astype(np.float16)
    gemm_oracle.gemm_f32_blas(a[:8], b, "fp16", False, True)  # warm the BLAS threads
    t0 = time.perf_counter()
    c = gemm_oracle.gemm_f32_blas(a, b, "fp16", False, True)
    dt = time.perf_counter() - t0
    return dt, float(c[0, 0])


def cpu_baseline_gemm(M, N, K, budget_s=12.0):
    cores = os.cpu_count() or 1
    dt, _ = cpu_gemm_sample(M, N, K, 256)
    rate = 2.0 * 256 * N * K / dt
    rows = int(min(M, max(256, budget_s * rate / (2.0 * N * K))))
    rows = max(256, rows // 256 * 256)
    dt, _ = cpu_gemm_sample(M, N, K, rows)
    return {"value": round(2.0 * rows * N * K / dt / 1e12, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
            "sample": f"{rows} of {M} rows of the 4096^3 fp16 GEMM, numpy fp32 BLAS over the rounded inputs, "
                      f"conversion included, {dt:.2f} s"}


def run_reference(args):
    """The reference's CPU path for this op is its numpy oracle style (the reference has no
    executed GEMM, so the oracle port stands in): timed on the host cores."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    M = N = K = 4096
    cores = os.cpu_count() or 1
    dt, _ = cpu_gemm_sample(M, N, K, 256)
    rate = 2.0 * 256 * N * K / dt
    total_steps = args.steps + args.warmup
    rows = int(min(M, max(256, (120.0 / max(1, total_steps)) * rate / (2.0 * N * K))))
    rows = max(256, rows // 256 * 256)
    for _ in range(args.warmup):
        cpu_gemm_sample(M, N, K, rows)
    times = [cpu_gemm_sample(M, N, K, rows)[0] for _ in range(args.steps)]
    total = sum(times)
    value = 2.0 * rows * N * K * args.steps / total / 1e12
    sample = f"each step = {rows} of {M} rows of the 4096^3 fp16 GEMM (numpy fp32 BLAS, all host threads)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(1e3 * total / args.steps * (M / rows), 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": "fp16 GEMM M=N=K=4096, A row-major, B column-major (NT), fp32 accumulate",
                   "note": "CPU oracle port on the host cores; ms_per_step is scaled to the full 4096 rows"},
        "cpu_baseline": {"value": round(value, 4), "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-secondary", action="store_true", help="skip the informational extra workloads")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

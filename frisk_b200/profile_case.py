"""Launch one hot-path kernel a few times on a profiling-sized case.

    python -m frisk_b200.profile_case --kernel tcgen05|skinny|simt|attention [--launches 4]

Meant to be run under a profiler (one kernel, a few launches, a few hundred MB on the
device, operands larger than the 126 MB L2 where the kernel is memory-bound) and also
prints the CUDA-event time of each launch when run plainly.
"""
import argparse
import math

import torch

from frisk_b200 import capi


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", required=True, choices=["tcgen05", "skinny", "simt", "attention"])
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--m", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--heads", type=int, default=64)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    ctx = capi.Context(0)
    stream = torch.cuda.current_stream().cuda_stream
    dev = "cuda"
    if args.kernel == "tcgen05":
        M, N, K = args.m or 8192, args.n or 4096, args.k or 4096
        a = (torch.randn(M, K, device=dev) / math.sqrt(K)).half()
        b = torch.randn(N, K, device=dev).half()
        c = torch.empty(M, N, device=dev, dtype=torch.float16)
        desc = capi.gemm_desc(M, N, K, "fp16", "fp16", False, True)
        work, unit = 2.0 * M * N * K / 1e12, "TFLOP"
        fn = lambda: ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=stream)  # noqa: E731
    elif args.kernel == "skinny":
        M, N, K = args.m or 16, args.n or 28672, args.k or 8192
        a = torch.randn(M, K, device=dev).bfloat16()
        b = (torch.randn(N, K, device=dev) * 0.02).bfloat16()
        c = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        desc = capi.gemm_desc(M, N, K, "bf16", "bf16", False, True)
        work, unit = (N * K + M * K + M * N) * 2 / 1e9, "GB"
        fn = lambda: ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=stream)  # noqa: E731
    elif args.kernel == "simt":
        M, N, K = args.m or 1024, args.n or 1024, args.k or 1024
        a = torch.rand(M, K, device=dev) * 2 - 1
        b = torch.rand(K, N, device=dev) * 2 - 1
        c = torch.empty(M, N, device=dev)
        desc = capi.gemm_desc(M, N, K, "fp32", "fp32")
        work, unit = 2.0 * M * N * K / 1e12, "TFLOP"
        fn = lambda: ctx.gemm(desc, a.data_ptr(), b.data_ptr(), c.data_ptr(), stream=stream)  # noqa: E731
    else:
        B, H, S, D = 1, args.heads, args.m or 4096, 128
        q, k, v = (torch.randn(B, H, S, D, device=dev).bfloat16() for _ in range(3))
        o = torch.empty_like(q)
        desc = capi.attn_desc(B, H, S, S, D, 1 / math.sqrt(D), True, "bf16")
        work, unit = 4.0 * B * H * S * S * D / 2 / 1e12, "TFLOP"
        fn = lambda: ctx.attention_fwd(desc, q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),  # noqa: E731
                                       stream=stream)
    times = []
    for _ in range(args.launches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ctx.check(stream)
    for t in times:
        print(f"{args.kernel}: {t * 1e3:.1f} us  {work / (t * 1e-3):.1f} {unit}/s")
    ctx.close()


if __name__ == "__main__":
    main()

"""Runs one operator a few times on one GPU with seeded synthetic operands: the small, bounded
case to put under a profiler (``ncu -k regex:fused_gemm_kernel ... python -m
mkernel_b200.profile_case --op ag --m 4096 --n 3584 --k 8192``) or to time by hand.

World size is 1 here (the exchange step is empty); multi-GPU timing is bench.py's job.
"""
from __future__ import annotations

import argparse

import torch

import mkernel_b200
from mkernel_b200 import _lib, ops


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=["gemm", "ag", "rs", "ar"], default="ag")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=3584)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--cta-pair", type=int, default=1)
    args = ap.parse_args()
    M, N, K = args.m, args.n, args.k
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(1)
    A = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
    B_nk = (torch.randn((N, K), device=dev, generator=g) * K ** -0.5).to(torch.bfloat16)
    _lib.set_option("block_n", args.block_n)
    _lib.set_option("cta_pair", args.cta_pair)

    if args.op == "gemm":
        C = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        run = lambda i: ops.gemm_bf16(A, B_nk, C)
    elif args.op == "ag":
        mod = mkernel_b200.load("ag_gemm_warp_specialized")
        Ab = mod.DistBuffer((1, M, K), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
        Ab.data_[0].copy_(A)
        ready = mod.DistBuffer((mod.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                               local_rank=0, local_world_size=1)
        ready.data_.zero_()
        C = torch.empty((1, M, N), device=dev, dtype=torch.bfloat16)

        def run(i):
            mod.ag_gemm_warp_specialized_prepare(ready, M, N)
            mod.ag_gemm_warp_specialized_launch(Ab, ready, B_nk, C)
    elif args.op == "rs":
        mod = mkernel_b200.load("gemm_rs_blackwell")
        Cb = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
        sync = mod.DistBuffer(mod.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=0,
                              local_world_size=1)
        mod.gemm_rs_blackwell_prepare(A, B_nk, Cb, sync)
        run = lambda i: mod.gemm_rs_blackwell_launch(A, B_nk, Cb, sync)
    else:
        mod = mkernel_b200.load("gemm_ar_blackwell")
        B_kn = B_nk.t().contiguous()
        Cb = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
        Cf = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
        bar = mod.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=0, local_world_size=1)
        bar.data_.zero_()
        run = lambda i: mod.gemm_ar_intranode_blackwell(A, B_kn, Cb, bar, Cf, i + 1)

    for i in range(args.warmup):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.iters):
        run(args.warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.iters
    print(f"op={args.op} M={M} N={N} K={K}: {ms:.4f} ms/iter, {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")


if __name__ == "__main__":
    main()

"""Generates the fixtures in this directory.  Run once, in a container that has the reference
tree mounted; the tests only read the generated files.

    python tests/golden/make_golden.py <path to a checkout of uccl-project/mKernel>

1. check_close_cases.json -- verdicts of the REFERENCE's own acceptance function
   (bench/common.py:312-367, imported from the reference tree and run unmodified in a
   single-process gloo group; the only shim is that the 5-number statistics tensor it creates
   with device="cuda" is created on the CPU, since this container has no GPU).
2. torch_path_w2.npz -- outputs of the reference's torch path (torch.matmul +
   torch.distributed all_gather / reduce_scatter / all_reduce, bench/ag_gemm_bench.py:567-568,
   bench/gemm_rs_bench.py:408-410, bench/gemm_ar_blackwell_bench.py:423-425) run as two gloo
   ranks on seeded bf16 inputs, plus the plumbing case (fp32, 256x256 @ 256x512, all_reduce).
   Outputs are stored subsampled (every 8th row and column) with their full-tensor sums.
"""
from __future__ import annotations

import io
import json
import os
import sys
import contextlib
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle.tp_gemm_oracle import synth_inputs  # noqa: E402

SMALL = dict(M=256, N=192, K=128)   # per-rank K for rs/ar; total K for ag


def make_pair(seed: int, rows: int, cols: int, noise: float, outliers: int, outlier_mag: float):
    g = torch.Generator().manual_seed(seed)
    expected = torch.randn((rows, cols), generator=g)
    observed = expected + noise * torch.randn((rows, cols), generator=g)
    if outliers:
        idx = torch.randint(0, rows * cols, (outliers,), generator=g)
        observed.view(-1)[idx] += outlier_mag
    return observed.to(torch.bfloat16), expected


def gen_check_close(ref_root: Path):
    sys.path.insert(0, str(ref_root / "bench"))
    import common as ref_common  # the reference's bench/common.py

    real_tensor = torch.tensor

    def cpu_tensor(*a, **k):
        if k.get("device") == "cuda":
            k["device"] = "cpu"
        return real_tensor(*a, **k)

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29641")
    dist.init_process_group("gloo", rank=0, world_size=1)
    cases = []
    grid = [
        (0.0, 0, 0.0), (0.004, 0, 0.0), (0.05, 0, 0.0), (0.2, 0, 0.0), (0.5, 0, 0.0),
        (0.004, 3, 1.0), (0.004, 3, 40.0), (0.03, 50, 2.0), (1.5, 0, 0.0), (0.004, 2000, 3.0),
    ]
    seed = 100
    for noise, outliers, mag in grid:
        for atol, rtol in ((0.35, 0.08), (0.55, 0.12), (0.01, 0.001)):
            seed += 1
            obs, exp = make_pair(seed, 96, 80, noise, outliers, mag)
            torch.tensor = cpu_tensor
            try:
                with contextlib.redirect_stdout(io.StringIO()):
                    ok = ref_common.check_close("golden", obs, exp, atol=atol, rtol=rtol)
            finally:
                torch.tensor = real_tensor
            cases.append(dict(seed=seed, rows=96, cols=80, noise=noise, outliers=outliers,
                              outlier_mag=mag, atol=atol, rtol=rtol, ok=bool(ok)))
    dist.destroy_process_group()
    (HERE / "check_close_cases.json").write_text(json.dumps(cases, indent=1))
    print(f"check_close_cases.json: {len(cases)} cases, {sum(c['ok'] for c in cases)} pass")


def _torch_path_rank(rank: int, world: int, port: int, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, N, K = SMALL["M"], SMALL["N"], SMALL["K"]
    out = {}
    # AllGather + GEMM (seed 1 + rank)
    a, b = synth_inputs("ag", rank, world, M, N, K, seed=1)
    a_full = torch.empty((M, K), dtype=torch.bfloat16)
    dist.all_gather_into_tensor(a_full, a)
    out["ag_c"] = torch.mm(a_full.float(), b.float())
    out["ag_a_full"] = a_full.float()
    # GEMM + ReduceScatter (seed 2 + rank); reference computes a @ b_nk.T
    a, b = synth_inputs("rs", rank, world, M, N, K, seed=2)
    c = torch.mm(a.float(), b.t().contiguous().float().t())
    rs = torch.empty((M // world, N), dtype=torch.float32)
    dist.reduce_scatter_tensor(rs, c)
    out["rs_out"] = rs
    # GEMM + AllReduce (seed 3 + rank)
    a, b = synth_inputs("ar", rank, world, M, N, K, seed=3)
    c = torch.matmul(a.float(), b.float())
    out["ar_partial"] = c.clone()
    dist.all_reduce(c, op=dist.ReduceOp.SUM)
    out["ar_out"] = c
    # the plumbing case: fp32, A_r [256,256], B_r [256,512], A~N(0,1), B~N(0,1/256), seed 0 + r
    g = torch.Generator().manual_seed(0 + rank)
    a1 = torch.randn((256, 256), generator=g)
    b1 = torch.randn((256, 512), generator=g) * (1.0 / 16.0)
    c1 = a1 @ b1
    dist.all_reduce(c1, op=dist.ReduceOp.SUM)
    out["cfg1_out"] = c1
    q.put((rank, {k: v.numpy() for k, v in out.items()}))
    dist.barrier()
    dist.destroy_process_group()


def gen_torch_path():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_torch_path_rank, args=(r, world, 29643, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get() for _ in range(world))
    for p in procs:
        p.join()
    store = {}
    for r in range(world):
        for k, v in got[r].items():
            store[f"r{r}_{k}_sub"] = v[::8, ::8].astype(np.float32)
            store[f"r{r}_{k}_sum"] = np.array(v.astype(np.float64).sum())
    np.savez_compressed(HERE / "torch_path_w2.npz", **store)
    print(f"torch_path_w2.npz: {len(store)} arrays")


if __name__ == "__main__":
    ref_root = Path(sys.argv[1] if len(sys.argv) > 1 else
                    Path(__file__).resolve().parents[3] / "reference")
    gen_torch_path()
    gen_check_close(ref_root)

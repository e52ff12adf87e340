"""The multi-rank semantics of the path on CPU ranks (gloo, world size 2): the reference's own
torch path -- torch.matmul + all_gather / reduce_scatter / all_reduce -- must agree with the
oracle's single-process restatement, including the plumbing case (fp32, 256x256 @ 256x512,
all_reduce over 2 ranks)."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import tp_gemm_oracle as orc


def _rank(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    out = {}
    # the plumbing case: fp32 operands, two ranks
    g = torch.Generator().manual_seed(0 + rank)
    a = torch.randn((256, 256), generator=g)
    b = torch.randn((256, 512), generator=g) / 16.0
    c = a @ b
    dist.all_reduce(c)
    out["cfg1"] = c
    # the three operators on bf16 inputs
    M, N, K = 128, 96, 64
    a, b = orc.synth_inputs("ag", rank, world, M, N, K, seed=1)
    a_full = torch.empty((M, K), dtype=torch.bfloat16)
    dist.all_gather_into_tensor(a_full, a)
    out["ag"] = a_full.float() @ b.float()
    out["ag_a"] = a_full
    a, b = orc.synth_inputs("rs", rank, world, M, N, K, seed=2)
    full = a.float() @ b.float()
    rs = torch.empty((M // world, N))
    dist.reduce_scatter_tensor(rs, full)
    out["rs"] = rs
    a, b = orc.synth_inputs("ar", rank, world, M, N, K, seed=3)
    ar = a.float() @ b.float()
    dist.all_reduce(ar)
    out["ar"] = ar
    # Tensors travel by value (raw bytes), not as shared-memory handles: a handle is only valid
    # while this process lives, and the parent may read the queue after it has exited.
    q.put((rank, {k: (str(v.dtype), tuple(v.shape), v.contiguous().view(torch.uint8).numpy().tobytes())
                  for k, v in out.items()}))
    dist.barrier()
    dist.destroy_process_group()


def test_gloo_ranks_match_oracle():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    from tests.conftest import free_port
    port = free_port()
    procs = [ctx.Process(target=_rank, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        rank, packed = q.get(timeout=180)
        got[rank] = {k: torch.frombuffer(bytearray(raw), dtype=torch.uint8)
                     .view(getattr(torch, dt.split(".")[1])).view(shape)
                     for k, (dt, shape, raw) in packed.items()}
    for p in procs:
        p.join(60)
    # config 1 against an fp64 evaluation
    parts = []
    for r in range(world):
        g = torch.Generator().manual_seed(0 + r)
        a = torch.randn((256, 256), generator=g)
        b = torch.randn((256, 512), generator=g) / 16.0
        parts.append(a.double() @ b.double())
    ref = parts[0] + parts[1]
    for r in range(world):
        assert (got[r]["cfg1"].double() - ref).abs().max() < 5e-5
    M, N, K = 128, 96, 64
    ag = [orc.synth_inputs("ag", r, world, M, N, K, seed=1) for r in range(world)]
    rs = [orc.synth_inputs("rs", r, world, M, N, K, seed=2) for r in range(world)]
    ar = [orc.synth_inputs("ar", r, world, M, N, K, seed=3) for r in range(world)]
    rs_ref = orc.gemm_rs_ref([a for a, _ in rs], [b for _, b in rs])
    ar_ref, _ = orc.gemm_ar_ref([a for a, _ in ar], [b for _, b in ar])
    for r in range(world):
        a_full, c = orc.ag_gemm_ref([a for a, _ in ag], ag[r][1])
        assert torch.equal(got[r]["ag_a"], a_full)
        assert orc.rel_error(got[r]["ag"], c) < 1e-5
        assert orc.rel_error(got[r]["rs"], rs_ref[r]) < 1e-5
        assert orc.rel_error(got[r]["ar"], ar_ref) < 1e-5

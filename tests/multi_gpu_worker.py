"""One rank of a multi-GPU parity run (spawned by test_multi_gpu.py, also usable by hand:
``python -m torch.distributed.run --nproc-per-node 2 tests/multi_gpu_worker.py``).

Every rank regenerates all ranks' seeded inputs on the CPU, computes the oracle result for the
rows it checks, runs the fused operator through the reference-shaped API and returns the error
figures.  Host coordination uses a gloo group; the operators use only their own transport.
"""
from __future__ import annotations

import json
import os
import sys
import traceback
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import mkernel_b200  # noqa: E402
from mkernel_b200 import _lib  # noqa: E402
from oracle import tp_gemm_oracle as orc  # noqa: E402


def _sample_rows(n_rows: int, max_rows: int, seed: int) -> torch.Tensor:
    if n_rows <= max_rows:
        return torch.arange(n_rows)
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(n_rows, generator=g)[:max_rows].sort().values


def sync_all():
    torch.cuda.synchronize()
    dist.barrier()


def identical_on_all_ranks(t: torch.Tensor) -> bool:
    """True when every rank holds the same BITS in `t` (the reference's cross-rank identity
    check, bench/common.py:469-500): the raw bytes are gathered and compared."""
    mine = t.detach().contiguous().view(torch.uint8).cpu()
    world = dist.get_world_size()
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    return all(torch.equal(gathered[0], g) for g in gathered[1:])


def case_ag(rank, world, M, N, K, seed, iters, max_rows, multicast=False):
    mod = mkernel_b200.load("ag_gemm_warp_specialized")
    dev = torch.device("cuda", rank)
    Ms = M // world
    shards = [orc.synth_inputs("ag", r, world, M, N, K, seed=seed)[0] for r in range(world)]
    b_kn = orc.synth_inputs("ag", rank, world, M, N, K, seed=seed)[1]
    A = mod.DistBuffer((world, Ms, K), dtype=torch.bfloat16, local_rank=rank,
                       local_world_size=world, multicast=multicast)
    A.data_.zero_()
    A.data_[rank].copy_(shards[rank])
    ready = mod.DistBuffer((mod.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                           local_rank=rank, local_world_size=world, multicast=multicast)
    ready.data_.zero_()
    B = b_kn.t().contiguous().to(dev)
    C = torch.zeros((world, Ms, N), device=dev, dtype=torch.bfloat16)
    sync_all()
    rows = _sample_rows(M, max_rows, seed)
    a_full = torch.cat(shards, 0)
    ref = a_full[rows].float() @ b_kn.float()
    res = dict(op="ag", M=M, N=N, K=K, rel=[], gathered_exact=[], status=[], rerun_identical=[])
    previous = None
    for it in range(iters):
        C.zero_()
        if it > 0:  # poison the remote slabs so a stale gather would be noticed
            for r in range(world):
                if r != rank:
                    A.data_[r].zero_()
            sync_all()
        mod.ag_gemm_warp_specialized_prepare(ready, M, N)
        mod.ag_gemm_warp_specialized_launch(A, ready, B, C)
        torch.cuda.synchronize()
        res["status"].append(list(mod.op_status(ready)) if True else None)
        res["gathered_exact"].append(bool(torch.equal(A.data_.view(M, K).cpu(), a_full)))
        res["rel"].append(orc.rel_error(C.view(M, N)[rows.to(dev)].cpu(), ref))
        # a re-run on the same inputs reproduces the output bit for bit (bench/common.py:503-531)
        if previous is not None:
            res["rerun_identical"].append(bool(torch.equal(previous, C)))
        previous = C.clone()
        dist.barrier()
    sync_all()
    return res


def case_rs(rank, world, M, N, K, seed, iters, max_rows, multicast=False):
    mod = mkernel_b200.load("gemm_rs_blackwell")
    dev = torch.device("cuda", rank)
    Ms = M // world
    rows = _sample_rows(Ms, max_rows, seed)
    ref = None
    mine = None
    scale = None
    for r in range(world):
        a, b = orc.synth_inputs("rs", r, world, M, N, K, seed=seed)
        p = a[rank * Ms + rows].float() @ b.float()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
        if r == rank:
            mine = (a, b)
    A = mine[0].to(dev)
    B = mine[1].t().contiguous().to(dev)
    C = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world,
                       multicast=multicast)
    sync = mod.DistBuffer(mod.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=rank,
                          local_world_size=world, multicast=False)
    mod.gemm_rs_blackwell_prepare(A, B, C, sync)
    sync_all()
    res = dict(op="rs", M=M, N=N, K=K, rel=[], rel_plain=[], status=[])
    sign = 1.0
    for it in range(iters):
        if it > 0:      # back-to-back launches without host barriers; A negated in between
            A.neg_()
            sign = -sign
        mod.gemm_rs_blackwell_launch(A, B, C, sync)
        torch.cuda.synchronize()
        out = C.data_.narrow(0, rank * Ms, Ms)
        res["rel"].append(orc.rel_error(out[rows.to(dev)].cpu(), sign * ref, scale))
        res["rel_plain"].append(orc.rel_error(out[rows.to(dev)].cpu(), sign * ref))
        res["status"].append(list(mod.op_status(sync)))
        dist.barrier()   # the reduced slice is read above before any rank launches again
    sync_all()
    return res


def case_ar(rank, world, M, N, K, seed, iters, max_rows, layout=_lib.MK_B_KN, multicast=False):
    mod = mkernel_b200.load("gemm_ar_blackwell")
    dev = torch.device("cuda", rank)
    rows = _sample_rows(M, max_rows, seed)
    ref = None
    mine = None
    scale = None
    for r in range(world):
        a, b = orc.synth_inputs("ar", r, world, M, N, K, seed=seed)
        p = a[rows].float() @ b.float()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
        if r == rank:
            mine, mine_partial = (a, b), p
    A = mine[0].to(dev)
    B = (mine[1] if layout == _lib.MK_B_KN else mine[1].t()).contiguous().to(dev)
    C = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world,
                       multicast=multicast)
    Cf = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world,
                        multicast=multicast)
    barrier = mod.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=rank,
                             local_world_size=world, multicast=multicast)
    barrier.data_.zero_()
    C.data_.zero_()
    Cf.data_.zero_()
    sync_all()
    res = dict(op="ar", M=M, N=N, K=K, layout=layout, rel=[], rel_plain=[], rel_partial=[],
               status=[], identical_across_ranks=[])
    for it in range(iters):
        mod.gemm_ar_intranode_blackwell(A, B, C, barrier, Cf, it + 1, layout)
        torch.cuda.synchronize()
        res["rel"].append(orc.rel_error(Cf.data_[rows.to(dev)].cpu(), ref, scale))
        res["rel_plain"].append(orc.rel_error(Cf.data_[rows.to(dev)].cpu(), ref))
        res["rel_partial"].append(orc.rel_error(C.data_[rows.to(dev)].cpu(), mine_partial))
        res["status"].append(list(mod.op_status(barrier)))
        # every rank must hold bit-identical output (bench/common.py:469-500)
        res["identical_across_ranks"].append(identical_on_all_ranks(Cf.data_))
        Cf.data_.zero_()
        sync_all()
    return res


def case_compat(rank, world, M, N, K, seed, iters, max_rows):
    """The multi-node style signatures (ag_gemm_multinode / gemm_rs_fused / gemm_ar_multinode)
    served on one node: B is [K, N] and the epoch comes from the caller."""
    dev = torch.device("cuda", rank)
    res = dict(op="compat", M=M, N=N, K=K, rel=[], status=[], gathered_exact=[])
    rows = _sample_rows(M, max_rows, seed)
    # --- AllGather + GEMM
    ag = mkernel_b200.load("ag_gemm")
    Ms = M // world
    shards = [orc.synth_inputs("ag", r, world, M, N, K, seed=seed)[0] for r in range(world)]
    b_kn = orc.synth_inputs("ag", rank, world, M, N, K, seed=seed)[1]
    A = ag.DistBuffer((M, K), dtype=torch.bfloat16, local_rank=rank, local_world_size=world,
                      multicast=True)
    A.data_.zero_()
    A.data_[rank * Ms:(rank + 1) * Ms].copy_(shards[rank])
    barrier = ag.DistBuffer((3, 1024, 1024), dtype=torch.int32, local_rank=rank,
                            local_world_size=world, multicast=True)
    barrier.data_.zero_()
    B = b_kn.contiguous().to(dev)
    C = torch.zeros((M, N), device=dev, dtype=torch.bfloat16)
    ag.create_session(0, "127.0.0.1", 0, 0, 0, 0, 0, 0, rank)
    fifo = ag.get_fifo_handles()
    sync_all()
    a_full = torch.cat(shards, 0)
    ref = a_full[rows].float() @ b_kn.float()
    for it in range(iters):
        ag.ag_gemm_multinode(A, B, C, barrier, ag.get_recv_buf_ptr(), *fifo,
                             ag.get_arrival_flags_ptr(), it + 1, 0, 8, Ms * K * 2, None, 148, 0, 1)
        torch.cuda.synchronize()
        res["status"].append(list(ag.op_status(barrier)))
        res["gathered_exact"].append(bool(torch.equal(A.data_.cpu(), a_full)))
        res["rel"].append(orc.rel_error(C[rows.to(dev)].cpu(), ref))
        sync_all()
    # --- GEMM + ReduceScatter
    rs = mkernel_b200.load("gemm_rs")
    rrows = _sample_rows(Ms, max_rows, seed)
    ref = scale = mine = None
    for r in range(world):
        a, b = orc.synth_inputs("rs", r, world, M, N, K, seed=seed + 1)
        p = a[rank * Ms + rrows].float() @ b.float()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
        if r == rank:
            mine = (a, b)
    A2, B2 = mine[0].to(dev), mine[1].contiguous().to(dev)
    work = rs.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    out = rs.DistBuffer((Ms, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    bar2 = rs.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=rank, local_world_size=world)
    bar2.data_.zero_()
    sync_all()
    for it in range(iters):
        rs.gemm_rs_fused(A2, B2, work, out, bar2, None, 0, 0, 0, 0, 0, 0, 0, 0, it + 1, 0, 100, 8,
                         8, 8, False, 0, None, None, 1)
        torch.cuda.synchronize()
        res["status"].append(list(rs.op_status(bar2)))
        res["rel"].append(orc.rel_error(out.data_[rrows.to(dev)].cpu(), ref, scale))
        sync_all()
    # --- GEMM + AllReduce
    ar = mkernel_b200.load("gemm_ar")
    ref = scale = mine = None
    for r in range(world):
        a, b = orc.synth_inputs("ar", r, world, M, N, K, seed=seed + 2)
        p = a[rows].float() @ b.float()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
        if r == rank:
            mine = (a, b)
    A3, B3 = mine[0].to(dev), mine[1].contiguous().to(dev)
    C3 = ar.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    C3f = ar.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    bar3 = ar.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=rank, local_world_size=world)
    bar3.data_.zero_()
    sync_all()
    for it in range(iters):
        ar.gemm_ar_multinode(A3, B3, C3, bar3, C3f, 0, 0, 0, 0, 0, 0, 0, 0, it + 1, 0, 8, 0, 0, 1,
                             use_acquire_poll=False)
        torch.cuda.synchronize()
        res["status"].append(list(ar.op_status(bar3)))
        res["rel"].append(orc.rel_error(C3f.data_[rows.to(dev)].cpu(), ref, scale))
        sync_all()
    return res


def _capture(fn):
    """Capture one call of fn in a CUDA graph (after a warm-up call on a side stream)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    sync_all()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        fn()
    sync_all()
    return g


def case_graph(rank, world, M, N, K, seed, replays, max_rows):
    """CUDA-graph replays at world size > 1, each replay checked: AllGather+GEMM with C zeroed
    and the gathered slabs poisoned between replays (bench/ag_gemm_bench.py:886-904),
    GEMM+ReduceScatter with A negated between replays and no prepare in between
    (bench/gemm_rs_bench.py:226-242), GEMM+AllReduce with the epoch kept on the device."""
    dev = torch.device("cuda", rank)
    res = dict(op="graph", M=M, N=N, K=K, rel=[], status=[], gathered_exact=[],
               identical_across_ranks=[])
    Ms = M // world
    rows = _sample_rows(M, max_rows, seed)
    # ---- AllGather + GEMM
    ag = mkernel_b200.load("ag_gemm_warp_specialized")
    shards = [orc.synth_inputs("ag", r, world, M, N, K, seed=seed)[0] for r in range(world)]
    b_kn = orc.synth_inputs("ag", rank, world, M, N, K, seed=seed)[1]
    A = ag.DistBuffer((world, Ms, K), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    A.data_.zero_()
    A.data_[rank].copy_(shards[rank])
    ready = ag.DistBuffer((ag.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                          local_rank=rank, local_world_size=world)
    ready.data_.zero_()
    B = b_kn.t().contiguous().to(dev)
    C = torch.zeros((world, Ms, N), device=dev, dtype=torch.bfloat16)
    sync_all()

    def ag_call():
        ag.ag_gemm_warp_specialized_prepare(ready, M, N)
        ag.ag_gemm_warp_specialized_launch(A, ready, B, C)

    g = _capture(ag_call)
    a_full = torch.cat(shards, 0)
    ref = a_full[rows].float() @ b_kn.float()
    for _ in range(replays):
        C.zero_()
        for r in range(world):
            if r != rank:
                A.data_[r].zero_()
        sync_all()
        g.replay()
        torch.cuda.synchronize()
        res["status"].append(list(ag.op_status(ready)))
        res["gathered_exact"].append(bool(torch.equal(A.data_.view(M, K).cpu(), a_full)))
        res["rel"].append(orc.rel_error(C.view(M, N)[rows.to(dev)].cpu(), ref))
        sync_all()
    del g
    # ---- GEMM + ReduceScatter
    rs = mkernel_b200.load("gemm_rs_blackwell")
    rrows = _sample_rows(Ms, max_rows, seed)
    ref = scale = mine = None
    for r in range(world):
        a, b = orc.synth_inputs("rs", r, world, M, N, K, seed=seed + 1)
        p = a[rank * Ms + rrows].float() @ b.float()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
        if r == rank:
            mine = (a, b)
    A2, B2 = mine[0].to(dev), mine[1].t().contiguous().to(dev)
    C2 = rs.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    sync2 = rs.DistBuffer(rs.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=rank,
                          local_world_size=world)
    rs.gemm_rs_blackwell_prepare(A2, B2, C2, sync2)
    sync_all()
    g = _capture(lambda: rs.gemm_rs_blackwell_launch(A2, B2, C2, sync2))
    sign = 1.0
    for _ in range(replays):
        A2.neg_()
        sign = -sign
        sync_all()
        g.replay()
        torch.cuda.synchronize()
        out = C2.data_.narrow(0, rank * Ms, Ms)
        res["status"].append(list(rs.op_status(sync2)))
        res["rel"].append(orc.rel_error(out[rrows.to(dev)].cpu(), sign * ref, scale))
        sync_all()
    del g
    # ---- GEMM + AllReduce (device-resident epoch)
    ar = mkernel_b200.load("gemm_ar_blackwell")
    ref = scale = mine = None
    for r in range(world):
        a, b = orc.synth_inputs("ar", r, world, M, N, K, seed=seed + 2)
        p = a[rows].float() @ b.float()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
        if r == rank:
            mine = (a, b)
    A3, B3 = mine[0].to(dev), mine[1].contiguous().to(dev)
    C3 = ar.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    C3f = ar.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=rank, local_world_size=world)
    bar3 = ar.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=rank, local_world_size=world)
    bar3.data_.zero_()
    sync_all()
    g = _capture(lambda: ar.gemm_ar_intranode_blackwell(A3, B3, C3, bar3, C3f, 0))
    for _ in range(replays):
        C3f.data_.zero_()
        sync_all()
        g.replay()
        torch.cuda.synchronize()
        res["status"].append(list(ar.op_status(bar3)))
        res["rel"].append(orc.rel_error(C3f.data_[rows.to(dev)].cpu(), ref, scale))
        res["identical_across_ranks"].append(identical_on_all_ranks(C3f.data_))
        sync_all()
    del g
    return res


def case_mlp(rank, world, M, K, I, N, seed, iters, max_rows):
    """The tensor-parallel MLP: AllGather+GEMM(gate, up) with the SwiGLU epilogue, then
    GEMM+ReduceScatter(down), two launches back to back with no host synchronisation between."""
    from mkernel_b200 import ops
    dev = torch.device("cuda", rank)
    Ms, Il = M // world, I // world
    g = torch.Generator().manual_seed(seed)
    xs = [torch.randn((Ms, K), generator=g).to(torch.bfloat16) for _ in range(world)]
    wgs = [(torch.randn((Il, K), generator=g) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
    wus = [(torch.randn((Il, K), generator=g) / K ** 0.5).to(torch.bfloat16) for _ in range(world)]
    wds = [(torch.randn((N, Il), generator=g) / I ** 0.5).to(torch.bfloat16) for _ in range(world)]
    rows = _sample_rows(Ms, max_rows, seed)
    x_full = torch.cat(xs, 0)
    grow = rank * Ms + rows
    ref = scale = None
    h_mine = None
    for s_ in range(world):
        gate = x_full.float() @ wgs[s_].float().t()
        up = x_full.float() @ wus[s_].float().t()
        h = (gate * torch.sigmoid(gate) * up).to(torch.bfloat16)
        if s_ == rank:
            h_mine = h
        p = h[grow].float() @ wds[s_].float().t()
        ref = p if ref is None else ref + p
        scale = p.abs() if scale is None else scale + p.abs()
    mlp = ops.TpMlp(M, K, Il, N, rank, world)
    mlp.load_weights(wgs[rank].to(dev), wus[rank].to(dev), wds[rank].to(dev))
    mlp.x.data_.zero_()
    mlp.x.data_[rank].copy_(xs[rank])
    sync_all()
    res = dict(op="mlp", M=M, N=N, K=K, rel=[], rel_plain=[], rel_h=[], status=[], gathered_exact=[])
    for it in range(iters):
        y = mlp.forward()
        torch.cuda.synchronize()
        res["status"].append(list(ops.op_status(mlp.ready)))
        res["status"].append(list(ops.op_status(mlp.sync)))
        res["gathered_exact"].append(bool(torch.equal(mlp.x.data_.view(M, K).cpu(), x_full)))
        res["rel_h"].append(orc.rel_error(mlp.h.view(M, Il).cpu(), h_mine.float()))
        res["rel"].append(orc.rel_error(y[rows.to(dev)].cpu(), ref, scale))
        res["rel_plain"].append(orc.rel_error(y[rows.to(dev)].cpu(), ref))
        dist.barrier()
    sync_all()
    mlp.free()
    return res


CASES = {"ag": case_ag, "rs": case_rs, "ar": case_ar, "compat": case_compat, "graph": case_graph,
         "mlp": case_mlp}


def run_rank(rank: int, world: int, port: int, key: str, cases: list, out_dir: str, options=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["MKB200_BROKER_KEY"] = key
    torch.cuda.set_device(rank)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))   # the oracle runs on every rank
    dist.init_process_group("gloo", rank=rank, world_size=world)
    results = []
    try:
        for name, value in (options or {}).items():
            _lib.set_option(name, value)
        for c in cases:
            c = dict(c)
            fn = CASES[c.pop("op")]
            results.append(fn(rank, world, **c))
    except Exception:
        results.append({"error": traceback.format_exc()})
    Path(out_dir).mkdir(parents=True, exist_ok=True)
    Path(out_dir, f"rank{rank}.json").write_text(json.dumps(results))
    try:
        dist.barrier()
        dist.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cases = json.loads(os.environ.get("MKB200_CASES", "[]"))
    run_rank(rank, world, int(os.environ.get("MASTER_PORT", "29700")),
             os.environ.get("MKB200_BROKER_KEY", "manual"), cases,
             os.environ.get("MKB200_OUT", "multi_gpu_results"))

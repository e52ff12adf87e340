"""Multi-GPU parity: one process per GPU on this box (2..8), every fused operator through the
reference-shaped API against the CPU oracle.  Skipped when fewer than two GPUs are visible."""
import json
import os
import tempfile
import time
import uuid

import pytest
import torch
import torch.multiprocessing as mp

from oracle import tp_gemm_oracle as orc
from tests import multi_gpu_worker as worker

pytestmark = pytest.mark.gpu


def n_gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def launch(world, cases, options=None, timeout=600):
    """One process per GPU.  Every device-side wait of the operators is bounded (4 s), so a rank
    that cannot make progress returns with a status instead of hanging; the join deadline is one
    shared budget for all ranks, and ranks still alive after it are reported, not killed while
    they may hold memory bound to an NVSwitch multicast object."""
    out_dir = tempfile.mkdtemp(prefix="mkb200_mgpu_")
    key = uuid.uuid4().hex[:12]
    from tests.conftest import free_port
    port = free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=worker.run_rank, args=(r, world, port, key, cases, out_dir, options))
             for r in range(world)]
    for p in procs:
        p.start()
    deadline = time.monotonic() + timeout
    for p in procs:
        p.join(max(0.0, deadline - time.monotonic()))
    alive = [p for p in procs if p.is_alive()]
    if alive:
        for p in alive:
            p.join(30.0)            # their bounded waits run out; give them time to unwind
        uses_multicast = bool(options and options.get("use_nvls")) or \
            any(c.get("multicast") for c in cases)
        for p in alive:
            if p.is_alive() and not uses_multicast:
                p.kill()
        raise AssertionError("a rank did not finish within the deadline")
    results = []
    for r in range(world):
        with open(os.path.join(out_dir, f"rank{r}.json")) as f:
            results.append(json.load(f))
    return results


def check(results, rel_tol=orc.REL_TOL, label=""):
    worst = {}
    for rank, per_rank in enumerate(results):
        for res in per_rank:
            assert "error" not in res, res.get("error")
            for st in res["status"]:
                assert st[0] == 0, (rank, res)
            assert max(res["rel"]) <= rel_tol, (rank, res)
            key = (res["op"], res["M"], res["N"], res["K"])
            w = worst.setdefault(key, {"rel": 0.0, "rel_plain": 0.0})
            w["rel"] = max(w["rel"], max(res["rel"]))
            w["rel_plain"] = max(w["rel_plain"], max(res.get("rel_plain") or res["rel"]))
            if "gathered_exact" in res:
                assert all(res["gathered_exact"]), (rank, res)
            if res.get("rerun_identical"):
                assert all(res["rerun_identical"]), (rank, res)
            if "rel_h" in res:
                assert max(res["rel_h"]) <= orc.REL_TOL, (rank, res)
            if "rel_partial" in res:
                assert max(res["rel_partial"]) <= orc.REL_TOL, (rank, res)
            if "identical_across_ranks" in res:
                assert all(res["identical_across_ranks"]), (rank, res)
    # Both error figures per case, for the record: `rel` is the acceptance metric (denominator
    # floored by the rounded partial magnitudes for the reduced operators), `rel_plain` the
    # same without that floor.
    world = len(results)
    for key, w in sorted(worst.items()):
        line = {"world": world, "case": label, "op": key[0], "M": key[1], "N": key[2], "K": key[3],
                "rel": w["rel"], "rel_plain": w["rel_plain"]}
        print("parity", json.dumps(line))
        log = os.environ.get("MKB200_PARITY_LOG")
        if log:
            with open(log, "a") as f:
                f.write(json.dumps(line) + "\n")


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_small_shapes_all_ops():
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=world * 256, N=264, K=200, seed=1, iters=3, max_rows=4096),
        dict(op="ag", M=world * 72, N=512, K=1024, seed=1, iters=2, max_rows=4096),
        dict(op="rs", M=world * 256, N=512, K=192, seed=2, iters=3, max_rows=4096),
        dict(op="rs", M=world * 128, N=264, K=72, seed=2, iters=2, max_rows=4096),
        dict(op="ar", M=128, N=1024, K=256, seed=3, iters=3, max_rows=4096),
        dict(op="ar", M=100, N=264, K=72, seed=3, iters=2, max_rows=4096, layout=0),
        dict(op="ar", M=world * 128, N=512, K=128, seed=3, iters=2, max_rows=4096),
        dict(op="compat", M=world * 128, N=256, K=192, seed=5, iters=2, max_rows=4096),
    ]
    check(launch(world, cases), label="small shapes")


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_baseline_shapes_sampled_rows():
    """The three headline shapes (up-projection AllGather+GEMM, down-projection
    GEMM+ReduceScatter, decode GEMM+AllReduce) at their per-rank sizes, world = GPUs on this box; the oracle is
    evaluated on sampled rows (the full CPU product would take minutes)."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=8192, N=3584, K=8192, seed=1, iters=2, max_rows=256),
        dict(op="rs", M=8192, N=8192, K=3584, seed=2, iters=2, max_rows=256),
        dict(op="ar", M=128, N=8192, K=1024, seed=3, iters=3, max_rows=128),
    ]
    check(launch(world, cases, timeout=900), label="full-size shapes")


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_graph_replays_keep_parity():
    """CUDA-graph replays of all three operators at world size > 1: every replay is checked
    (stale counters, epochs or flags from the previous replay would show)."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="graph", M=world * 256, N=512, K=256, seed=7, replays=3, max_rows=4096),
        dict(op="graph", M=world * 128, N=1024, K=1024, seed=8, replays=3, max_rows=512),
    ]
    check(launch(world, cases), label="graph replays")


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_allgather_variants():
    """The AllGather push through TMA bulk stores, and the one-shot AllReduce, give the same
    results as the defaults."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=world * 256, N=264, K=1024, seed=1, iters=2, max_rows=4096),
        dict(op="ag", M=world * 72, N=512, K=200, seed=1, iters=2, max_rows=4096),
        dict(op="ar", M=128, N=1024, K=256, seed=3, iters=2, max_rows=4096),
    ]
    check(launch(world, cases, options={"push_bulk": 1, "ar_one_shot": 1}))


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_tensor_parallel_mlp_chain():
    """AllGather+GEMM(gate, up) + SwiGLU epilogue -> GEMM+ReduceScatter(down), back to back."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="mlp", M=world * 128, K=256, I=world * 256, N=512, seed=9, iters=3, max_rows=4096),
        dict(op="mlp", M=world * 256, K=1024, I=world * 128, N=264, seed=10, iters=2, max_rows=4096),
    ]
    # two bf16 roundings (H, then the partial products) lie between inputs and output
    check(launch(world, cases), rel_tol=1.5 * orc.REL_TOL, label="TP MLP chain")


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_allreduce_fetching_partials():
    """The two-shot AllReduce in which owners fetch the partials from their producers (the path
    large outputs take; small outputs default to staging slabs filled by posted stores)."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ar", M=128, N=1024, K=256, seed=3, iters=3, max_rows=4096),
        dict(op="ar", M=100, N=264, K=72, seed=3, iters=2, max_rows=4096, layout=0),
        dict(op="ar", M=128, N=8192, K=1024, seed=3, iters=2, max_rows=128),
    ]
    check(launch(world, cases, options={"ar_push": 0}), label="AllReduce, fetched partials")


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_allgather_fanout():
    """The AllGather push that loads a row group once and stores it to every peer gives the same
    (bit-exact gathered operand, same product) results as the per-receiver push."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=world * 256, N=264, K=1024, seed=1, iters=2, max_rows=4096),
        dict(op="ag", M=world * 72, N=512, K=200, seed=1, iters=2, max_rows=4096),
        dict(op="ag", M=world * 1024, N=512, K=2048, seed=4, iters=2, max_rows=64),
    ]
    check(launch(world, cases, options={"ag_fanout": 1}))


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_allgather_k_range_items():
    """The AllGather push in K-range form (an item is every row of a row-block over one K-range;
    the consumer's TMA producer waits range by range inside its K loop) gives a bit-exact gathered
    operand and the same product, ragged K and ragged row-blocks included."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=world * 256, N=264, K=1024, seed=1, iters=2, max_rows=4096),
        dict(op="ag", M=world * 72, N=512, K=200, seed=1, iters=2, max_rows=4096),
        dict(op="ag", M=world * 1024, N=512, K=2048, seed=4, iters=2, max_rows=64),
        dict(op="ag", M=8192, N=3584, K=8192, seed=6, iters=2, max_rows=16),
    ]
    check(launch(world, cases, options={"ag_chunks": 1}))


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_allgather_paced_push():
    """Pacing the AllGather push against the GEMM's own progress changes timing only."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=world * 1024, N=1024, K=1024, seed=5, iters=2, max_rows=64),
        dict(op="ag", M=world * 72, N=512, K=200, seed=1, iters=2, max_rows=4096),
        dict(op="ag", M=8192, N=3584, K=8192, seed=6, iters=2, max_rows=16),
    ]
    check(launch(world, cases, options={"ag_lead": 1}))


@pytest.mark.skipif(n_gpus() < 2, reason="needs at least 2 GPUs")
def test_nvswitch_multicast_paths():
    """Exchange through the multicast alias (multimem.st pushes for AllGather, multimem.ld_reduce +
    multimem.st for AllReduce, multimem.ld_reduce over partials that stay with their producers
    for ReduceScatter) gives the same results; buffers without an alias (multicast not
    supported) fall back to peer loads and stores."""
    world = min(n_gpus(), 8)
    world = 1 << (world.bit_length() - 1)
    cases = [
        dict(op="ag", M=world * 256, N=264, K=1024, seed=1, iters=2, max_rows=4096, multicast=True),
        dict(op="ag", M=8192, N=3584, K=8192, seed=6, iters=2, max_rows=16, multicast=True),
        dict(op="ar", M=128, N=8192, K=1024, seed=3, iters=3, max_rows=128, multicast=True),
        dict(op="rs", M=world * 256, N=512, K=192, seed=2, iters=3, max_rows=4096, multicast=True),
        dict(op="rs", M=8192, N=8192, K=3584, seed=2, iters=2, max_rows=64, multicast=True),
    ]
    # The in-switch sum (multimem.ld_reduce, fp32 accumulate) is not rounded to nearest: at 2 GPUs
    # the AllReduce measured 0.0106 on the parity metric, where the fp32 sum of the default path
    # is bounded by 0.0078.  This opt-in path is therefore held to 1.25e-2; AllGather through
    # multimem.st is a copy and stays bit-exact.
    check(launch(world, cases, options={"use_nvls": 1}), rel_tol=1.25e-2)

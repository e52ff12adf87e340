#!/usr/bin/env python
"""Benchmark of the fused tensor-parallel GEMM + collective operators on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Headline workload (one "step" = prepare + one fused launch, i.e. one kernel): AllGather+GEMM at the
Llama-70B MLP up-projection shape with tensor parallel degree = N: every rank holds an A shard
[8192/N, 8192] and its column shard of B [8192 -> 3584], and produces C [8192, 3584] (bf16 in,
fp32 accumulate, bf16 out).  Work per GPU is fixed (481 GFLOP), so scaling is weak.  The same
run also times GEMM+ReduceScatter (down-projection shape) and GEMM+AllReduce (decode shape) and
their unfused cuBLAS(+NCCL) counterparts and reports them under "ops".

Prints ONE JSON line on rank 0.  `--impl reference` times the reference's CPU path
(torch.matmul on the host cores over a bounded sample of the same workload) instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG2 = dict(M=8192, N=3584, K=8192)          # AllGather+GEMM (headline), N is per rank
CFG3 = dict(M=8192, N=8192, K=3584)          # GEMM+ReduceScatter, K is per rank
CFG4 = dict(M=128, N=8192, K=1024)           # GEMM+AllReduce decode shape, K is per rank
NVLINK_GBS = 900.0                           # per direction per GPU (nominal NVLink 5)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)

# dram__bytes_read.sum + dram__bytes_write.sum of one fused launch at the headline shape on one
# GPU.  Captured with ncu on the half-height case (M=4096: 286.6 MB read + 24.2 MB written per
# launch, profiles/fused_gemm_kernel_vs_cublas_4096x3584x8192.md) and scaled by the tiles
# processed (x2 for M=8192): the raster re-streams B once per group of row-blocks, so traffic
# grows with the number of row-blocks.  Algorithmic bytes of the full launch: 251.7 MB.
NCU_TRAFFIC_BYTES_PER_LAUNCH = 2 * (286.62e6 + 24.25e6)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"],
                    bf16_tflops_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap"}

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(1.0)

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# ------------------------------------------------------------------------------------------------
# distributed plumbing
# ------------------------------------------------------------------------------------------------
class Dist:
    def __init__(self, n_gpus: int):
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != n_gpus:
            if self.world == 1 and n_gpus > 1:
                raise SystemExit(f"--gpus {n_gpus} needs a torchrun launch with {n_gpus} ranks")
            n_gpus = self.world
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))
            self.dist = dist
        else:
            torch.cuda.set_device(0)
        self.device = torch.device("cuda", self.local_rank)

    def barrier(self):
        torch.cuda.synchronize()
        if self.dist is not None:
            self.dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        if self.dist is None:
            return value
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def timed_loop(dst: Dist, step, steps: int, warmup: int, sampler=None):
    """Warm up, then time exactly `steps` calls of step(i, ev0, ev1) with CUDA events on the
    current stream between two barriers.  step records ev0/ev1 around its fused launch.
    Returns (total ms max over ranks, mean fused-launch ms max over ranks)."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(steps)]
    null = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    for i in range(warmup):
        step(i, *null)
    dst.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        t0.record()
        for i in range(steps):
            step(warmup + i, *evs[i])
        t1.record()
        torch.cuda.synchronize()
    dst.barrier()
    total = dst.max_over_ranks(t0.elapsed_time(t1))
    kern = dst.max_over_ranks(sum(a.elapsed_time(b) for a, b in evs) / steps)
    return total, kern


def interleaved_ms(dst: Dist, step_a, step_b, rounds: int, per_round: int):
    """Mean fused-launch time of two arms timed in alternating blocks (a, b, a, b, ...), so that
    both see the same power and thermal state: on this power-capped part a seconds-long kernel
    sequence timed after another one runs measurably slower than the same sequence timed first.
    Returns (ms_a, ms_b), each the max over ranks of the mean over all its blocks."""
    null = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    for i in range(3):
        step_a(i, *null)
        step_b(i, *null)
    sums = [0.0, 0.0]
    for r in range(rounds):
        for arm, step in enumerate((step_a, step_b)):
            evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                   for _ in range(per_round)]
            dst.barrier()
            for i, (e0, e1) in enumerate(evs):
                step(3 + r * per_round + i, e0, e1)
            torch.cuda.synchronize()
            sums[arm] += sum(a.elapsed_time(b) for a, b in evs)
    n = rounds * per_round
    return dst.max_over_ranks(sums[0] / n), dst.max_over_ranks(sums[1] / n)


def graph_time_us(dst: Dist, fn, launches: int, replays: int) -> float:
    """Mean microseconds per call of fn when `launches` calls are captured in one CUDA graph and
    the graph is replayed `replays` times (max over ranks)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            fn()
    dst.barrier()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(launches):
            fn()
    dst.barrier()
    g.replay()
    dst.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(replays):
        g.replay()
    t1.record()
    torch.cuda.synchronize()
    dst.barrier()
    return dst.max_over_ranks(t0.elapsed_time(t1)) * 1e3 / (launches * replays)


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


# ------------------------------------------------------------------------------------------------
# parity (outside every timed region): the operators' outputs against the CPU oracle on sampled
# rows and against an fp32 product of the same bf16 operands over all rows
# ------------------------------------------------------------------------------------------------
PARITY_TOL = 1e-2


def error_figures(out, ref, rounded_scale=None):
    """Error figures of a bf16 output against an fp32 reference, both on the same device.
    rel_plain  = max |out - ref| / max(|ref|, rms(ref));
    rel        = the same with the denominator also floored by `rounded_scale` (the sum over
                 ranks of |partial|: everything that travelled as bf16 on the way to a reduced
                 output); equal to rel_plain when no scale is given;
    three_tier = the reference's own acceptance (bench/common.py:312-367: max_abs <= 0.35 or
                 max_rel <= 0.08 or mean_abs <= 1 % of mean |ref|)."""
    o, e = out.float(), ref.float()
    d = (o - e).abs()
    rms = e.pow(2).mean().sqrt().clamp_min(1e-30)
    den = e.abs().clamp_min(rms)
    plain = float((d / den).max())
    rel = plain if rounded_scale is None else float((d / torch.maximum(den, rounded_scale.abs())).max())
    max_abs, mean_abs, ref_mean = float(d.max()), float(d.mean()), float(e.abs().mean())
    max_rel = float((d / e.abs().clamp_min(1e-6)).max())
    tier = max_abs <= 0.35 or max_rel <= 0.08 or mean_abs <= 0.01 * max(ref_mean, 1e-6)
    return {"rel": rel, "rel_plain": plain, "three_tier_ok": bool(tier)}


def merge_parity(dst, rec):
    """MAX of the error figures / AND of the verdicts over ranks; adds the overall verdict."""
    if dst.dist is not None:
        keys = sorted(k for k, v in rec.items() if isinstance(v, float))
        t = torch.tensor([rec[k] for k in keys], dtype=torch.float64, device=dst.device)
        dst.dist.all_reduce(t, op=dst.dist.ReduceOp.MAX)
        for k, v in zip(keys, t.tolist()):
            rec[k] = v
        flags = sorted(k for k, v in rec.items() if isinstance(v, bool))
        t = torch.tensor([1.0 if rec[k] else 0.0 for k in flags], dtype=torch.float64, device=dst.device)
        dst.dist.all_reduce(t, op=dst.dist.ReduceOp.MIN)
        for k, v in zip(flags, t.tolist()):
            rec[k] = bool(v)
    rec["tolerance"] = PARITY_TOL
    rec["ok"] = bool(rec["rel"] <= PARITY_TOL and rec["rel_oracle"] <= PARITY_TOL and
                     rec["three_tier_ok"] and rec.get("gathered_exact", True))
    return rec


def sum_over_ranks(dst, t):
    if dst.dist is not None:
        dst.dist.all_reduce(t)
    return t


def sample_rows(n_rows, count, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randperm(n_rows, generator=g)[:min(count, n_rows)].sort().values


class NvlinkCounters:
    """Bytes this GPU sent / received over NVLink, read from NVML's per-device throughput
    counters (read-only field values; KiB, summed over links)."""

    TX, RX = 138, 139      # NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_TX / _RX

    def __init__(self, index):
        self.h, self.why = None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.read()
        except Exception as e:
            self.h, self.why = None, repr(e)[:160]

    def read(self):
        if self.h is None:
            return None
        vals = self.nv.nvmlDeviceGetFieldValues(self.h, [(self.TX, 0xFFFFFFFF), (self.RX, 0xFFFFFFFF)])
        out = []
        for v in vals:
            if v.nvmlReturn != 0:
                raise RuntimeError(f"NVML NVLink throughput field returned error {v.nvmlReturn} "
                                   "(3 = not supported on this system)")
            out.append(int(v.value.ullVal) * 1024)
        return out

    def per_launch(self, fn, launches, sync):
        """Runs fn `launches` times and returns {tx_bytes, rx_bytes} per launch, or None."""
        if self.h is None:
            return {"unavailable": self.why}
        try:
            sync()
            a = self.read()
            for i in range(launches):
                fn(i)
            sync()
            time.sleep(0.05)
            b = self.read()
            return {"tx_bytes": (b[0] - a[0]) / launches, "rx_bytes": (b[1] - a[1]) / launches,
                    "launches": launches}
        except Exception as e:
            return {"error": repr(e)[:120]}


def randn_bf16(shape, seed, device, scale=1.0):
    g = torch.Generator(device=device).manual_seed(seed)
    return (torch.randn(shape, device=device, generator=g) * scale).to(torch.bfloat16)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------
def run_ours(args):
    import mkernel_b200
    from mkernel_b200 import _lib, ops
    from oracle import tp_gemm_oracle as orc      # the checker of the parity records only

    dst = Dist(args.gpus)
    W, rank, dev = dst.world, dst.local_rank, dst.device
    peaks, peak_kind = load_peaks()
    steps, warmup = args.steps, max(args.warmup, 3)
    torch.backends.cuda.matmul.allow_tf32 = False          # fp32 checker products stay fp32
    torch.set_float32_matmul_precision("highest")
    cores = os.cpu_count() or 1
    nvl = NvlinkCounters(rank) if W > 1 else None

    def sync():
        dst.barrier()

    # ---------------- headline: AllGather + GEMM ----------------
    M, N, K = CFG2["M"], CFG2["N"], CFG2["K"]
    Ms = M // W
    ag = mkernel_b200.load("ag_gemm_warp_specialized")
    A = ag.DistBuffer((W, Ms, K), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
    ready = ag.DistBuffer((ag.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                          local_rank=rank, local_world_size=W)
    ready.data_.zero_()
    A.data_.zero_()
    A.data_[rank].copy_(randn_bf16((Ms, K), 1 + rank, dev))
    B = randn_bf16((N, K), 101 + rank, dev, K ** -0.5)      # stored [N, K] as the operator takes it
    C = torch.zeros((W, Ms, N), device=dev, dtype=torch.bfloat16)
    dst.barrier()

    def ag_step(i, e0, e1):
        ag.ag_gemm_warp_specialized_prepare(ready, M, N)
        e0.record()
        ag.ag_gemm_warp_specialized_launch(A, ready, B, C)
        e1.record()

    # Set-up, untimed: an idle GPU sits at its lowest clocks and takes tens of milliseconds of
    # work to ramp; without this the first timed steps of a short run measure the ramp (at four
    # GPUs one slow-ramping rank held the whole job at 0.62 of peak instead of 0.75).
    ramp_ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    for i in range(60):
        ag_step(i, *ramp_ev)
    dst.barrier()
    sampler = ClockSampler(rank)
    total_ms, kern_ms = timed_loop(dst, ag_step, steps, warmup, sampler)
    ag.op_status(ready)
    flops_per_gpu = 2.0 * M * N * K
    ms_per_step = total_ms / steps
    value = W * flops_per_gpu / (ms_per_step * 1e-3) / 1e12
    achieved = flops_per_gpu / (kern_ms * 1e-3) / 1e12
    ag_bytes = (W - 1) / W * M * K * 2
    t_roof_ms = max(flops_per_gpu / (peaks["bf16_tflops"] * 1e12), ag_bytes / (NVLINK_GBS * 1e9)) * 1e3
    null_ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    ag_nvlink = nvl.per_launch(lambda i: ag_step(i, *null_ev), 50, sync) if nvl else None

    # sustained: the same launch back to back for at least a second (power-capped clocks)
    sus_sampler = ClockSampler(rank)
    sus_steps = max(200, int(1.2 / (kern_ms * 1e-3)))
    sus_total, _ = timed_loop(dst, ag_step, sus_steps, 3, sus_sampler)
    ag.op_status(ready)
    sus_tflops = flops_per_gpu / (sus_total / sus_steps * 1e-3) / 1e12
    sustained = {"seconds": sus_total * 1e-3, "launches": sus_steps, "tflops_per_gpu": sus_tflops,
                 "peak": peaks["bf16_tflops_sustained"],
                 "frac": sus_tflops / peaks["bf16_tflops_sustained"], "clocks": sus_sampler.summary()}

    # ---------------- parity of the headline operator (untimed) ----------------
    # Poison the remote slabs first so that a gather that did not happen would be noticed.
    for r in range(W):
        if r != rank:
            A.data_[r].zero_()
    C.zero_()
    dst.barrier()
    ag_step(0, *null_ev)
    dst.barrier()
    a_full = torch.cat([randn_bf16((Ms, K), 1 + r, dev) for r in range(W)], 0)
    rec = {"gathered_exact": bool(torch.equal(A.data_.view(M, K), a_full))}
    rec.update(error_figures(C.view(M, N), a_full.float() @ B.float().t()))
    rows = sample_rows(M, 256, 11)
    torch.set_num_threads(max(1, cores // W))
    _, c_orc = orc.ag_gemm_ref([a_full[rows.to(dev)].cpu()], B.t().cpu())
    rec["rel_oracle"] = orc.rel_error(C.view(M, N)[rows.to(dev)].cpu(), c_orc)
    rec["rows_oracle"], rec["rows_fp32"] = int(rows.numel()), M
    ag_parity = merge_parity(dst, rec)
    del a_full

    # ---------------- end to end through the public API, host buffers ----------------
    # Three streams: the host-to-device copy of step i+1, the kernel of step i and the
    # device-to-host copy of step i-1 overlap; operands and outputs are double buffered.
    hA = randn_bf16((Ms, K), 1 + rank, "cpu").pin_memory()
    hB = B.cpu().pin_memory()
    A2 = ag.DistBuffer((W, Ms, K), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
    ready2 = ag.DistBuffer((ag.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                           local_rank=rank, local_world_size=W)
    ready2.data_.zero_()
    A2.data_.zero_()
    bufA, bufR = (A, A2), (ready, ready2)
    bufB = (torch.empty_like(B), torch.empty_like(B))
    bufC = (C, torch.zeros_like(C))
    hC = (torch.empty((W, Ms, N), dtype=torch.bfloat16).pin_memory(),
          torch.empty((W, Ms, N), dtype=torch.bfloat16).pin_memory())
    s_in, s_k, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    dst.barrier()

    def e2e_run(n):
        ev_in = [torch.cuda.Event() for _ in range(n)]
        ev_k = [torch.cuda.Event() for _ in range(n)]
        ev_out = [torch.cuda.Event() for _ in range(n)]
        for i in range(n):
            b = i & 1
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_k[i - 2])        # kernel i-2 has read these buffers
                bufA[b].data_[rank].copy_(hA, non_blocking=True)
                bufB[b].copy_(hB, non_blocking=True)
                ev_in[i].record(s_in)
            with torch.cuda.stream(s_k):
                s_k.wait_event(ev_in[i])
                if i >= 2:
                    s_k.wait_event(ev_out[i - 2])       # output buffer has been read back
                ag.ag_gemm_warp_specialized_prepare(bufR[b], M, N)
                ag.ag_gemm_warp_specialized_launch(bufA[b], bufR[b], bufB[b], bufC[b])
                ev_k[i].record(s_k)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[i])
                hC[b].copy_(bufC[b], non_blocking=True)
                ev_out[i].record(s_out)
        for st in (s_in, s_k, s_out):
            torch.cuda.current_stream().wait_stream(st)

    e2e_steps = max(6, min(steps, 20))
    e2e_run(4)
    dst.barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    e2e_run(e2e_steps)
    t1.record()
    torch.cuda.synchronize()
    dst.barrier()
    e2e_total = dst.max_over_ranks(t0.elapsed_time(t1))
    ag.op_status(ready)
    ag.op_status(ready2)
    e2e_ok = bool(torch.equal(hC[0], hC[1]) and torch.equal(hC[0].to(dev), C))
    e2e_value = W * flops_per_gpu / (e2e_total / e2e_steps * 1e-3) / 1e12
    h2d = hA.numel() * 2 + hB.numel() * 2
    d2h = hC[0].numel() * 2

    # ---------------- unfused comparator for the headline ----------------
    ops_out = {}
    A_full = torch.empty((M, K), device=dev, dtype=torch.bfloat16)
    A_loc = A.data_[rank]
    C2 = torch.empty((M, N), device=dev, dtype=torch.bfloat16)

    def ag_unfused(i, e0, e1):
        e0.record()
        if W > 1:
            dst.dist.all_gather_into_tensor(A_full, A_loc)
            torch.matmul(A_full, B.t(), out=C2)
        else:
            torch.matmul(A_loc, B.t(), out=C2)
        e1.record()

    sub_steps = max(5, min(steps, 20))
    # fused and unfused arms of every operator record are timed in alternating blocks
    ag_f_ms, ag_unf_ms = interleaved_ms(dst, ag_step, ag_unfused, 4, max(2, sub_steps // 4))
    ag.op_status(ready)
    ops_out["ag_gemm"] = op_record("AllGather+GEMM", CFG2, W, ag_f_ms, ag_unf_ms, flops_per_gpu,
                                   ag_bytes, peaks)
    ops_out["ag_gemm"]["parity"] = ag_parity
    ops_out["ag_gemm"]["nvlink_measured"] = ag_nvlink
    del A_full, C2, hA, hB, hC, bufB, bufC
    A2.free(); ready2.free()

    # ---------------- GEMM + ReduceScatter (config 3) ----------------
    M3, N3, K3 = CFG3["M"], CFG3["N"], CFG3["K"]
    rs = mkernel_b200.load("gemm_rs_blackwell")
    A3 = randn_bf16((M3, K3), 2 + rank, dev)
    B3 = randn_bf16((N3, K3), 202 + rank, dev, (K3 * W) ** -0.5)
    C3 = rs.DistBuffer((M3, N3), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
    sync3 = rs.DistBuffer(rs.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=rank,
                          local_world_size=W)
    rs.gemm_rs_blackwell_prepare(A3, B3, C3, sync3)
    dst.barrier()

    def rs_step(i, e0, e1):
        e0.record()
        rs.gemm_rs_blackwell_launch(A3, B3, C3, sync3)
        e1.record()

    rs_nvlink = nvl.per_launch(lambda i: rs_step(i, *null_ev), 50, sync) if nvl else None
    c3 = torch.empty((M3, N3), device=dev, dtype=torch.bfloat16)
    c3_rs = torch.empty((M3 // W, N3), device=dev, dtype=torch.bfloat16)

    def rs_unfused(i, e0, e1):
        e0.record()
        torch.mm(A3, B3.t(), out=c3)
        if W > 1:
            dst.dist.reduce_scatter_tensor(c3_rs, c3)
        e1.record()

    rs_ms, rs_unf_ms = interleaved_ms(dst, rs_step, rs_unfused, 4, max(2, sub_steps // 4))
    rs.op_status(sync3)
    ops_out["gemm_rs"] = op_record("GEMM+ReduceScatter", CFG3, W, rs_ms, rs_unf_ms,
                                   2.0 * M3 * N3 * K3, (W - 1) / W * M3 * N3 * 2, peaks)
    del c3, c3_rs
    # parity: this rank's rows of the sum over ranks of the fp32 partial products
    dst.barrier()
    rs_step(0, *null_ev)
    dst.barrier()
    Ms3 = M3 // W
    part = A3.float() @ B3.float().t()
    scale = sum_over_ranks(dst, part.abs())[rank * Ms3:(rank + 1) * Ms3].clone()
    ref = sum_over_ranks(dst, part)[rank * Ms3:(rank + 1) * Ms3]
    out3 = C3.data_[rank * Ms3:(rank + 1) * Ms3]
    rec = error_figures(out3, ref, scale)
    del part, ref, scale
    per_owner = max(1, 256 // W)
    grows = torch.cat([o * Ms3 + sample_rows(Ms3, per_owner, 12) for o in range(W)])
    tot, parts = orc.gemm_ar_ref([A3[grows.to(dev)].cpu()], [B3.t().cpu()])
    tot = sum_over_ranks(dst, tot.to(dev)).cpu()
    sc = sum_over_ranks(dst, parts[0].abs().to(dev)).cpu()
    mine = slice(rank * per_owner, (rank + 1) * per_owner)
    own_rows = (grows[mine] - rank * Ms3).to(dev)
    rec["rel_oracle"] = orc.rel_error(out3[own_rows].cpu(), tot[mine], sc[mine])
    rec["rel_oracle_plain"] = orc.rel_error(out3[own_rows].cpu(), tot[mine])
    rec["rows_oracle"], rec["rows_fp32"] = int(grows.numel()), M3
    ops_out["gemm_rs"]["parity"] = merge_parity(dst, rec)
    ops_out["gemm_rs"]["nvlink_measured"] = rs_nvlink
    rs.op_status(sync3)
    C3.free(); sync3.free()
    del A3, B3

    # ---------------- GEMM + AllReduce (config 4, decode shape) ----------------
    M4, N4, K4 = CFG4["M"], CFG4["N"], CFG4["K"]
    ar = mkernel_b200.load("gemm_ar_blackwell")
    A4 = randn_bf16((M4, K4), 3 + rank, dev)
    B4 = randn_bf16((K4, N4), 303 + rank, dev, (K4 * W) ** -0.5)
    C4 = ar.DistBuffer((M4, N4), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
    C4f = ar.DistBuffer((M4, N4), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
    bar4 = ar.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=rank, local_world_size=W)
    bar4.data_.zero_()
    dst.barrier()

    def ar_step(i, e0, e1):
        e0.record()
        ar.gemm_ar_intranode_blackwell(A4, B4, C4, bar4, C4f, i + 1)
        e1.record()

    ar_steps = max(20, sub_steps)
    _, ar_ms = timed_loop(dst, ar_step, ar_steps, 5)
    ar.op_status(bar4)
    epoch_base = ar_steps + 5
    ar_nvlink = nvl.per_launch(lambda i: ar_step(epoch_base + i, *null_ev), 200, sync) if nvl else None
    epoch_base += 200
    c4 = torch.empty((M4, N4), device=dev, dtype=torch.bfloat16)

    def ar_unfused(i, e0, e1):
        e0.record()
        torch.matmul(A4, B4, out=c4)
        if W > 1:
            dst.dist.all_reduce(c4)
        e1.record()

    _, ar_unf_ms = timed_loop(dst, ar_unfused, ar_steps, 5)
    rec = op_record("GEMM+AllReduce (decode)", CFG4, W, ar_ms, ar_unf_ms, 2.0 * M4 * N4 * K4,
                    M4 * N4 * 2 if W > 1 else 0, peaks)
    hbm_bytes = (M4 * K4 + K4 * N4 + 2 * M4 * N4) * 2
    rec["fused_us"] = ar_ms * 1e3
    rec["hbm_floor_us"] = hbm_bytes / (peaks["hbm_gbs"] * 1e9) * 1e6
    rec["nvlink_measured"] = ar_nvlink
    # parity: output identical on all ranks, partial and sum against fp32 and the oracle
    C4f.data_.zero_()
    dst.barrier()
    ar_step(epoch_base, *null_ev)
    epoch_base += 1
    dst.barrier()
    part = A4.float() @ B4.float()
    par = error_figures(C4f.data_, sum_over_ranks(dst, part.clone()), sum_over_ranks(dst, part.abs()))
    par["rel_partial"] = error_figures(C4.data_, part)["rel"]
    tot, parts = orc.gemm_ar_ref([A4.cpu()], [B4.cpu()])
    tot = sum_over_ranks(dst, tot.to(dev)).cpu()
    sc = sum_over_ranks(dst, parts[0].abs().to(dev)).cpu()
    par["rel_oracle"] = orc.rel_error(C4f.data_.cpu(), tot, sc)
    par["rel_oracle_plain"] = orc.rel_error(C4f.data_.cpu(), tot)
    par["rows_oracle"], par["rows_fp32"] = M4, M4
    if W > 1:   # bit-identical output on every rank (bench/common.py:469-500)
        bits = C4f.data_.view(torch.int16).to(torch.int32)
        lo, hi = bits.clone(), bits.clone()
        dst.dist.all_reduce(lo, op=dst.dist.ReduceOp.MIN)
        dst.dist.all_reduce(hi, op=dst.dist.ReduceOp.MAX)
        par["identical_across_ranks"] = bool(torch.equal(lo, hi))
    rec["parity"] = merge_parity(dst, par)
    if W > 1:
        rec["parity"]["ok"] = rec["parity"]["ok"] and rec["parity"]["identical_across_ranks"]
    # The decode shape is latency-bound and an eager loop mostly measures host launch overhead,
    # so both arms are also timed as CUDA-graph replays of 10 launches (device-resident epoch).
    rec["graph_fused_us"], rec["graph_unfused_us"] = None, None
    try:
        def fused_dev_epoch():
            ar.gemm_ar_intranode_blackwell(A4, B4, C4, bar4, C4f, 0)

        def unfused():
            torch.matmul(A4, B4, out=c4)
            if W > 1:
                dst.dist.all_reduce(c4)

        rec["graph_fused_us"] = graph_time_us(dst, fused_dev_epoch, 10, 10)
        rec["graph_unfused_us"] = graph_time_us(dst, unfused, 10, 10)
        ar.op_status(bar4)
        # the replayed launches must still produce the checked result
        rec["parity"]["graph_replay_rel"] = dst.max_over_ranks(error_figures(
            C4f.data_, sum_over_ranks(dst, part.clone()), sum_over_ranks(dst, part.abs()))["rel"])
        rec["parity"]["ok"] = rec["parity"]["ok"] and rec["parity"]["graph_replay_rel"] <= PARITY_TOL
    except Exception as e:  # graph capture of the comparator is best effort
        rec["graph_error"] = repr(e)[:200]
    ops_out["gemm_ar"] = rec

    C4.free(); C4f.free(); bar4.free()
    del A4, B4, c4
    A.free(); ready.free()
    del B, C
    torch.cuda.empty_cache()

    # ---------------- in-switch ReduceScatter variant (opt-in), against the default ----------------
    if W > 1:
        ops_out["gemm_rs"]["in_switch_variant"] = rs_in_switch_record(dst, rs, _lib, sub_steps)

    # ---------------- TP MLP chain: AG+GEMM(gate, up)+SwiGLU -> GEMM+RS(down) ----------------
    ops_out["mlp_chain"] = mlp_chain_record(dst, ops, peaks, sub_steps)

    traffic = NCU_TRAFFIC_BYTES_PER_LAUNCH if W == 1 else None
    line = {
        "metric": "fused AG-GEMM TFLOPS (whole job; GEMM-RS / GEMM-AR under ops)",
        "value": value, "unit": "TFLOP/s", "per_gpu": value / W,
        "n_gpus": W, "steps": steps, "warmup": warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": headline_config(W),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops"],
                     "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"],
                     "peak_source": f"{peak_kind} (burst cuBLAS bf16)",
                     "kernel_ms": kern_ms, "fused_roofline_ms": t_roof_ms,
                     "fused_roofline_frac": t_roof_ms / kern_ms,
                     "traffic": traffic,
                     "traffic_note": ("DRAM bytes per launch from an ncu capture of the one-GPU case"
                                      if W == 1 else
                                      "not captured at this world size (a multi-rank launch is "
                                      "never put under ncu); one-GPU figure: "
                                      f"{NCU_TRAFFIC_BYTES_PER_LAUNCH:.3e} bytes"),
                     "sustained": sustained},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_total / e2e_steps,
                "pipeline": "3 streams, double-buffered operands and outputs",
                "outputs_match_device_result": e2e_ok},
        "gpu_launches": steps,
        "clocks": sampler.summary(),
        "parity": {k: v["parity"]["ok"] for k, v in ops_out.items() if "parity" in v},
        "ops": ops_out,
        "plan": plan_summary(_lib, W, rank),
    }
    if W == 1:
        line["cpu_baseline"] = cpu_baseline(CFG2, 1, budget_s=10.0)
    all_ok = all(line["parity"].values()) and e2e_ok
    if dst.rank == 0:
        print(json.dumps(line), flush=True)
    dst.barrier()
    if dst.dist is not None:
        dst.dist.destroy_process_group()
    if not all_ok:
        raise SystemExit("parity check failed: see the 'parity' records of the line above")


def rs_in_switch_record(dst, rs, _lib, steps):
    """GEMM+ReduceScatter with the partials left in place and summed by the NVSwitch
    (multimem.ld_reduce) instead of pushed into the owner's slabs and summed by SMs: time and
    error figure next to the default's.  Needs buffers with a multicast alias."""
    W, rank, dev = dst.world, dst.local_rank, dst.device
    M3, N3, K3 = CFG3["M"], CFG3["N"], CFG3["K"]
    A3 = randn_bf16((M3, K3), 2 + rank, dev)
    B3 = randn_bf16((N3, K3), 202 + rank, dev, (K3 * W) ** -0.5)
    try:
        C3 = rs.DistBuffer((M3, N3), dtype=torch.bfloat16, local_rank=rank, local_world_size=W,
                           multicast=True)
    except Exception as e:
        return {"unavailable": repr(e)[:160]}
    sync3 = rs.DistBuffer(rs.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=rank,
                          local_world_size=W)
    rs.gemm_rs_blackwell_prepare(A3, B3, C3, sync3)
    dst.barrier()
    rec = {"multicast": bool(C3.multicast_enabled)}
    if C3.multicast_enabled:
        def step(i, e0, e1):
            e0.record()
            rs.gemm_rs_blackwell_launch(A3, B3, C3, sync3)
            e1.record()
        for name, flag in (("default_ms", 0), ("in_switch_ms", 1)):
            _lib.set_option("use_nvls", flag)
            dst.barrier()
            _, rec[name] = timed_loop(dst, step, steps, 3)
        # error figure of the in-switch path (its sum is not rounded to nearest)
        Ms3 = M3 // W
        part = A3.float() @ B3.float().t()
        scale = sum_over_ranks(dst, part.abs())[rank * Ms3:(rank + 1) * Ms3].clone()
        ref = sum_over_ranks(dst, part)[rank * Ms3:(rank + 1) * Ms3]
        f = error_figures(C3.data_[rank * Ms3:(rank + 1) * Ms3], ref, scale)
        rec["in_switch_rel"] = dst.max_over_ranks(f["rel"])
        rec["in_switch_rel_plain"] = dst.max_over_ranks(f["rel_plain"])
        _lib.set_option("use_nvls", 0)
        rs.op_status(sync3)
        del part, ref, scale
    dst.barrier()
    C3.free(); sync3.free()
    return rec


def mlp_chain_record(dst, ops, peaks, steps):
    """Llama-70B MLP with TP = n_gpus (I_local = 3584 per GPU): the fused chain (two launches:
    AllGather+GEMM of gate and up with the SwiGLU epilogue, GEMM+ReduceScatter of down) against
    the same two operators with the activation as a separate elementwise kernel, and against the
    unfused cuBLAS + NCCL chain."""
    W, rank, dev = dst.world, dst.local_rank, dst.device
    M, K, I, N = 8192, 8192, 3584, 8192
    Ms = M // W
    mlp = ops.TpMlp(M, K, I, N, rank, W)
    wg = randn_bf16((I, K), 701 + rank, dev, K ** -0.5)
    wu = randn_bf16((I, K), 801 + rank, dev, K ** -0.5)
    wd = randn_bf16((N, I), 901 + rank, dev, (I * W) ** -0.5)
    mlp.load_weights(wg, wu, wd)
    mlp.x.data_.zero_()
    mlp.x.data_[rank].copy_(randn_bf16((Ms, K), 601 + rank, dev))
    dst.barrier()

    def fused(i, e0, e1):
        e0.record()
        mlp.forward()
        e1.record()

    for i in range(3):
        fused(i, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    ops.op_status(mlp.ready); ops.op_status(mlp.sync)
    # parity of the chain (untimed): fp32 products of the same bf16 operands, H stored as bf16
    y = mlp.forward()
    dst.barrier()
    x_full = torch.cat([randn_bf16((Ms, K), 601 + r, dev) for r in range(W)], 0)
    gate = x_full.float() @ wg.float().t()
    gate = gate * torch.sigmoid(gate)
    gate *= x_full.float() @ wu.float().t()
    h_ref = gate.to(torch.bfloat16)
    del gate
    rel_h = error_figures(mlp.h.view(M, I), h_ref.float())["rel"]
    part = h_ref.float() @ wd.float().t()
    scale = sum_over_ranks(dst, part.abs())[rank * Ms:(rank + 1) * Ms].clone()
    ref = sum_over_ranks(dst, part)[rank * Ms:(rank + 1) * Ms]
    f = error_figures(y, ref, scale)
    parity = {"rel": dst.max_over_ranks(f["rel"]), "rel_plain": dst.max_over_ranks(f["rel_plain"]),
              "rel_activation": dst.max_over_ranks(rel_h),
              "gathered_exact": bool(torch.equal(mlp.x.data_.view(M, K), x_full)),
              "tolerance": PARITY_TOL}
    # Two bf16 roundings lie between the inputs and this output (H, then the partial products),
    # and H is computed with the fast exponential: the chain is held to 1.5e-2, each of its two
    # operators alone to 1e-2 (the activation here, GEMM+ReduceScatter in its own record).
    parity["tolerance_chain"] = 1.5 * PARITY_TOL
    parity["ok"] = bool(parity["rel"] <= parity["tolerance_chain"] and
                        parity["rel_activation"] <= PARITY_TOL and parity["gathered_exact"])
    del part, ref, scale, h_ref, x_full

    # the same two operators, activation as its own kernel on [M, 2I]
    gu = torch.empty((W, Ms, 2 * I), device=dev, dtype=torch.bfloat16)

    def separate(i, e0, e1):
        e0.record()
        ops.ag_gemm_warp_specialized_prepare(mlp.ready, M, 2 * I)
        ops.ag_gemm_warp_specialized_launch(mlp.x, mlp.ready, mlp.w_gate_up, gu)
        g4 = gu.view(M, I // 128, 2, 128)
        torch.mul(torch.nn.functional.silu(g4[:, :, 0]), g4[:, :, 1], out=mlp.h.view(M, I // 128, 128))
        ops.gemm_rs_blackwell_launch(mlp.h.view(M, I), mlp.w_down, mlp.y, mlp.sync)
        e1.record()

    fused_ms, sep_ms = interleaved_ms(dst, fused, separate, 4, max(2, steps // 4))
    ops.op_status(mlp.ready); ops.op_status(mlp.sync)
    del gu
    # unfused: NCCL all-gather, cuBLAS, elementwise, cuBLAS, NCCL reduce-scatter
    x_all = torch.empty((M, K), device=dev, dtype=torch.bfloat16)
    g_u = torch.empty((M, 2 * I), device=dev, dtype=torch.bfloat16)
    hh = torch.empty((M, I), device=dev, dtype=torch.bfloat16)
    yy = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    y_rs = torch.empty((Ms, N), device=dev, dtype=torch.bfloat16)
    w_cat = torch.cat((wg, wu), 0)

    def unfused(i, e0, e1):
        e0.record()
        if W > 1:
            dst.dist.all_gather_into_tensor(x_all, mlp.x.data_[rank])
            torch.matmul(x_all, w_cat.t(), out=g_u)
        else:
            torch.matmul(mlp.x.data_[rank], w_cat.t(), out=g_u)
        torch.mul(torch.nn.functional.silu(g_u[:, :I]), g_u[:, I:], out=hh)
        torch.mm(hh, wd.t(), out=yy)
        if W > 1:
            dst.dist.reduce_scatter_tensor(y_rs, yy)
        e1.record()

    fused_vs_sep_ms = fused_ms
    fused_ms, unf_ms = interleaved_ms(dst, fused, unfused, 4, max(2, steps // 4))
    flops = 2.0 * M * (2 * I) * K + 2.0 * M * N * I
    nvlink = (W - 1) / W * (M * K + M * N) * 2
    t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), nvlink / (NVLINK_GBS * 1e9)) * 1e3
    rec = {"name": "TP MLP chain (AG+GEMM gate/up + SwiGLU -> GEMM+RS down)",
           "shape": {"M": M, "K": K, "I_per_gpu": I, "N": N}, "tp": W,
           "fused_ms": fused_ms, "separate_activation_ms": sep_ms, "unfused_ms": unf_ms,
           "speedup_vs_separate": sep_ms / fused_vs_sep_ms, "speedup_vs_unfused": unf_ms / fused_ms,
           "tflops_per_gpu": flops / (fused_ms * 1e-3) / 1e12,
           "fused_roofline_ms": t_roof, "fused_roofline_frac": t_roof / fused_ms,
           "launches_per_step": 2, "parity": parity}
    mlp.free()
    return rec


def headline_config(W):
    M, N, K = CFG2["M"], CFG2["N"], CFG2["K"]
    return {"workload": "AllGather+GEMM, Llama-70B MLP up-proj, TP=n_gpus: A shard "
                        f"[{M // W},{K}] x B [{K},{N}] -> C [{M},{N}] per GPU",
            "M": M, "N_per_gpu": N, "K": K, "tp": W,
            "l2": "operands 246 MB per GPU exceed the 126 MB L2; no flush between steps",
            "step": "one fused persistent kernel (prepare is host-side validation only)"}


def run_sweep(args):
    """The scaling sweep: AllGather+GEMM and GEMM+ReduceScatter at total M in {2048, 8192, 32768},
    K = 8192, global N = 28672 sharded by the world size.  Prints one JSON line {"sweep": [...]}
    with TFLOP/s per GPU, the fused-roofline fraction and the unfused cuBLAS(+NCCL) time.  The two
    arms of a point are timed in alternating blocks (see interleaved_ms)."""
    import mkernel_b200

    dst = Dist(args.gpus)
    W, rank, dev = dst.world, dst.local_rank, dst.device
    peaks, _ = load_peaks()
    ag = mkernel_b200.load("ag_gemm_warp_specialized")
    rs = mkernel_b200.load("gemm_rs_blackwell")
    out = []
    steps = max(5, min(args.steps, 20))
    for M in (2048, 8192, 32768):
        K, NG = 8192, 28672
        Nl = NG // W
        # ---- AllGather + GEMM: A_r [M/W, K], B_r [Nl, K] -> C [M, Nl]
        Ms = M // W
        A = ag.DistBuffer((W, Ms, K), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
        ready = ag.DistBuffer((ag.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                              local_rank=rank, local_world_size=W)
        ready.data_.zero_()
        A.data_.zero_()
        A.data_[rank].copy_(randn_bf16((Ms, K), 4 + rank, dev))
        B = randn_bf16((Nl, K), 404 + rank, dev, K ** -0.5)
        C = torch.empty((W, Ms, Nl), device=dev, dtype=torch.bfloat16)
        A_full = torch.empty((M, K), device=dev, dtype=torch.bfloat16)
        C2 = torch.empty((M, Nl), device=dev, dtype=torch.bfloat16)
        dst.barrier()

        def ag_step(i, e0, e1):
            ag.ag_gemm_warp_specialized_prepare(ready, M, Nl)
            e0.record()
            ag.ag_gemm_warp_specialized_launch(A, ready, B, C)
            e1.record()

        def ag_unf(i, e0, e1):
            e0.record()
            if W > 1:
                dst.dist.all_gather_into_tensor(A_full, A.data_[rank])
                torch.matmul(A_full, B.t(), out=C2)
            else:
                torch.matmul(A.data_[rank], B.t(), out=C2)
            e1.record()

        f_ms, u_ms = interleaved_ms(dst, ag_step, ag_unf, 4, max(2, steps // 4))
        ag.op_status(ready)
        out.append(op_record("AllGather+GEMM", dict(M=M, N=Nl, K=K), W, f_ms, u_ms,
                             2.0 * M * Nl * K, (W - 1) / W * M * K * 2, peaks))
        A.free(); ready.free()
        del B, C, A_full, C2
        # ---- GEMM + ReduceScatter: A_r [M, NG/W], B_r [K, NG/W] -> out_r [M/W, K]
        Kl, N3 = NG // W, K
        A3 = randn_bf16((M, Kl), 4 + rank, dev)
        B3 = randn_bf16((N3, Kl), 504 + rank, dev, NG ** -0.5)
        C3 = rs.DistBuffer((M, N3), dtype=torch.bfloat16, local_rank=rank, local_world_size=W)
        s3 = rs.DistBuffer(rs.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=rank,
                           local_world_size=W)
        rs.gemm_rs_blackwell_prepare(A3, B3, C3, s3)
        c3 = torch.empty((M, N3), device=dev, dtype=torch.bfloat16)
        c3r = torch.empty((M // W, N3), device=dev, dtype=torch.bfloat16)
        dst.barrier()

        def rs_step(i, e0, e1):
            e0.record()
            rs.gemm_rs_blackwell_launch(A3, B3, C3, s3)
            e1.record()

        def rs_unf(i, e0, e1):
            e0.record()
            torch.mm(A3, B3.t(), out=c3)
            if W > 1:
                dst.dist.reduce_scatter_tensor(c3r, c3)
            e1.record()

        f_ms, u_ms = interleaved_ms(dst, rs_step, rs_unf, 4, max(2, steps // 4))
        rs.op_status(s3)
        out.append(op_record("GEMM+ReduceScatter", dict(M=M, N=N3, K=Kl), W, f_ms, u_ms,
                             2.0 * M * N3 * Kl, (W - 1) / W * M * N3 * 2, peaks))
        C3.free(); s3.free()
        del A3, B3, c3, c3r
        torch.cuda.empty_cache()
    if dst.rank == 0:
        print(json.dumps({"sweep": out, "n_gpus": W, "peak_tflops": peaks["bf16_tflops"]}), flush=True)
    dst.barrier()
    if dst.dist is not None:
        dst.dist.destroy_process_group()


def run_case(args):
    """One operator a few times on one GPU (world size 1, empty exchange step) with seeded
    synthetic operands: the small, bounded case to put under a profiler, e.g.
    ``ncu -k regex:fused_gemm_kernel ... python bench.py --case ag --m 4096 --n 3584 --k 8192``.
    --with-cublas also runs torch.mm (cuBLAS) on the same operands so that one capture holds
    both kernels.  Prints a plain text line, not the bench JSON."""
    import mkernel_b200
    from mkernel_b200 import _lib, ops

    M, N, K = args.m, args.n, args.k
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator(device=dev).manual_seed(1)
    A = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
    B_nk = (torch.randn((N, K), device=dev, generator=g) * K ** -0.5).to(torch.bfloat16)
    if args.block_n:
        _lib.set_option("block_n", args.block_n)
    if args.cta_pair is not None:
        _lib.set_option("cta_pair", args.cta_pair)
    if args.case == "gemm":
        C = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        run = lambda i: ops.gemm_bf16(A, B_nk, C)
    elif args.case == "ag":
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
    elif args.case == "rs":
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

    def timed(fn, iters, warmup):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    ms = timed(run, args.iters, args.case_warmup)
    print(f"case={args.case} M={M} N={N} K={K}: {ms:.4f} ms/iter, "
          f"{2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")
    if args.with_cublas:
        C2 = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        ms = timed(lambda i: torch.mm(A, B_nk.t(), out=C2), args.iters, args.case_warmup)
        print(f"cublas M={M} N={N} K={K}: {ms:.4f} ms/iter, {2.0 * M * N * K / ms / 1e9:.1f} TFLOP/s")


def plan_summary(_lib, W, rank):
    out = {}
    for name, op, cfg, layout in (("ag_gemm", _lib.OP_AG, CFG2, 0), ("gemm_rs", _lib.OP_RS, CFG3, 0),
                                  ("gemm_ar", _lib.OP_AR, CFG4, 1)):
        p = _lib.plan_op(op, rank, W, cfg["M"], cfg["N"], cfg["K"], layout,
                         torch.cuda.get_device_properties(rank).multi_processor_count)
        out[name] = {"block_n": p.block_n, "stages": p.stages, "exchange_ctas": p.n_comm,
                     "grid": p.grid}
    return out


def op_record(name, cfg, W, fused_ms, unfused_ms, flops, nvlink_bytes, peaks):
    t_roof = max(flops / (peaks["bf16_tflops"] * 1e12), nvlink_bytes / (NVLINK_GBS * 1e9)) * 1e3
    return {"name": name, "shape": cfg, "tp": W, "fused_ms": fused_ms, "unfused_ms": unfused_ms,
            "tflops_per_gpu": flops / (fused_ms * 1e-3) / 1e12,
            "unfused_tflops_per_gpu": flops / (unfused_ms * 1e-3) / 1e12,
            "speedup_vs_unfused": unfused_ms / fused_ms,
            "fused_roofline_ms": t_roof, "fused_roofline_frac": t_roof / fused_ms,
            "nvlink_bytes_per_gpu": nvlink_bytes}


# ------------------------------------------------------------------------------------------------
# CPU baseline / reference arm: the reference's torch path on the host cores
# ------------------------------------------------------------------------------------------------
def cpu_sample(cfg, W, rows, literal=False):
    """One bounded sample of the headline workload on the CPU: gather W shards and multiply
    `rows` rows of the gathered A by B.  literal=False: the oracle (fp32 product of the bf16
    operands).  literal=True: the reference's own calls on CPU tensors -- concatenation as
    all_gather_into_tensor produces it, then torch.mm on the bf16 tensors
    (bench/ag_gemm_bench.py:567-568)."""
    from oracle import tp_gemm_oracle as orc
    K, N = cfg["K"], cfg["N"]
    g = torch.Generator().manual_seed(1)
    per = max(1, rows // W)
    shards = [torch.randn((per, K), generator=g).to(torch.bfloat16) for _ in range(W)]
    b_kn = (torch.randn((K, N), generator=g) * K ** -0.5).to(torch.bfloat16)
    t0 = time.perf_counter()
    if literal:
        c = torch.mm(torch.cat(shards, 0), b_kn)
    else:
        _, c = orc.ag_gemm_ref(shards, b_kn)
    dt = time.perf_counter() - t0
    return 2.0 * per * W * N * K, dt, float(c[0, 0])


def cpu_baseline(cfg, W, budget_s):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    flops, dt, _ = cpu_sample(cfg, W, 64)               # calibration
    rate = flops / max(dt, 1e-6)
    rows = int(min(cfg["M"], max(64, budget_s * rate / (2.0 * cfg["N"] * cfg["K"]))))
    rows = max(W, rows // W * W)
    flops, dt, _ = cpu_sample(cfg, W, rows)
    return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
            "kind": "port",
            "sample": f"{rows} of {cfg['M']} gathered rows x N={cfg['N']} x K={cfg['K']}, "
                      f"fp32 torch.matmul on bf16-rounded operands ({dt:.2f} s)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    W = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cfg = CFG2
    budget = min(3.0, 120.0 / max(1, steps + warmup))   # whole run within a few minutes
    flops, dt, _ = cpu_sample(cfg, W, 256, literal=True)
    rate = flops / max(dt, 1e-6)
    rows = int(min(cfg["M"], max(64, budget * rate / (2.0 * cfg["N"] * cfg["K"]))))
    rows = max(W, rows // W * W)
    for _ in range(warmup):
        cpu_sample(cfg, W, rows, literal=True)
    t_total, f_total = 0.0, 0.0
    for _ in range(steps):
        f, dt, _ = cpu_sample(cfg, W, rows, literal=True)
        t_total += dt
        f_total += f
    value = f_total / t_total / 1e12
    sample = (f"{rows} of {cfg['M']} gathered rows per step x N={cfg['N']} x K={cfg['K']}; "
              "torch.cat + torch.mm on bf16 CPU tensors (the reference's check path run on the host)")
    line = {
        "impl": "reference",
        "metric": "fused AG-GEMM TFLOPS (whole job; GEMM-RS / GEMM-AR under ops)",
        "value": value, "unit": "TFLOP/s", "n_gpus": W, "steps": steps, "warmup": warmup,
        "ms_per_step": t_total / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(W),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--sweep", action="store_true",
                    help="time the M x world-size sweep instead of the headline")
    ap.add_argument("--case", choices=["gemm", "ag", "rs", "ar"],
                    help="run one operator on one GPU a few times (a small case for a profiler)")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=3584)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--case-warmup", type=int, default=2)
    ap.add_argument("--block-n", type=int, default=0)
    ap.add_argument("--cta-pair", type=int, default=None)
    ap.add_argument("--with-cublas", action="store_true")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.sweep:
        run_sweep(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

"""CPU oracle for the tensor-parallel GEMM + collective operators.  TEST INFRASTRUCTURE ONLY:
nothing in the product package imports this file; it is the checker for tests/, for
__graft_entry__.smoke() and for bench.py's CPU baseline.

It restates, in plain torch-on-CPU / numpy, the computation the reference's own check mode
treats as ground truth (the reference has no golden files; its checks compare the fused kernels
with torch.matmul + torch.distributed collectives on seeded inputs):

  AllGather+GEMM    A_full = cat_r(A_r); C = A_full @ B           bench/ag_gemm_bench.py:554-568
  GEMM+ReduceScatter out_r = (sum_s A_s @ B_s^T)[r*M/W:(r+1)*M/W] bench/gemm_rs_bench.py:408-410, 433-435
  GEMM+AllReduce    C = sum_s A_s @ B_s on every rank             bench/gemm_ar_blackwell_bench.py:423-438
  acceptance        three-tier check_close                        bench/common.py:312-367
  TP MLP chain      AG+GEMM(gate, up) -> SwiGLU -> GEMM+RS(down)  the two operators back to back

Arithmetic contract: operands are bf16 values; products and sums are taken in fp32 (or fp64 with
``exact=True``) over the bf16-rounded operands; results are compared before any rounding of the
oracle's output, so the tolerance covers exactly one bf16 rounding plus accumulation order.

Pinning: the reference ships no golden vectors for this path.  This oracle is pinned by
(a) tests/golden/check_close_cases.json, produced by running the reference's own
bench/common.py:check_close (imported from the reference tree, single-process gloo group) on
seeded cases -- see tests/golden/make_golden.py -- and (b) the reference torch path itself
(torch.matmul + gloo collectives) run as processes in tests/test_oracle_gloo.py.  The numeric
outputs of the three operators have no reference-held fixtures: parity of those is "unpinned"
beyond (b).
"""
from __future__ import annotations

import math
from typing import List, Sequence

import numpy as np
import torch

# ---------------------------------------------------------------------------------------------
# bf16 helpers (numpy has no bf16; round-to-nearest-even on the top 16 bits of fp32)
# ---------------------------------------------------------------------------------------------


def bf16_round_np(x: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest bf16 (ties to even), returned as fp32."""
    u = np.asarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32)


def synth_inputs(kind: str, rank: int, world: int, M: int, N: int, K: int, seed: int,
                 sigma_b: float | None = None):
    """Seeded synthetic operands with the distributions of the benchmark configurations:
    A ~ N(0,1), B ~ N(0, sigma_b^2) with sigma_b = 1/sqrt(K_total) unless given; seed + rank.

    kind "ag": A_r [M/W, K], B [K, N] (logical).   kind "rs"/"ar": A_r [M, K], B_r [K, N]
    (K is the per-rank contraction length; sigma uses K * world).
    Returns bf16 tensors on CPU.
    """
    g = torch.Generator().manual_seed(seed + rank)
    if kind == "ag":
        rows, k_total = M // world, K
    else:
        rows, k_total = M, K * world
    if sigma_b is None:
        sigma_b = 1.0 / math.sqrt(k_total)
    A = torch.randn((rows, K), generator=g, dtype=torch.float32)
    B = torch.randn((K, N), generator=g, dtype=torch.float32) * sigma_b
    return A.to(torch.bfloat16), B.to(torch.bfloat16)


def _mm(a: torch.Tensor, b: torch.Tensor, exact: bool) -> torch.Tensor:
    dt = torch.float64 if exact else torch.float32
    return a.to(dt) @ b.to(dt)


# ---------------------------------------------------------------------------------------------
# the three operators
# ---------------------------------------------------------------------------------------------


def ag_gemm_ref(A_shards: Sequence[torch.Tensor], B_kn: torch.Tensor, exact: bool = False):
    """AllGather+GEMM.  A_shards[r]: [M/W, K] bf16; B_kn: [K, N] bf16 (this rank's columns).
    Returns (A_full [M, K] bf16 -- must match the gathered buffer bit for bit,
             C [M, N] fp32/fp64)."""
    A_full = torch.cat(list(A_shards), dim=0)
    return A_full, _mm(A_full, B_kn, exact)


def gemm_rs_ref(A_list: Sequence[torch.Tensor], B_kn_list: Sequence[torch.Tensor],
                exact: bool = False) -> List[torch.Tensor]:
    """GEMM+ReduceScatter.  A_list[s]: [M, K_s]; B_kn_list[s]: [K_s, N].  Returns out[r] =
    rows [r*M/W, (r+1)*M/W) of sum_s A_s @ B_s."""
    W = len(A_list)
    total = None
    for a, b in zip(A_list, B_kn_list):
        p = _mm(a, b, exact)
        total = p if total is None else total + p
    M = total.shape[0]
    assert M % W == 0
    return [total[r * (M // W):(r + 1) * (M // W)] for r in range(W)]


def gemm_ar_ref(A_list: Sequence[torch.Tensor], B_kn_list: Sequence[torch.Tensor],
                exact: bool = False):
    """GEMM+AllReduce.  Returns (C = sum_s A_s @ B_s, [partial_s])."""
    partials = [_mm(a, b, exact) for a, b in zip(A_list, B_kn_list)]
    total = partials[0].clone()
    for p in partials[1:]:
        total = total + p
    return total, partials


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor, block: int = 128) -> torch.Tensor:
    """Row layout the fused SwiGLU epilogue expects for the up-projection weights: blocks of
    `block` gate rows followed by the `block` up rows of the same output columns, so that one
    2*block-wide output tile of the GEMM holds matching gate and up columns.
    w_gate, w_up: [I, K] -> [2I, K].  I must be a multiple of `block`."""
    I, K = w_gate.shape
    assert w_up.shape == (I, K) and I % block == 0
    g = w_gate.view(I // block, block, K)
    u = w_up.view(I // block, block, K)
    return torch.stack((g, u), dim=1).reshape(2 * I, K).contiguous()


def tp_mlp_ref(x_shards: Sequence[torch.Tensor], w_gate_list: Sequence[torch.Tensor],
               w_up_list: Sequence[torch.Tensor], w_down_list: Sequence[torch.Tensor],
               exact: bool = False):
    """The tensor-parallel MLP the two fused operators form back to back (the reference's fused
    gate/up GEMM + SwiGLU epilogue is described at src/dispatch_gemm_glu_combine.cu:21-25; its
    AllGather+GEMM and GEMM+ReduceScatter are the operators above):
        x   = cat_r(x_r)                                  gathered rows, [M, K]
        h_s = silu(x @ w_gate_s^T) * (x @ w_up_s^T)       rank s's columns, [M, I/W], stored bf16
        out = (sum_s h_s @ w_down_s^T)[r*M/W:(r+1)*M/W]   row-scattered, [M/W, N] per rank
    w_gate_s, w_up_s: [I/W, K]; w_down_s: [N, I/W].  Returns (out per rank, [h_s as bf16])."""
    x = torch.cat(list(x_shards), dim=0)
    dt = torch.float64 if exact else torch.float32
    hs, total = [], None
    for wg, wu, wd in zip(w_gate_list, w_up_list, w_down_list):
        g = x.to(dt) @ wg.to(dt).t()
        u = x.to(dt) @ wu.to(dt).t()
        h = (g * torch.sigmoid(g) * u).to(torch.bfloat16)     # h crosses HBM as bf16
        hs.append(h)
        p = h.to(dt) @ wd.to(dt).t()
        total = p if total is None else total + p
    W = len(hs)
    M = total.shape[0]
    assert M % W == 0
    return [total[r * (M // W):(r + 1) * (M // W)] for r in range(W)], hs


# ---------------------------------------------------------------------------------------------
# acceptance
# ---------------------------------------------------------------------------------------------


def check_close_stats(observed: torch.Tensor, expected: torch.Tensor, atol: float = 0.35,
                      rtol: float = 0.08, mean_rtol: float = 0.01) -> dict:
    """The reference's three-tier acceptance (bench/common.py:312-367) on one rank:
    pass if max_abs <= atol, or max_rel <= rtol (denominator clamped at 1e-6), or
    mean_abs <= mean_rtol * mean|expected|."""
    o = observed.detach().float()
    e = expected.detach().float()
    diff = (o - e).abs()
    n = diff.numel()
    max_abs = float(diff.max()) if n else 0.0
    mean_abs = float(diff.mean()) if n else 0.0
    ref_mean = float(e.abs().mean()) if n else 0.0
    max_rel = float((diff / e.abs().clamp_min(1e-6)).max()) if n else 0.0
    bulk_clean = mean_abs <= mean_rtol * max(ref_mean, 1e-6)
    ok = (max_abs <= atol) or (max_rel <= rtol) or bulk_clean
    return {"ok": bool(ok), "max_abs": max_abs, "max_rel": max_rel, "mean_abs": mean_abs,
            "ref_mean": ref_mean, "bulk_clean": bool(bulk_clean)}


def rel_error(observed: torch.Tensor, expected: torch.Tensor,
              rounded_scale: torch.Tensor | None = None) -> float:
    """The build's own acceptance metric: max over elements of
    |observed - expected| / max(|expected|, rms(expected) [, rounded_scale]).

    A plain elementwise relative error is unbounded where the reference crosses zero, so the
    denominator is floored at the RMS of the reference.  For the reduced operators the per-rank
    partial products travel as bf16 (that is the operator contract: the symmetric C buffer is
    bf16), so each partial carries a rounding error of up to 2^-8 of ITS magnitude, which can
    exceed the magnitude of the sum when partials cancel; `rounded_scale` = sum over ranks of
    |partial| per element (everything that was rounded on the way) then floors the denominator
    too, which bounds the metric by 2 * 2^-8 for any world size.  The bound is 1e-2 in every
    case."""
    o = observed.detach().double()
    e = expected.detach().double()
    if e.numel() == 0:
        return 0.0
    rms = float(e.pow(2).mean().sqrt())
    denom = e.abs().clamp_min(max(rms, 1e-30))
    if rounded_scale is not None:
        denom = torch.maximum(denom, rounded_scale.detach().double().abs())
    return float(((o - e).abs() / denom).max())


REL_TOL = 1e-2

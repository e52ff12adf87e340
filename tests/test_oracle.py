"""The CPU oracle against the committed fixtures (tests/golden/, made by make_golden.py from the
reference's own acceptance function and the reference's torch path under gloo)."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import tp_gemm_oracle as orc
from tests.golden.make_golden import SMALL, make_pair

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_check_close_matches_reference_verdicts():
    cases = json.loads((GOLDEN / "check_close_cases.json").read_text())
    assert len(cases) >= 30 and any(c["ok"] for c in cases) and not all(c["ok"] for c in cases)
    for c in cases:
        obs, exp = make_pair(c["seed"], c["rows"], c["cols"], c["noise"], c["outliers"],
                             c["outlier_mag"])
        got = orc.check_close_stats(obs, exp, atol=c["atol"], rtol=c["rtol"])
        assert got["ok"] == c["ok"], (c, got)


def _fixture():
    return np.load(GOLDEN / "torch_path_w2.npz")


def _cmp(fix, key, full: torch.Tensor, tol=2e-5):
    sub = full.float().numpy()[::8, ::8]
    np.testing.assert_allclose(sub, fix[f"{key}_sub"], rtol=tol, atol=tol)
    assert abs(float(full.double().sum()) - float(fix[f"{key}_sum"])) <= 1e-3 * max(1.0, abs(float(fix[f"{key}_sum"])))


def test_oracle_matches_torch_path_fixture():
    fix = _fixture()
    W = 2
    M, N, K = SMALL["M"], SMALL["N"], SMALL["K"]
    ag = [orc.synth_inputs("ag", r, W, M, N, K, seed=1) for r in range(W)]
    for r in range(W):
        a_full, c = orc.ag_gemm_ref([a for a, _ in ag], ag[r][1])
        _cmp(fix, f"r{r}_ag_c", c)
        _cmp(fix, f"r{r}_ag_a_full", a_full, tol=0.0)        # the gather is a copy: bit exact
    rs = [orc.synth_inputs("rs", r, W, M, N, K, seed=2) for r in range(W)]
    outs = orc.gemm_rs_ref([a for a, _ in rs], [b for _, b in rs])
    for r in range(W):
        _cmp(fix, f"r{r}_rs_out", outs[r])
    ar = [orc.synth_inputs("ar", r, W, M, N, K, seed=3) for r in range(W)]
    total, partials = orc.gemm_ar_ref([a for a, _ in ar], [b for _, b in ar])
    for r in range(W):
        _cmp(fix, f"r{r}_ar_out", total)
        _cmp(fix, f"r{r}_ar_partial", partials[r])


def test_fp32_and_fp64_oracles_agree():
    W, M, N, K = 4, 128, 64, 256
    ins = [orc.synth_inputs("ar", r, W, M, N, K, seed=3) for r in range(W)]
    c32, _ = orc.gemm_ar_ref([a for a, _ in ins], [b for _, b in ins])
    c64, _ = orc.gemm_ar_ref([a for a, _ in ins], [b for _, b in ins], exact=True)
    assert orc.rel_error(c32, c64) < 1e-5


def test_bf16_rounding_matches_torch():
    x = torch.randn(10000, generator=torch.Generator().manual_seed(5)) * 37.0
    mine = orc.bf16_round_np(x.numpy())
    theirs = x.to(torch.bfloat16).float().numpy()
    assert np.array_equal(mine, theirs)


def test_rel_error_metric():
    e = torch.tensor([1.0, -2.0, 0.0, 4.0])
    assert orc.rel_error(e, e) == 0.0
    o = e.clone()
    o[2] = 0.01     # reference is exactly zero there: floored by the RMS, not a division by 0
    assert 0 < orc.rel_error(o, e) < 0.01
    assert orc.rel_error(torch.zeros(0), torch.zeros(0)) == 0.0

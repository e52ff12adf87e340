"""Parity of the sm_100a GEMM core with the CPU oracle, through the C ABI (mk_gemm_bf16)."""
import pytest
import torch

from mkernel_b200 import _lib, ops
from oracle import tp_gemm_oracle as orc

pytestmark = pytest.mark.gpu

NK, KN = _lib.MK_B_NK, _lib.MK_B_KN


def run_gemm(M, N, K, layout, block_n=0, seed=7, sigma_b=None):
    dev = torch.device("cuda:0")
    a, b_kn = orc.synth_inputs("ag", 0, 1, M, N, K, seed=seed, sigma_b=sigma_b)
    A = a.to(dev)
    B = (b_kn.t().contiguous() if layout == NK else b_kn.contiguous()).to(dev)
    C = torch.full((M, N), float("nan"), device=dev, dtype=torch.bfloat16)
    status = torch.zeros(4, device=dev, dtype=torch.int32)
    _lib.set_option("block_n", block_n)
    try:
        ops.gemm_bf16(A, B, C, layout, status)
        torch.cuda.synchronize()
    finally:
        _lib.set_option("block_n", 0)
    assert status.tolist() == [0, 0, 0, 0]
    return a, b_kn, C.cpu()


SHAPES = [
    # M, N, K, layout, block_n
    (128, 64, 64, NK, 64), (128, 256, 64, NK, 256), (128, 256, 1024, NK, 256),
    (128, 224, 128, NK, 224), (128, 192, 128, NK, 96), (256, 160, 192, NK, 160),
    (200, 264, 136, NK, 0), (64, 64, 64, NK, 0), (1, 8, 8, NK, 0), (129, 136, 72, NK, 32),
    (1024, 1024, 1024, NK, 0), (384, 640, 4096, NK, 128),
    (128, 64, 64, KN, 64), (128, 256, 128, KN, 256), (256, 512, 512, KN, 0),
    (200, 264, 136, KN, 0), (128, 8192, 1024, KN, 0), (77, 200, 328, KN, 192),
    # a partial last round of tiles, cut along K over all CTAs (pair mode; single-CTA mode;
    # ragged rows and columns in the cut tiles)
    (1280, 4096, 2048, NK, 0), (1152, 4352, 1024, NK, 0), (1250, 4088, 2048, NK, 0),
    (1280, 4096, 2048, KN, 0),
]


@pytest.mark.parametrize("M,N,K,layout,bn", SHAPES)
def test_gemm_matches_oracle(M, N, K, layout, bn):
    a, b_kn, C = run_gemm(M, N, K, layout, bn)
    _, ref = orc.ag_gemm_ref([a], b_kn)
    assert not torch.isnan(C.float()).any()
    assert orc.rel_error(C, ref) <= orc.REL_TOL          # bf16 output of an fp32 accumulation
    assert orc.check_close_stats(C, ref)["ok"]           # the reference's own acceptance


def test_gemm_is_deterministic():
    _, _, c1 = run_gemm(512, 768, 1024, NK)
    _, _, c2 = run_gemm(512, 768, 1024, NK)
    assert torch.equal(c1, c2)


def test_split_last_round_is_deterministic_and_optional():
    """The K-split of a partial last round sums its pieces in a fixed order: two runs agree bit
    for bit; with the option off the whole tiles give the same result within rounding."""
    _, _, c1 = run_gemm(1280, 4096, 2048, NK)
    a, b_kn, c2 = run_gemm(1280, 4096, 2048, NK)
    assert torch.equal(c1, c2)
    _lib.set_option("split_tail", 0)
    try:
        _, _, c3 = run_gemm(1280, 4096, 2048, NK)
    finally:
        _lib.set_option("split_tail", 1)
    _, ref = orc.ag_gemm_ref([a], b_kn)
    assert orc.rel_error(c3, ref) <= orc.REL_TOL
    assert (c1.float() - c3.float()).abs().max() <= 2 ** -6 * ref.abs().max()


def test_gemm_exact_on_small_integers():
    """Products of small integers are exact in fp32 and representable in bf16: bit-exact."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    A = torch.randint(-2, 3, (256, 128), generator=g).to(torch.bfloat16)
    B = torch.randint(-2, 3, (320, 128), generator=g).to(torch.bfloat16)
    C = torch.empty((256, 320), dtype=torch.bfloat16, device=dev)
    ops.gemm_bf16(A.to(dev), B.to(dev), C)
    torch.cuda.synchronize()
    ref = (A.float() @ B.float().t())
    assert ref.abs().max() <= 256                          # exactly representable in bf16
    assert torch.equal(C.cpu().float(), ref)


def test_gemm_linearity_at_headline_size():
    """Size-independent property at the up-projection GEMM shape (8192 x 3584 x 8192):
    scaling A by 2 scales every output by exactly 2 (a power of two commutes with rounding), and
    64 sampled rows agree with the oracle."""
    dev = torch.device("cuda:0")
    M, N, K = 8192, 3584, 8192
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randn((M, K), device=dev, generator=g).to(torch.bfloat16)
    B = (torch.randn((N, K), device=dev, generator=g) / K ** 0.5).to(torch.bfloat16)
    C1 = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
    C2 = torch.empty_like(C1)
    ops.gemm_bf16(A, B, C1)
    ops.gemm_bf16(A * 2, B, C2)
    torch.cuda.synchronize()
    assert torch.equal(C1.float() * 2, C2.float())
    rows = torch.randint(0, M, (64,), generator=torch.Generator().manual_seed(1))
    ref = A[rows.to(dev)].cpu().float() @ B.cpu().float().t()
    assert orc.rel_error(C1[rows.to(dev)].cpu(), ref) <= orc.REL_TOL


def test_rejects_bad_shapes():
    dev = torch.device("cuda:0")
    A = torch.zeros((128, 60), device=dev, dtype=torch.bfloat16)      # K not a multiple of 8
    B = torch.zeros((64, 60), device=dev, dtype=torch.bfloat16)
    C = torch.zeros((128, 64), device=dev, dtype=torch.bfloat16)
    with pytest.raises(_lib.MkError):
        ops.gemm_bf16(A, B, C)
    with pytest.raises(RuntimeError):
        ops.gemm_bf16(A.float(), B, C)

"""The three operators through the reference-shaped Python API on one GPU (world size 1, where
the exchange step is empty), checked against the CPU oracle; plus the bounded-wait path."""
import ctypes

import pytest
import torch

import mkernel_b200
from mkernel_b200 import _lib
from oracle import tp_gemm_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_ag_gemm_world1():
    mod = mkernel_b200.load("ag_gemm_warp_specialized")
    M, N, K = 520, 264, 200        # ragged everywhere (M/W and N padded to 8 by the caller)
    a, b_kn = orc.synth_inputs("ag", 0, 1, M, N, K, seed=1)
    A = mod.DistBuffer((1, M, K), dtype=torch.bfloat16, local_rank=0, local_world_size=1,
                       multicast=True)
    A.data_[0].copy_(a)
    ready = mod.DistBuffer((mod.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                           local_rank=0, local_world_size=1, multicast=True)
    ready.data_.zero_()
    B = b_kn.t().contiguous().to(DEV)
    C = torch.zeros((1, M, N), device=DEV, dtype=torch.bfloat16)
    for _ in range(3):             # re-launch without host resets (the epoch lives on the device)
        C.zero_()
        mod.ag_gemm_warp_specialized_prepare(ready, M, N)
        mod.ag_gemm_warp_specialized_launch(A, ready, B, C)
        torch.cuda.synchronize()
        assert mod.op_status(ready)[0] == 0
        a_full, ref = orc.ag_gemm_ref([a], b_kn)
        assert torch.equal(A.data_.cpu().view(M, K), a_full)          # gathered operand: bit exact
        assert orc.rel_error(C.cpu().view(M, N), ref) <= orc.REL_TOL
    assert int(ready.data_[8]) == 3                                    # device epoch advanced
    assert not A.multicast_enabled                                     # one device: no multicast


def test_gemm_rs_world1_and_graph_replay():
    mod = mkernel_b200.load("gemm_rs_blackwell")
    M, N, K = 384, 512, 320
    a, b_kn = orc.synth_inputs("rs", 0, 1, M, N, K, seed=2)
    A = a.to(DEV)
    B = b_kn.t().contiguous().to(DEV)
    C = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1, multicast=True)
    sync = mod.DistBuffer(mod.gemm_rs_blackwell_sync_shape, dtype=torch.int32, local_rank=0,
                          local_world_size=1, multicast=False)
    mod.gemm_rs_blackwell_prepare(A, B, C, sync)
    torch.cuda.synchronize()
    mod.gemm_rs_blackwell_launch(A, B, C, sync)
    torch.cuda.synchronize()
    ref = orc.gemm_rs_ref([a], [b_kn])[0]
    assert orc.rel_error(C.data_.cpu(), ref) <= orc.REL_TOL
    # The reference's stale-state test (bench/gemm_rs_bench.py:226-242): capture one launch,
    # replay it with A negated in between, never running prepare again.
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        mod.gemm_rs_blackwell_launch(A, B, C, sync)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        mod.gemm_rs_blackwell_launch(A, B, C, sync)
    sign = 1.0
    for _ in range(3):
        A.neg_()
        sign = -sign
        g.replay()
        torch.cuda.synchronize()
        assert orc.rel_error(C.data_.cpu(), sign * ref) <= orc.REL_TOL
    assert mod.op_status(sync)[0] == 0
    assert int(sync.data_[8]) == 5                                     # one epoch per executed launch


@pytest.mark.parametrize("layout", [_lib.MK_B_KN, _lib.MK_B_NK])
def test_gemm_ar_world1(layout):
    mod = mkernel_b200.load("gemm_ar_blackwell")
    M, N, K = 128, 1024, 256        # decode-shaped
    a, b_kn = orc.synth_inputs("ar", 0, 1, M, N, K, seed=3)
    A = a.to(DEV)
    B = (b_kn if layout == _lib.MK_B_KN else b_kn.t()).contiguous().to(DEV)
    C = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1, multicast=True)
    Cf = mod.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1, multicast=True)
    barrier = mod.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=0, local_world_size=1,
                             multicast=True)
    barrier.data_.zero_()
    total, partials = orc.gemm_ar_ref([a], [b_kn])
    for epoch in (1, 2):
        Cf.data_.zero_()
        mod.gemm_ar_intranode_blackwell(A, B, C, barrier, Cf, epoch, layout)
        torch.cuda.synchronize()
        assert orc.rel_error(C.data_.cpu(), partials[0]) <= orc.REL_TOL     # local partial
        assert orc.rel_error(Cf.data_.cpu(), total) <= orc.REL_TOL          # reduced output
    # M outside the reference's {2048..32768} table is an ordinary case here; a negative epoch is
    # an error, and epoch 0 hands the epoch to the device (continues from the last launch)
    with pytest.raises(RuntimeError):
        mod.gemm_ar_intranode_blackwell(A, B, C, barrier, Cf, -1, layout)
    Cf.data_.zero_()
    mod.gemm_ar_intranode_blackwell(A, B, C, barrier, Cf, 0, layout)
    torch.cuda.synchronize()
    assert orc.rel_error(Cf.data_.cpu(), total) <= orc.REL_TOL
    assert int(barrier.data_.view(-1)[8]) == 3


def test_shape_errors_raise():
    mod = mkernel_b200.load("gemm_rs_blackwell")
    A = torch.zeros((256, 64), device=DEV, dtype=torch.bfloat16)
    B = torch.zeros((128, 72), device=DEV, dtype=torch.bfloat16)         # K mismatch
    C = mod.DistBuffer((256, 128), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
    sync = mod.DistBuffer((4096,), dtype=torch.int32, local_rank=0, local_world_size=1)
    with pytest.raises(RuntimeError):
        mod.gemm_rs_blackwell_launch(A, B, C, sync)
    with pytest.raises(RuntimeError):
        mod.gemm_rs_blackwell_prepare(A, B, C, sync)                     # sync buffer too small


def test_wait_that_nothing_satisfies_returns_a_status():
    """Failure detection without a GPU fault: a two-rank reduce-scatter view is built by hand on
    one GPU with a second 'rank' that never runs, so the tile flags of rank 1 are never raised.
    The reduce role's wait must run out, record a status and let the kernel return; the context
    stays usable."""
    lib = _lib.lib()
    M, N, K = 256, 256, 128
    A = torch.randn((M, K), device=DEV).to(torch.bfloat16)
    B = torch.randn((N, K), device=DEV).to(torch.bfloat16)
    c = [torch.zeros((M, N), device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    s = [torch.zeros((_lib.MK_RS_SYNC_WORDS,), device=DEV, dtype=torch.int32) for _ in range(2)]

    def view(bufs):
        v = _lib.SymmView()
        v.rank, v.world, v.bytes = 0, 2, bufs[0].numel() * bufs[0].element_size()
        v.peer[0], v.peer[1] = bufs[0].data_ptr(), bufs[1].data_ptr()
        return v

    cv, sv = view(c), view(s)
    _lib.set_option("wait_limit_ms", 300)
    try:
        rc = lib.mk_gemm_rs_launch(A.data_ptr(), B.data_ptr(), ctypes.byref(cv), ctypes.byref(sv),
                                   M, N, K, None)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()                                        # returns: the wait is bounded
    finally:
        _lib.set_option("wait_limit_ms", 4000)
    out = (ctypes.c_uint32 * 4)()
    rc = lib.mk_op_status(ctypes.byref(sv), out)
    # whichever bounded wait ran out first is recorded: the reduce role waiting for rank 1's tile
    # flags (3), the epilogue waiting for rank 1 to enter the launch before writing into its
    # buffer (5), or a pipeline role starved by one of those (1)
    assert rc == -5 and out[0] in (1, 3, 5), (rc, list(out))
    assert "device wait expired" in _lib.last_error()
    # the context is intact: a fresh launch on the same device computes the right product
    C = torch.empty((M, N), device=DEV, dtype=torch.bfloat16)
    from mkernel_b200 import ops
    ops.gemm_bf16(A, B, C)
    torch.cuda.synchronize()
    assert orc.rel_error(C.cpu(), (A.float() @ B.float().t()).cpu()) <= orc.REL_TOL


def test_multinode_signatures_on_one_gpu():
    """The multi-node style entry points (B stored [K, N], epoch from the caller, transport
    arguments ignored) give the same results as the oracle with a world of one."""
    M, N, K = 256, 192, 320
    ag = mkernel_b200.load("ag_gemm")
    a, b_kn = orc.synth_inputs("ag", 0, 1, M, N, K, seed=1)
    A = ag.DistBuffer((M, K), dtype=torch.bfloat16, local_rank=0, local_world_size=1, multicast=True)
    A.data_.copy_(a)
    barrier = ag.DistBuffer((3, 1024, 1024), dtype=torch.int32, local_rank=0, local_world_size=1)
    barrier.data_.zero_()
    C = torch.zeros((M, N), device=DEV, dtype=torch.bfloat16)
    ag.create_session(0, "127.0.0.1", 0, 0, 0, 0, 0, 0, 0)
    fifo = ag.get_fifo_handles()
    for epoch in (1, 2):
        ag.ag_gemm_multinode(A, b_kn.contiguous().to(DEV), C, barrier, ag.get_recv_buf_ptr(), *fifo,
                             ag.get_arrival_flags_ptr(), epoch, 0, 8, M * K * 2, None, 148, 0, 1)
        torch.cuda.synchronize()
        assert orc.rel_error(C.cpu(), orc.ag_gemm_ref([a], b_kn)[1]) <= orc.REL_TOL
    with pytest.raises(RuntimeError):       # more than one node is not served
        ag.ag_gemm_multinode(A, b_kn.contiguous().to(DEV), C, barrier, 0, *fifo, 0, 3, 0, 8, 0, None,
                             148, 0, 2)

    rs = mkernel_b200.load("gemm_rs")
    a, b_kn = orc.synth_inputs("rs", 0, 1, M, N, K, seed=2)
    work = rs.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
    out = rs.DistBuffer((M, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
    bar2 = rs.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=0, local_world_size=1)
    bar2.data_.zero_()
    rs.gemm_rs_fused(a.to(DEV), b_kn.contiguous().to(DEV), work, out, bar2, None, 0, 0, 0, 0, 0, 0, 0,
                     0, 1, 0, 100, 8, 8, 8, False, 0, None, None, 1)
    torch.cuda.synchronize()
    assert orc.rel_error(out.data_.cpu(), orc.gemm_rs_ref([a], [b_kn])[0]) <= orc.REL_TOL

    ar = mkernel_b200.load("gemm_ar")
    a, b_kn = orc.synth_inputs("ar", 0, 1, 128, N, K, seed=3)
    C3 = ar.DistBuffer((128, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
    C3f = ar.DistBuffer((128, N), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
    bar3 = ar.DistBuffer((2, 1024, 1024), dtype=torch.int32, local_rank=0, local_world_size=1)
    bar3.data_.zero_()
    ar.gemm_ar_multinode(a.to(DEV), b_kn.contiguous().to(DEV), C3, bar3, C3f, 0, 0, 0, 0, 0, 0, 0, 0,
                         1, 0, 8, 0, 0, 1, trace_slot=-1)
    torch.cuda.synchronize()
    assert orc.rel_error(C3f.data_.cpu(), orc.gemm_ar_ref([a], [b_kn])[0]) <= orc.REL_TOL


def test_swiglu_epilogue_and_mlp_chain_world1():
    """AllGather+GEMM(gate, up) with the fused SwiGLU epilogue, then GEMM+ReduceScatter(down), on
    one GPU: H within the tolerance of the oracle's fp32 activation (rounded once to bf16), the
    chain's output within the tolerance of an oracle that also stores H as bf16."""
    from mkernel_b200 import ops
    torch.cuda.set_device(0)
    _mlp_chain_world1(384, 320, 256, 264)
    _mlp_chain_world1(1280, 2048, 2048, 512)     # the gate/up GEMM's last round is cut along K


def _mlp_chain_world1(M, K, I, N):
    from mkernel_b200 import ops
    g = torch.Generator().manual_seed(5)
    x = torch.randn((M, K), generator=g).to(torch.bfloat16)
    wg = (torch.randn((I, K), generator=g) / K ** 0.5).to(torch.bfloat16)
    wu = (torch.randn((I, K), generator=g) / K ** 0.5).to(torch.bfloat16)
    wd = (torch.randn((N, I), generator=g) / I ** 0.5).to(torch.bfloat16)
    mlp = ops.TpMlp(M, K, I, N, 0, 1)
    mlp.load_weights(wg.to(DEV), wu.to(DEV), wd.to(DEV))
    mlp.x.data_[0].copy_(x)
    assert torch.equal(mlp.w_gate_up.cpu(), orc.interleave_gate_up(wg, wu))
    outs, hs = orc.tp_mlp_ref([x], [wg], [wu], [wd])
    for _ in range(2):                      # second pass: epochs advance, nothing is reset
        mlp.h.zero_()
        y = mlp.forward()
        torch.cuda.synchronize()
        assert ops.op_status(mlp.ready)[0] == 0 and ops.op_status(mlp.sync)[0] == 0
        # the activation: fp32 silu(g) * u rounded once to bf16 (fast exp/divide on the device)
        assert orc.rel_error(mlp.h.view(M, I).cpu(), hs[0].float()) <= orc.REL_TOL
        assert orc.rel_error(y.cpu(), outs[0]) <= orc.REL_TOL
    mlp.free()


def test_swiglu_rejects_widths_that_split_a_gate_up_block():
    from mkernel_b200 import ops
    mod = mkernel_b200.load("ag_gemm_warp_specialized")
    A = mod.DistBuffer((1, 128, 64), dtype=torch.bfloat16, local_rank=0, local_world_size=1)
    ready = mod.DistBuffer((mod.ag_gemm_warp_specialized_ready_words,), dtype=torch.int32,
                           local_rank=0, local_world_size=1)
    ready.data_.zero_()
    B = torch.zeros((384, 64), device=DEV, dtype=torch.bfloat16)      # 2I = 384: not 256-aligned
    H = torch.zeros((1, 128, 192), device=DEV, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.ag_gemm_swiglu_launch(A, ready, B, H)

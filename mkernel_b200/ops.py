"""Host-side operator functions with the reference's Python-callable signatures.

Each function checks shapes the way the reference's pybind lambdas do and forwards raw pointers
to the C ABI on the current torch CUDA stream.  References:
  ag_gemm_warp_specialized_prepare/_launch  include/operators/ag_gemm/ag_gemm_warp_specialized_session.cuh:12-47
  gemm_rs_blackwell_prepare/_launch         include/operators/gemm_rs/gemm_rs_blackwell_session.cuh:11-40
  gemm_ar_intranode_blackwell               include/operators/gemm_ar/gemm_ar_blackwell.cuh:205-246
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .dist_buffer import DistBuffer

ag_gemm_warp_specialized_ready_words = _lib.MK_AG_READY_WORDS
gemm_rs_blackwell_sync_shape = (_lib.MK_RS_SYNC_WORDS,)
gemm_ar_blackwell_barrier_shape = (2, 1024, 1024)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current torch CUDA stream of the current device as a raw cudaStream_t."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _on_device:
    """Make `index` the current CUDA device for the duration of a call; free when it already is
    (the common case: one process per GPU), since these wrappers sit on latency-bound paths."""

    __slots__ = ("index", "prev")

    def __init__(self, index):
        self.index = index.index if isinstance(index, torch.device) else int(index)
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _bf16_matrix(t: torch.Tensor, name: str) -> None:
    _require(isinstance(t, torch.Tensor) and t.is_cuda, f"{name} must be a CUDA tensor")
    _require(t.dtype == torch.bfloat16, f"{name} must be bfloat16")
    _require(t.is_contiguous(), f"{name} must be contiguous")


def gemm_bf16(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, b_layout: int = _lib.MK_B_NK,
              status: torch.Tensor | None = None) -> None:
    """C[M,N] = A[M,K] @ B on one GPU; B is [N,K] (MK_B_NK) or [K,N] (MK_B_KN)."""
    for t, n in ((A, "A"), (B, "B"), (C, "C")):
        _bf16_matrix(t, n)
    M, K = A.shape
    N = B.shape[0] if b_layout == _lib.MK_B_NK else B.shape[1]
    kb = B.shape[1] if b_layout == _lib.MK_B_NK else B.shape[0]
    _require(kb == K, f"A and B disagree on K: {K} vs {kb}")
    _require(tuple(C.shape) == (M, N), f"C must be [{M},{N}]")
    with _on_device(A.device):
        _lib.check(_lib.lib().mk_gemm_bf16(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K,
                                           b_layout, status.data_ptr() if status is not None else None,
                                           _stream()))


def ag_gemm_warp_specialized_prepare(A_copy_ready: DistBuffer, M: int = 0, N: int = 0) -> None:
    """All-rank entry barrier + epoch bump on the current stream (M, N kept for compatibility)."""
    _require(isinstance(A_copy_ready, DistBuffer), "A_copy_ready must be a DistBuffer")
    with _on_device(A_copy_ready.local_rank_):
        _lib.check(_lib.lib().mk_ag_gemm_prepare(A_copy_ready.view_ref(), _stream()))


def ag_gemm_warp_specialized_launch(A: DistBuffer, A_copy_ready: DistBuffer, B: torch.Tensor,
                                    C: torch.Tensor) -> None:
    """C[d] = A_shard[d] @ B^T for every shard d.  A: DistBuffer [W, M/W, K]; B: [N, K];
    C: [W, M/W, N]."""
    _require(isinstance(A, DistBuffer) and isinstance(A_copy_ready, DistBuffer),
             "A and A_copy_ready must be DistBuffers")
    _require(A.dtype == torch.bfloat16 and len(A.shape) == 3, "A must be bf16 [W, M/W, K]")
    _bf16_matrix(B, "B")
    _require(C.dtype == torch.bfloat16 and C.is_cuda and C.is_contiguous() and C.dim() == 3,
             "C must be a contiguous bf16 CUDA tensor [W, M/W, N]")
    W, Ms, K = A.shape
    _require(W == A.local_world_size_, "A.shape[0] must equal the local world size")
    N = B.size(0)
    _require(B.size(1) == K, f"B must be [N, K] with K={K}")
    _require(tuple(C.shape) == (W, Ms, N), f"C must be [{W},{Ms},{N}]")
    with _on_device(A.local_rank_):
        _lib.check(_lib.lib().mk_ag_gemm_launch(A.view_ref(), A_copy_ready.view_ref(),
                                                B.data_ptr(), C.data_ptr(), W * Ms, N, K,
                                                _stream()))


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Weight layout of ``ag_gemm_swiglu_launch``: per block of 256 rows, 128 rows of the gate
    projection followed by the 128 rows of the up projection of the same outputs.
    w_gate, w_up: [I, K] with I a multiple of 128 -> [2 I, K]."""
    I, K = w_gate.shape
    _require(tuple(w_up.shape) == (I, K) and I % 128 == 0,
             "w_gate and w_up must both be [I, K] with I a multiple of 128")
    return torch.stack((w_gate.view(I // 128, 128, K), w_up.view(I // 128, 128, K)),
                       dim=1).reshape(2 * I, K).contiguous()


def ag_gemm_swiglu_launch(A: DistBuffer, A_copy_ready: DistBuffer, B_gate_up: torch.Tensor,
                          H: torch.Tensor) -> None:
    """H[d] = silu(A_shard[d] @ G^T) * (A_shard[d] @ U^T) for every shard d: AllGather+GEMM of
    the gate and up projections with the activation fused into the epilogue (the gated
    activation never crosses HBM as [M, 2I]).  A: DistBuffer [W, M/W, K]; B_gate_up: [2I, K] from
    ``interleave_gate_up``; H: [W, M/W, I].  No counterpart call in the reference's TP modules;
    its MoE kernel fuses the same epilogue (src/dispatch_gemm_glu_combine.cu:21-25)."""
    _require(isinstance(A, DistBuffer) and isinstance(A_copy_ready, DistBuffer),
             "A and A_copy_ready must be DistBuffers")
    _require(A.dtype == torch.bfloat16 and len(A.shape) == 3, "A must be bf16 [W, M/W, K]")
    _bf16_matrix(B_gate_up, "B_gate_up")
    W, Ms, K = A.shape
    N2 = B_gate_up.size(0)
    _require(B_gate_up.size(1) == K and N2 % 256 == 0,
             f"B_gate_up must be [2I, K] with K={K} and 2I a multiple of 256")
    _require(H.dtype == torch.bfloat16 and H.is_cuda and H.is_contiguous() and
             tuple(H.shape) == (W, Ms, N2 // 2), f"H must be a contiguous bf16 [{W},{Ms},{N2 // 2}]")
    with _on_device(A.local_rank_):
        _lib.check(_lib.lib().mk_ag_gemm_swiglu_launch(A.view_ref(), A_copy_ready.view_ref(),
                                                       B_gate_up.data_ptr(), H.data_ptr(),
                                                       W * Ms, N2, K, _stream()))


class TpMlp:
    """The tensor-parallel MLP as two fused launches on one stream:
    AllGather+GEMM(gate, up) with the SwiGLU epilogue -> H, then GEMM+ReduceScatter(down) on H.
    Both kernels are launched with programmatic stream serialization (the default), so the
    second one's set-up overlaps the first one's tail; captured in a CUDA graph they are two
    nodes.  All buffers are allocated once, collectively (same order on every rank):
      x:    DistBuffer [W, M/W, K]    rank r fills x.data_[r]
      out:  rows [rank*M/W, (rank+1)*M/W) of y.data_ (the reduced slice)"""

    def __init__(self, M: int, K: int, I_local: int, N_out: int, local_rank: int,
                 local_world_size: int):
        W = int(local_world_size)
        _require(M % W == 0, "M must be divisible by the world size")
        dev = torch.device("cuda", local_rank)
        self.M, self.K, self.I, self.N, self.W, self.rank = M, K, I_local, N_out, W, local_rank
        self.x = DistBuffer((W, M // W, K), torch.bfloat16, local_rank, W)
        self.ready = DistBuffer((ag_gemm_warp_specialized_ready_words,), torch.int32, local_rank, W)
        self.ready.data_.zero_()
        self.h = torch.empty((W, M // W, I_local), device=dev, dtype=torch.bfloat16)
        self.y = DistBuffer((M, N_out), torch.bfloat16, local_rank, W)
        self.sync = DistBuffer(gemm_rs_blackwell_sync_shape, torch.int32, local_rank, W)
        gemm_rs_blackwell_prepare(None, None, self.y, self.sync)
        self.w_gate_up = None
        self.w_down = None

    def load_weights(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> None:
        """w_gate, w_up: [I_local, K]; w_down: [N_out, I_local] (this rank's shards)."""
        self.w_gate_up = interleave_gate_up(w_gate, w_up)
        _bf16_matrix(w_down, "w_down")
        _require(tuple(w_down.shape) == (self.N, self.I), f"w_down must be [{self.N},{self.I}]")
        self.w_down = w_down

    def forward(self) -> torch.Tensor:
        """Enqueue both launches on the current stream; returns the view of this rank's output
        rows (valid when the stream has completed)."""
        ag_gemm_warp_specialized_prepare(self.ready, self.M, 2 * self.I)
        ag_gemm_swiglu_launch(self.x, self.ready, self.w_gate_up, self.h)
        gemm_rs_blackwell_launch(self.h.view(self.M, self.I), self.w_down, self.y, self.sync)
        Ms = self.M // self.W
        return self.y.data_[self.rank * Ms:(self.rank + 1) * Ms]

    def free(self) -> None:
        for b in (self.x, self.ready, self.y, self.sync):
            b.free()


def gemm_rs_blackwell_prepare(A, B, C: DistBuffer, sync: DistBuffer) -> None:
    """Zero the synchronisation words once; the caller then synchronises and barriers."""
    _require(isinstance(sync, DistBuffer), "sync must be a DistBuffer")
    with _on_device(sync.local_rank_):
        _lib.check(_lib.lib().mk_gemm_rs_prepare(sync.view_ref(), _stream()))


def gemm_rs_blackwell_launch(A: torch.Tensor, B: torch.Tensor, C: DistBuffer,
                             sync: DistBuffer) -> None:
    """Partial C = A @ B^T, then rows [rank*M/W, (rank+1)*M/W) of C.data_ hold the sum over ranks."""
    _bf16_matrix(A, "A")
    _bf16_matrix(B, "B")
    _require(isinstance(C, DistBuffer) and isinstance(sync, DistBuffer),
             "C and sync must be DistBuffers")
    M, K = A.shape
    N = B.size(0)
    _require(B.size(1) == K, f"B must be [N, K] with K={K}")
    _require(C.dtype == torch.bfloat16 and tuple(C.shape) == (M, N), f"C must be bf16 [{M},{N}]")
    with _on_device(C.local_rank_):
        _lib.check(_lib.lib().mk_gemm_rs_launch(A.data_ptr(), B.data_ptr(), C.view_ref(),
                                                sync.view_ref(), M, N, K, _stream()))


def gemm_ar_intranode_blackwell(A: torch.Tensor, B: torch.Tensor, C: DistBuffer,
                                barrier: DistBuffer, C_final: DistBuffer, epoch: int,
                                b_layout: int = _lib.MK_B_KN) -> None:
    """C_final = sum over ranks of A_r @ B_r on every rank; C receives this rank's partial."""
    _bf16_matrix(A, "A")
    _bf16_matrix(B, "B")
    for d, n in ((C, "C"), (barrier, "barrier"), (C_final, "C_final")):
        _require(isinstance(d, DistBuffer), f"{n} must be a DistBuffer")
    M, K = A.shape
    if b_layout == _lib.MK_B_KN:
        _require(B.size(0) == K, f"B must be [K, N] with K={K}")
        N = B.size(1)
    else:
        _require(B.size(1) == K, f"B must be [N, K] with K={K}")
        N = B.size(0)
    for d, n in ((C, "C"), (C_final, "C_final")):
        _require(d.dtype == torch.bfloat16 and tuple(d.shape) == (M, N), f"{n} must be bf16 [{M},{N}]")
    _require(int(epoch) >= 0, "epoch starts at 1 and must increase by one per call "
                              "(0 = keep the epoch on the device; graph-replayable)")
    with _on_device(C.local_rank_):
        _lib.check(_lib.lib().mk_gemm_ar_launch(A.data_ptr(), B.data_ptr(), C.view_ref(),
                                                barrier.view_ref(), C_final.view_ref(), M, N, K,
                                                int(epoch), b_layout, _stream()))


def op_status(sync: DistBuffer) -> tuple[int, int, int, int]:
    """Status words of an operator's synchronisation buffer; raises MkError if a device wait
    expired.  Synchronises the device."""
    out = (ctypes.c_uint32 * 4)()
    with _on_device(sync.local_rank_):
        _lib.check(_lib.lib().mk_op_status(sync.view_ref(), out))
    return tuple(int(x) for x in out)


def op_status_clear(sync: DistBuffer) -> None:
    with _on_device(sync.local_rank_):
        _lib.check(_lib.lib().mk_op_status_clear(sync.view_ref(), _stream()))

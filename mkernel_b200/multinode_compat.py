"""Single-node stand-ins for the reference's multi-node operator modules (``ag_gemm``,
``gemm_rs``, ``gemm_ar``): the same function names and argument order, with the RDMA session
functions reduced to no-ops, so that a driver written for those modules runs on one NVSwitch box.

Reference signatures: include/operators/ag_gemm/session.cuh:194-229 (``ag_gemm_multinode``),
include/operators/gemm_rs/session.cuh:105-153 (``gemm_rs_fused``),
include/operators/gemm_ar/session.cuh:163-216 (``gemm_ar_multinode``).

What carries over and what does not:
* Operands, layouts and results are the reference's: A is the node-wide ``DistBuffer`` (AG) or a
  plain tensor, B is ``[K, N]``, epochs come from the caller and must increase by one per call.
* Everything that describes the RDMA transport (FIFO handles, arrival flags, receive/staging
  buffers, SM split hints, proxy tuning) is accepted and ignored; ``num_nodes`` must be 1.
* The reference's ``barrier`` buffers (``(3,1024,1024)`` / ``(2,1024,1024)`` int32) are used as this
  library's synchronisation words.  They must be zeroed once before the first call and not be
  zeroed while a launch is in flight on any rank.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .dist_buffer import DistBuffer
from .ops import _bf16_matrix, _on_device, _require, _stream, gemm_ar_intranode_blackwell

_NO_FIFO = (0, 0, 0, 0, 0)


# ---- session functions: there is no NIC path on one box -------------------------------------
def create_session(*args, **kwargs) -> None:
    """No transport session is needed inside one node; accepted for call compatibility."""
    return None


def destroy_session(*args, **kwargs) -> None:
    return None


def set_epoch(epoch: int) -> None:
    return None


def prepare_epoch(*args, **kwargs) -> None:
    return None


def commit_epoch(*args, **kwargs) -> None:
    return None


def zero_recv_buf(*args, **kwargs) -> None:
    return None


def reset_arrival_flags(*args, **kwargs) -> None:
    return None


def get_fifo_handles():
    return _NO_FIFO


def get_arrival_flags_ptr() -> int:
    return 0


def get_arrival_tails_ptr() -> int:
    return 0


def get_recv_buf_ptr() -> int:
    return 0


def get_num_qps() -> int:
    return 0


def get_proxy_diagnostics() -> dict:
    return {}


def get_proxy_timelines() -> dict:
    return {}


def _single_node(num_nodes: int) -> None:
    _require(int(num_nodes) == 1, "this build drives one NVSwitch node: num_nodes must be 1")


# ---- operators ---------------------------------------------------------------------------------
def ag_gemm_multinode(A: DistBuffer, B: torch.Tensor, C: torch.Tensor, barrier: DistBuffer,
                      recv_buf_ptr=0, fifo_triggers=0, fifo_head=0, fifo_tail=0, fifo_tail_cache=0,
                      fifo_capacity=0, arrival_flags_ptr=0, epoch: int = 1, node_idx: int = 0,
                      num_comm_sms: int = 0, a_half_bytes: int = 0, A_recv=None,
                      active_sms: int = 132, num_intra_comm_override: int = 0,
                      num_nodes: int = 1) -> None:
    """C[M, N] = AllGather(A)[M, K] @ B[K, N].  A: DistBuffer (M, K), rank r has filled rows
    [r*M/W, (r+1)*M/W); barrier: the reference's (3,1024,1024) int32 DistBuffer."""
    _single_node(num_nodes)
    _require(isinstance(A, DistBuffer) and isinstance(barrier, DistBuffer),
             "A and barrier must be DistBuffers")
    _require(A.dtype == torch.bfloat16 and len(A.shape) == 2, "A must be a bf16 DistBuffer (M, K)")
    _bf16_matrix(B, "B")
    _bf16_matrix(C, "C")
    M, K = A.shape
    _require(B.size(0) == K, f"B must be [K, N] with K={K}")
    N = B.size(1)
    _require(tuple(C.shape) == (M, N), f"C must be [{M},{N}]")
    _require(int(epoch) >= 1, "epoch starts at 1")
    with _on_device(A.local_rank_):
        _lib.check(_lib.lib().mk_ag_gemm_launch_ex(A.view_ref(), barrier.view_ref(), B.data_ptr(),
                                                   C.data_ptr(), M, N, K, _lib.MK_B_KN,
                                                   int(epoch), _stream()))


def gemm_rs_fused(A: torch.Tensor, B: torch.Tensor, workspace: DistBuffer, output: DistBuffer,
                  barrier: DistBuffer, ready=None, recv_buf_ptr=0, staging_buf_ptr=0,
                  fifo_triggers=0, fifo_head=0, fifo_tail=0, fifo_tail_cache=0, fifo_capacity=0,
                  arrival_flags_ptr=0, epoch: int = 1, node_idx: int = 0, num_comp_sms: int = 0,
                  num_intra_comm: int = 0, num_send_sms: int = 0, num_reduce_sms: int = 0,
                  use_acquire_poll: bool = False, reduce_poll_sleep_ns: int = 0, ready_chunk=None,
                  staging=None, num_nodes: int = 1) -> None:
    """output[M/W, N] = rows [rank*M/W, (rank+1)*M/W) of sum over ranks of A_r[M, K_r] @ B_r[K_r, N].
    workspace: DistBuffer (M, N) bf16; output: DistBuffer (M/W, N) bf16."""
    _single_node(num_nodes)
    _bf16_matrix(A, "A")
    _bf16_matrix(B, "B")
    for d, n in ((workspace, "workspace"), (output, "output"), (barrier, "barrier")):
        _require(isinstance(d, DistBuffer), f"{n} must be a DistBuffer")
    M, K = A.shape
    _require(B.size(0) == K, f"B must be [K, N] with K={K}")
    N = B.size(1)
    W = workspace.local_world_size_
    _require(tuple(workspace.shape) == (M, N) and workspace.dtype == torch.bfloat16,
             f"workspace must be bf16 ({M},{N})")
    _require(M % W == 0 and tuple(output.shape) == (M // W, N) and output.dtype == torch.bfloat16,
             f"output must be bf16 ({M // W},{N})")
    _require(int(epoch) >= 1, "epoch starts at 1")
    with _on_device(workspace.local_rank_):
        _lib.check(_lib.lib().mk_gemm_rs_launch_ex(A.data_ptr(), B.data_ptr(), workspace.view_ref(),
                                                   barrier.view_ref(), M, N, K, _lib.MK_B_KN,
                                                   int(epoch), _stream()))
        rows = M // W
        output.data_.copy_(workspace.data_.narrow(0, workspace.local_rank_ * rows, rows),
                           non_blocking=True)


def gemm_ar_multinode(A: torch.Tensor, B: torch.Tensor, C: DistBuffer, barrier: DistBuffer,
                      C_final: DistBuffer, staging_buf_ptr=0, recv_buf_ptr=0, fifo_triggers=0,
                      fifo_head=0, fifo_tail=0, fifo_tail_cache=0, fifo_capacity=0,
                      arrival_flags_ptr=0, epoch: int = 1, node_idx: int = 0,
                      num_intra_comm_sms: int = 0, num_inter_comm_sms: int = 0, ar_done_ptr=0,
                      num_nodes: int = 1, **ignored) -> None:
    """C_final[M, N] = sum over ranks of A_r[M, K_r] @ B_r[K_r, N] on every rank."""
    _single_node(num_nodes)
    gemm_ar_intranode_blackwell(A, B, C, barrier, C_final, int(epoch), _lib.MK_B_KN)


_SESSION = ("create_session", "destroy_session", "set_epoch", "get_fifo_handles",
            "get_arrival_flags_ptr", "get_recv_buf_ptr")

EXPORTS = {
    "ag_gemm": _SESSION + ("get_proxy_diagnostics", "get_proxy_timelines", "ag_gemm_multinode"),
    "gemm_rs": _SESSION + ("prepare_epoch", "commit_epoch", "zero_recv_buf", "gemm_rs_fused"),
    "gemm_ar": _SESSION + ("get_proxy_diagnostics", "get_proxy_timelines", "get_arrival_tails_ptr",
                           "reset_arrival_flags", "get_num_qps", "gemm_ar_multinode"),
}

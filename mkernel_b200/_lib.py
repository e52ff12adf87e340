"""ctypes binding of ``libmkernel_b200.so`` (the C ABI in ``include/mkernel_b200.h``).

There is no fallback: if the library is missing, or a call fails, an exception is raised.
Errors map the way the reference's do at its pybind boundary: argument problems become
``RuntimeError`` (the reference raises through ``TORCH_CHECK``); unlike the reference
(common/cuda_checks.cuh:19-36) a CUDA error raises instead of ending the process.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_int, c_longlong, c_size_t, c_uint32,
                    c_void_p)
from pathlib import Path

MK_MAX_WORLD = 8
MK_B_NK = 0
MK_B_KN = 1
MK_AG_READY_WORDS = 65536
MK_RS_SYNC_WORDS = 524288
MK_AR_BARRIER_WORDS = 2 * 1024 * 1024

OP_GEMM, OP_AG, OP_RS, OP_AR = 0, 1, 2, 3

STATUS_NAMES = {
    0: "ok",
    1: "pipeline wait expired",
    2: "gathered rows never arrived",
    3: "a peer's tile flag never arrived",
    4: "a peer never reported completion (exit handshake)",
    5: "a peer never reached the entry barrier",
    6: "a bulk copy never completed",
    7: "AllGather push pacing: this CTA's GEMM never reached the awaited tile",
}


class MkError(RuntimeError):
    """A call into the native library failed; ``code`` is the negative mk_status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"mkernel_b200 error {code}: {message}")
        self.code = code


class SymmView(Structure):
    _fields_ = [
        ("rank", c_int),
        ("world", c_int),
        ("bytes", c_size_t),
        ("peer", c_void_p * MK_MAX_WORLD),
        ("mc", c_void_p),
    ]


class Plan(Structure):
    _fields_ = [(n, c_int) for n in (
        "block_n", "stages", "n_comm", "grid", "smem_bytes", "row_blocks", "col_blocks",
        "k_blocks", "part_rows", "part_blocks", "interleave", "group_rows")] + [
        ("sync_words", c_longlong), ("group_cols", c_int)]


# MKERNEL_B200_LIB selects another build of the same library (the diagnostics build made by
# `python -m mkernel_b200.build --diag`); the reference has the same kind of override for where
# its .so files are taken from (python/load_module.py:19-74, MKERNEL_LOCAL_SO_DIR).
LIB_PATH = Path(os.environ.get("MKERNEL_B200_LIB") or
                Path(__file__).resolve().parent / "libmkernel_b200.so")
_lib = None

_SIGNATURES = {
    "mk_last_error": (c_char_p, []),
    "mk_version": (c_int, []),
    "mk_comm_create": (c_int, [c_char_p, c_int, c_int, c_int, POINTER(c_void_p)]),
    "mk_comm_destroy": (c_int, [c_void_p]),
    "mk_comm_rank": (c_int, [c_void_p]),
    "mk_comm_world": (c_int, [c_void_p]),
    "mk_comm_barrier": (c_int, [c_void_p]),
    "mk_comm_allgather": (c_int, [c_void_p, c_void_p, c_size_t, c_void_p]),
    "mk_comm_allgather_fd": (c_int, [c_void_p, c_int, POINTER(c_int)]),
    "mk_symm_alloc": (c_int, [c_void_p, c_size_t, c_int, POINTER(c_void_p)]),
    "mk_symm_free": (c_int, [c_void_p]),
    "mk_symm_get_view": (c_int, [c_void_p, POINTER(SymmView)]),
    "mk_gemm_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                             c_void_p]),
    "mk_ag_gemm_prepare": (c_int, [POINTER(SymmView), c_void_p]),
    "mk_ag_gemm_launch": (c_int, [POINTER(SymmView), POINTER(SymmView), c_void_p, c_void_p,
                                  c_int, c_int, c_int, c_void_p]),
    "mk_ag_gemm_launch_ex": (c_int, [POINTER(SymmView), POINTER(SymmView), c_void_p, c_void_p,
                                     c_int, c_int, c_int, c_int, c_uint32, c_void_p]),
    "mk_ag_gemm_swiglu_launch": (c_int, [POINTER(SymmView), POINTER(SymmView), c_void_p, c_void_p,
                                         c_int, c_int, c_int, c_void_p]),
    "mk_gemm_rs_launch_ex": (c_int, [c_void_p, c_void_p, POINTER(SymmView), POINTER(SymmView),
                                     c_int, c_int, c_int, c_int, c_uint32, c_void_p]),
    "mk_gemm_rs_prepare": (c_int, [POINTER(SymmView), c_void_p]),
    "mk_gemm_rs_launch": (c_int, [c_void_p, c_void_p, POINTER(SymmView), POINTER(SymmView),
                                  c_int, c_int, c_int, c_void_p]),
    "mk_gemm_rs_launch_noalloc": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_void_p]),
    "mk_gemm_ar_launch": (c_int, [c_void_p, c_void_p, POINTER(SymmView), POINTER(SymmView),
                                  POINTER(SymmView), c_int, c_int, c_int, c_uint32, c_int,
                                  c_void_p]),
    "mk_op_status": (c_int, [POINTER(SymmView), POINTER(c_uint32)]),
    "mk_op_status_clear": (c_int, [POINTER(SymmView), c_void_p]),
    "mk_set_option": (c_int, [c_char_p, c_longlong]),
    "mk_get_option": (c_longlong, [c_char_p]),
    "mk_plan_op": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                           POINTER(Plan)]),
    "mk_sched_tiles": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int),
                               POINTER(c_int), POINTER(c_int), POINTER(c_int), c_int]),
    "mk_sched_work_items": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int),
                                    POINTER(c_int), POINTER(c_int), POINTER(c_int), c_int]),
    "mk_sched_owner_items": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int),
                                     POINTER(c_int), c_int]),
}


def lib() -> ctypes.CDLL:
    """The loaded native library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} does not exist. Build it with `python -m mkernel_b200.build` "
                "(needs nvcc); there is no fallback path.")
        handle = ctypes.CDLL(str(LIB_PATH))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def last_error() -> str:
    msg = lib().mk_last_error()
    return msg.decode(errors="replace") if msg else ""


def check(code: int) -> int:
    if code < 0:
        raise MkError(code, last_error())
    return code


def set_option(name: str, value: int) -> None:
    check(lib().mk_set_option(name.encode(), int(value)))


def get_option(name: str) -> int:
    return int(lib().mk_get_option(name.encode()))


def plan_op(op: int, rank: int, world: int, M: int, N: int, K: int, b_layout: int = MK_B_NK,
            num_sms: int = 148) -> Plan:
    out = Plan()
    check(lib().mk_plan_op(op, rank, world, M, N, K, b_layout, num_sms, ctypes.byref(out)))
    return out


def sched_tiles(op: int, rank: int, world: int, M: int, N: int, block_n: int,
                group_rows: int = 8, group_cols: int = 0):
    """[(row0, rows, col0, rowblock)] in the order the compute CTAs visit the tiles."""
    n = check(lib().mk_sched_tiles(op, rank, world, M, N, block_n, group_rows, group_cols, None,
                                   None, None, None, 0))
    arr = [(c_int * n)() for _ in range(4)]
    check(lib().mk_sched_tiles(op, rank, world, M, N, block_n, group_rows, group_cols, *arr, n))
    return list(zip(*(list(a) for a in arr)))


def sched_owner_items(op: int, world: int, M: int, N: int, block_n: int, owner: int):
    n = check(lib().mk_sched_owner_items(op, world, M, N, block_n, owner, None, None, 0))
    a, b = (c_int * max(n, 1))(), (c_int * max(n, 1))()
    check(lib().mk_sched_owner_items(op, world, M, N, block_n, owner, a, b, n))
    return [(a[i], b[i]) for i in range(n)]


def sched_work_items(total_tiles: int, n_comp: int, cg: int, k_blocks: int, max_parts: int, cta: int):
    """[(tile, kb0, kb1, piece)] of one compute CTA, in order."""
    n = check(lib().mk_sched_work_items(total_tiles, n_comp, cg, k_blocks, max_parts, cta, None,
                                        None, None, None, 0))
    arr = [(c_int * max(n, 1))() for _ in range(4)]
    check(lib().mk_sched_work_items(total_tiles, n_comp, cg, k_blocks, max_parts, cta, *arr, n))
    return [tuple(a[i] for a in arr) for i in range(n)]

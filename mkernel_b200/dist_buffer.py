"""``DistBuffer``: a symmetric device buffer, the Python face of ``mk_symm_alloc``.

Mirrors the class every reference module registers (``dist::ParallelBuffer`` exposed as
``DistBuffer``, include/dist/parallel_buffer.cuh:391-414): same constructor forms, same members
(``data()``, ``data_``, ``multicast_ptr_u64``, ``multicast_enabled``, ``local_rank_``,
``local_world_size_``).  Construction is collective: every local rank must construct its buffers
in the same order.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Sequence, Union

import torch

from . import _lib

_comm = None          # one rendezvous per process, like the reference's single LocalBroker
_comm_params = None


def _default_key() -> str:
    key = os.environ.get("MKB200_BROKER_KEY") or os.environ.get("DIST_BROKER_KEY")
    if key:
        return key
    addr = os.environ.get("MASTER_ADDR", "local")
    port = os.environ.get("MASTER_PORT", str(os.getpid()))
    run = os.environ.get("TORCHELASTIC_RUN_ID", "")
    return f"{addr}:{port}:{run}"


def get_comm(local_rank: int, local_world_size: int) -> ctypes.c_void_p:
    """The process-wide communicator (created on first use)."""
    global _comm, _comm_params
    if _comm is None:
        handle = ctypes.c_void_p()
        _lib.check(_lib.lib().mk_comm_create(_default_key().encode(), local_rank,
                                             local_world_size, local_rank, ctypes.byref(handle)))
        _comm, _comm_params = handle, (local_rank, local_world_size)
    elif _comm_params != (local_rank, local_world_size):
        raise RuntimeError(
            f"DistBuffer: this process already joined as rank/world {_comm_params}, "
            f"got {(local_rank, local_world_size)}")
    return _comm


def host_barrier() -> None:
    """Barrier over the local ranks through the rendezvous sockets (no GPU work)."""
    if _comm is not None:
        _lib.check(_lib.lib().mk_comm_barrier(_comm))


class _DeviceBlob:
    """Exposes a raw device range through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self._owner = owner
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
            "strides": None,
        }


class DistBuffer:
    def __init__(self, shape_or_tensor: Union[Sequence[int], torch.Tensor],
                 dtype: Optional[torch.dtype] = None, local_rank: int = 0,
                 local_world_size: int = 1, multicast: bool = False, backing: str = "vmm"):
        src = None
        if isinstance(shape_or_tensor, torch.Tensor):
            src = shape_or_tensor
            shape, dtype = tuple(src.shape), src.dtype
        else:
            shape = tuple(int(s) for s in shape_or_tensor)
            if dtype is None:
                raise RuntimeError("DistBuffer: dtype is required when a shape is given")
        if backing != "vmm":
            raise RuntimeError(f"DistBuffer: unsupported backing '{backing}' (only 'vmm')")
        if any(s <= 0 for s in shape):
            raise RuntimeError(f"DistBuffer: shape {shape} must be positive")
        self.shape = shape
        self.dtype = dtype
        self.local_rank_ = int(local_rank)
        self.local_world_size_ = int(local_world_size)
        nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        comm = get_comm(self.local_rank_, self.local_world_size_)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.local_rank_):
            _lib.check(_lib.lib().mk_symm_alloc(comm, nbytes, 1 if multicast else 0,
                                                ctypes.byref(handle)))
        self._handle = handle
        self.view = _lib.SymmView()
        _lib.check(_lib.lib().mk_symm_get_view(handle, ctypes.byref(self.view)))
        self.multicast_ptr_u64 = int(self.view.mc or 0)
        self.multicast_enabled = self.multicast_ptr_u64 != 0
        local_ptr = int(self.view.peer[self.local_rank_])
        raw = torch.as_tensor(_DeviceBlob(local_ptr, nbytes, self),
                              device=torch.device("cuda", self.local_rank_))
        self.data_ = raw.view(dtype).view(shape)
        if src is not None:
            self.data_.copy_(src)

    def data(self) -> torch.Tensor:
        return self.data_

    def peer_ptr(self, rank: int) -> int:
        return int(self.view.peer[rank] or 0)

    def view_ref(self):
        return ctypes.byref(self.view)

    def free(self) -> None:
        """Release the allocation.  Collective in effect: no rank may still be using it."""
        h, self._handle = getattr(self, "_handle", None), None
        if h:
            self.data_ = None
            _lib.lib().mk_symm_free(h)

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

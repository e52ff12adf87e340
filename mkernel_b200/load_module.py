"""``load(name)``: the front door of the reference (python/load_module.py:19-74).

The reference imports ``build/lib<name>.so`` as the Python module ``mkernel_release_<name>``.
Here every name resolves to one in-tree native library; ``load`` returns a module object of the
same name carrying the same attributes, so callers written against the reference
(``mod.DistBuffer(...)``, ``mod.ag_gemm_warp_specialized_launch(...)``) run unchanged.
"""
from __future__ import annotations

import sys
import types

from . import _lib, multinode_compat, ops
from .dist_buffer import DistBuffer

_EXPORTS = {
    "ag_gemm_warp_specialized": (
        "ag_gemm_warp_specialized_ready_words",
        "ag_gemm_warp_specialized_prepare",
        "ag_gemm_warp_specialized_launch",
    ),
    "gemm_rs_blackwell": (
        "gemm_rs_blackwell_sync_shape",
        "gemm_rs_blackwell_prepare",
        "gemm_rs_blackwell_launch",
    ),
    "gemm_ar_blackwell": (
        "gemm_ar_intranode_blackwell",
        "gemm_ar_blackwell_barrier_shape",
    ),
}


def names() -> list[str]:
    """Operator module names this library serves."""
    return sorted(list(_EXPORTS) + list(multinode_compat.EXPORTS))


def populate(mod: types.ModuleType, name: str) -> types.ModuleType:
    """Fill `mod` with the attributes of operator module `name`.  Called by ``load`` and by the
    import shims (csrc/loader_shim.c) that the reference's own loader imports as
    ``build/lib<name>.so``."""
    if name not in _EXPORTS and name not in multinode_compat.EXPORTS:
        raise RuntimeError(f"unknown kernel module '{name}'; available: {names()}")
    _lib.lib()  # fail loudly now if the native library is missing
    mod.DistBuffer = DistBuffer
    if name in _EXPORTS:
        for attr in _EXPORTS[name]:
            setattr(mod, attr, getattr(ops, attr))
    else:
        # multi-node style signatures of the same operators, served on one node
        for attr in multinode_compat.EXPORTS[name]:
            setattr(mod, attr, getattr(multinode_compat, attr))
    if name == "gemm_rs_blackwell":
        mod.gemm_rs_blackwell_world_size = _lib.MK_MAX_WORLD
    mod.op_status = ops.op_status
    mod.op_status_clear = ops.op_status_clear
    mod.native_library = str(_lib.LIB_PATH)
    return mod


def load(name: str) -> types.ModuleType:
    """Return the operator module ``mkernel_release_<name>``.

    Raises RuntimeError if the name is not an operator of this library or the native library
    has not been built (same failure mode as the reference when the .so is absent).
    """
    mod_name = f"mkernel_release_{name}"
    mod = types.ModuleType(mod_name, f"B200-native stand-in for build/lib{name}.so")
    populate(mod, name)
    mod.__file__ = str(_lib.LIB_PATH)
    sys.modules[mod_name] = mod
    return mod

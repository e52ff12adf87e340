"""The C-ABI library loads on a machine without a GPU and exports every symbol the public
header declares; argument errors come back as codes + messages, never as a process exit."""
import ctypes
import re
from pathlib import Path

import pytest

from mkernel_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "mkernel_b200.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mk_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    lib = _lib.lib()
    names = declared_symbols()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f"{name} declared in mkernel_b200.h but not exported"


def test_binding_covers_header():
    assert set(declared_symbols()) == set(_lib._SIGNATURES)


def test_version():
    assert _lib.lib().mk_version() >= 100


def test_invalid_arguments_return_codes():
    lib = _lib.lib()
    assert lib.mk_gemm_bf16(None, None, None, 128, 128, 64, 0, None, None) == -1
    assert "null operand" in _lib.last_error()
    assert lib.mk_set_option(b"no_such_option", 1) == -1
    out = ctypes.c_void_p()
    assert lib.mk_comm_create(b"k", 9, 8, 0, ctypes.byref(out)) == -1
    assert lib.mk_comm_create(b"k", 0, 9, 0, ctypes.byref(out)) == -1
    with pytest.raises(_lib.MkError):
        _lib.plan_op(_lib.OP_AG, 0, 8, 8190, 3584, 8192)       # M not divisible by world
    with pytest.raises(_lib.MkError):
        _lib.plan_op(_lib.OP_RS, 0, 8, 8192, 8191, 3584)       # N not a multiple of 8


def test_options_roundtrip():
    assert _lib.get_option("wait_limit_ms") == 4000
    _lib.set_option("wait_limit_ms", 1000)
    assert _lib.get_option("wait_limit_ms") == 1000
    _lib.set_option("wait_limit_ms", 4000)
    with pytest.raises(_lib.MkError):
        _lib.set_option("block_n", -5)
    _lib.set_option("n_comm", 4)
    _lib.set_option("n_comm", -1)          # back to the heuristic
    # only n_comm accepts -1; the device wait budget cannot be configured away
    for name, bad in (("wait_limit_ms", -1), ("wait_limit_ms", 0), ("wait_limit_ms", 10 ** 9),
                      ("ag_lead", -1), ("cta_pair", 2), ("block_n", 512), ("max_stages", 99)):
        with pytest.raises(_lib.MkError):
            _lib.set_option(name, bad)
    assert _lib.get_option("wait_limit_ms") == 4000


def test_environment_options_are_range_checked():
    """MKERNEL_B200_OPTIONS goes through the same validation as mk_set_option: a bad entry is
    reported and skipped, it never disables the bounded waits."""
    import os
    import subprocess
    import sys
    code = ("from mkernel_b200 import _lib; "
            "print(_lib.get_option('wait_limit_ms'), _lib.get_option('block_n'), _lib.get_option('ag_lead'))")
    env = dict(os.environ, MKERNEL_B200_OPTIONS="wait_limit_ms=-1,block_n=128,ag_lead=-1,bogus=3")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True,
                         cwd=str(HEADER.parent.parent), check=True)
    assert out.stdout.split() == ["4000", "128", "6"]
    assert out.stderr.count("ignoring MKERNEL_B200_OPTIONS entry") == 3


def test_debug_flags_exist_only_in_the_diagnostics_build():
    with pytest.raises(_lib.MkError):
        _lib.set_option("debug_flags", 1)


def test_sched_owner_items_rejects_zero_block_n():
    lib = _lib.lib()
    assert lib.mk_sched_owner_items(_lib.OP_RS, 2, 256, 256, 0, 0, None, None, 0) == -1


def test_view_validation_without_gpu():
    lib = _lib.lib()
    v = _lib.SymmView()
    v.rank, v.world, v.bytes = 0, 1, 16
    assert lib.mk_ag_gemm_prepare(ctypes.byref(v), None) == -1      # too small, no address
    v.world = 99
    assert lib.mk_gemm_rs_prepare(ctypes.byref(v), None) == -1


def test_loader_names():
    import mkernel_b200
    mod = mkernel_b200.load("ag_gemm_warp_specialized")
    assert mod.__name__ == "mkernel_release_ag_gemm_warp_specialized"
    assert mod.ag_gemm_warp_specialized_ready_words == _lib.MK_AG_READY_WORDS
    assert callable(mod.ag_gemm_warp_specialized_launch) and hasattr(mod, "DistBuffer")
    mod = mkernel_b200.load("gemm_rs_blackwell")
    assert tuple(mod.gemm_rs_blackwell_sync_shape) == (524288,)
    mod = mkernel_b200.load("gemm_ar_blackwell")
    assert callable(mod.gemm_ar_intranode_blackwell)
    for name, fn in (("ag_gemm", "ag_gemm_multinode"), ("gemm_rs", "gemm_rs_fused"),
                     ("gemm_ar", "gemm_ar_multinode")):
        mod = mkernel_b200.load(name)            # multi-node signatures, served on one node
        assert callable(getattr(mod, fn)) and callable(mod.create_session)
        assert mod.get_fifo_handles() == (0, 0, 0, 0, 0)
    with pytest.raises(RuntimeError):
        mkernel_b200.load("ring_attention")


def test_options_from_environment():
    """MKERNEL_B200_OPTIONS sets start-up defaults; bad entries are reported and skipped."""
    import os
    import subprocess
    import sys
    env = dict(os.environ, MKERNEL_B200_OPTIONS="use_nvls=1,block_n=224,bogus=3,ag_fanout=x")
    code = ("from mkernel_b200 import _lib; "
            "print(_lib.get_option('use_nvls'), _lib.get_option('block_n'), "
            "_lib.get_option('ag_fanout'))")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True,
                         text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["1", "224", "0"]
    assert "bogus=3" in out.stderr and "ag_fanout=x" in out.stderr

"""The reference's front door, exercised without a GPU.

1. The import shims (mkernel_b200/csrc/loader_shim.c, one per operator module) are real CPython
   extensions exporting ``PyInit_mkernel_release_<name>``: they are built here with gcc and
   imported the way the reference's loader imports ``build/lib<name>.so``
   (python/load_module.py:19-74: importlib ``spec_from_file_location`` under the module name
   ``mkernel_release_<name>``).
2. Where a checkout of the reference is present next to this repository, its OWN, unmodified
   ``python/load_module.py`` is imported and pointed at the shim directory; ``load(name)`` must
   return a module with every attribute the reference's bench drivers use.
3. Every call the reference's bench drivers make on a loaded module (``mod.<function>(...)``,
   ``mod.DistBuffer(...)``) is extracted from their source with ``ast`` and bound against this
   library's Python signatures: same names, same arity, same keyword names.
Steps 2 and 3 are skipped where the reference tree is absent (it is never copied into this
repository).
"""
import ast
import importlib.util
import inspect
import os
import sys
from pathlib import Path

import pytest

from mkernel_b200 import build as mkbuild
from mkernel_b200 import load_module

REFERENCE = Path(os.environ.get("MKERNEL_REFERENCE_DIR") or
                 Path(__file__).resolve().parents[2] / "reference")
needs_reference = pytest.mark.skipif(not (REFERENCE / "python" / "load_module.py").exists(),
                                     reason="no checkout of the reference on this machine")


@pytest.fixture(scope="module")
def shim_dir(tmp_path_factory):
    out = tmp_path_factory.mktemp("shims")
    built = mkbuild.build_shims(out)
    assert sorted(p.name for p in built) == sorted(f"lib{n}.so" for n in load_module.names())
    return out


def test_shims_import_like_the_reference_loader(shim_dir):
    for name in load_module.names():
        mod_name = f"mkernel_release_{name}"
        spec = importlib.util.spec_from_file_location(mod_name, shim_dir / f"lib{name}.so")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[mod_name] = mod
        spec.loader.exec_module(mod)
        assert mod.__name__ == mod_name
        assert mod.DistBuffer is load_module.DistBuffer
        assert callable(mod.op_status)
    m = sys.modules["mkernel_release_ag_gemm_warp_specialized"]
    assert m.ag_gemm_warp_specialized_ready_words == 65536
    m = sys.modules["mkernel_release_gemm_rs_blackwell"]
    assert tuple(m.gemm_rs_blackwell_sync_shape) == (524288,)


def _reference_loader():
    spec = importlib.util.spec_from_file_location("reference_load_module",
                                                  REFERENCE / "python" / "load_module.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@needs_reference
def test_reference_loader_loads_the_shims(shim_dir, tmp_path, monkeypatch):
    ref = _reference_loader()
    monkeypatch.setattr(ref, "BUILD", Path(shim_dir))        # where `make` would have put them
    monkeypatch.setenv("MKERNEL_LOCAL_SO_DIR", str(tmp_path / "staged"))
    for name in ("ag_gemm_warp_specialized", "gemm_rs_blackwell", "gemm_ar_blackwell",
                 "ag_gemm", "gemm_rs", "gemm_ar"):
        mod = ref.load(name)
        assert mod.__name__ == f"mkernel_release_{name}"
        assert mod.DistBuffer is load_module.DistBuffer
    assert any((tmp_path / "staged").iterdir())               # the reference staged its copy


def _module_calls(path: Path, receivers=("mod", "mkernel_module", "kernel_mod")):
    """(function name, n positional, keyword names) for every call `<receiver>.<fn>(...)`."""
    tree = ast.parse(path.read_text())
    out = []
    optional = set()        # names the driver itself probes with hasattr(mod, "name")
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Name) and \
                node.func.id == "hasattr" and len(node.args) == 2 and \
                isinstance(node.args[1], ast.Constant):
            optional.add(node.args[1].value)
    for node in ast.walk(tree):
        if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and \
                isinstance(node.func.value, ast.Name) and node.func.value.id in receivers:
            if any(isinstance(a, ast.Starred) for a in node.args):
                n_pos = None                                    # *fifo etc.: arity not static
            else:
                n_pos = len(node.args)
            if node.func.attr not in optional:
                out.append((node.func.attr, n_pos, [k.arg for k in node.keywords if k.arg]))
    return out


BENCH_TO_MODULES = {
    "ag_gemm_bench.py": ("ag_gemm_warp_specialized", "ag_gemm"),
    "gemm_rs_bench.py": ("gemm_rs_blackwell", "gemm_rs"),
    "gemm_ar_blackwell_bench.py": ("gemm_ar_blackwell",),
    "gemm_ar_bench.py": ("gemm_ar",),
}


@needs_reference
@pytest.mark.parametrize("bench", sorted(BENCH_TO_MODULES))
def test_every_call_of_the_reference_benches_binds(bench):
    mods = [load_module.load(n) for n in BENCH_TO_MODULES[bench]]
    calls = _module_calls(REFERENCE / "bench" / bench)
    assert calls, "no module calls found: the extraction is broken"
    checked = 0
    for fn_name, n_pos, kw in calls:
        owners = [m for m in mods if hasattr(m, fn_name)]
        assert owners, f"{bench}: mod.{fn_name} has no counterpart in {BENCH_TO_MODULES[bench]}"
        fn = getattr(owners[0], fn_name)
        if n_pos is None:
            continue
        target = fn.__init__ if inspect.isclass(fn) else fn
        sig = inspect.signature(target)
        args = [object()] * (n_pos + (1 if inspect.isclass(fn) else 0))
        try:
            sig.bind(*args, **{k: object() for k in kw})
        except TypeError as e:
            raise AssertionError(f"{bench}: mod.{fn_name}({n_pos} positional, {kw}) does not bind: {e}")
        checked += 1
    assert checked > 0

"""The drop-in really drops in: with this package's `triton_kernels` imported first, the reference's own
`engine/paging.py`, `engine/cache.py` and `engine/runner.py` import unchanged, and every name they take from
`triton_kernels.*` resolves to an operator of this package.  Needs the reference copy under baseline/_ref
(`python baseline/make_ref.py`); skipped without it."""
import ast
import importlib
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "qwen3_5-triton-inference-engine_b200"
REF = ROOT / "baseline" / "_ref"

needs_ref = pytest.mark.skipif(not (REF / "engine" / "runner.py").exists(), reason="baseline/_ref is absent")


def imported_kernel_names():
    """(module, name) for every `from triton_kernels.X import Y` in the reference's three engine files."""
    found = []
    for rel in ("engine/paging.py", "engine/cache.py", "engine/runner.py"):
        tree = ast.parse((REF / rel).read_text())
        for node in ast.walk(tree):
            if isinstance(node, ast.ImportFrom) and node.module and node.module.startswith("triton_kernels."):
                found += [(node.module, alias.name, rel) for alias in node.names]
    return found


@needs_ref
def test_every_imported_name_resolves_in_the_shim():
    names = imported_kernel_names()
    assert len(names) >= 25, names
    for module, name, rel in names:
        mod = importlib.import_module(module)
        assert Path(mod.__file__).resolve().is_relative_to(PKG), f"{module} resolved outside this package"
        assert hasattr(mod, name), f"{rel}: `from {module} import {name}` does not resolve"


@needs_ref
def test_reference_engine_imports_on_top_of_the_shim():
    """A fresh interpreter, the way INTEGRATION.md describes it: package directory on sys.path, `import triton_kernels`
    (this package's), then the reference's engine modules from their own tree."""
    code = f"""
import sys
sys.path.insert(0, {str(PKG)!r})
import triton_kernels                      # this package's drop-in; must come before the reference's engine
sys.path.insert(1, {str(REF)!r})
import engine.paging, engine.cache, engine.runner
import pathlib, torch
assert pathlib.Path(triton_kernels.__file__).resolve().is_relative_to(pathlib.Path({str(PKG)!r}))
from engine.runner import Qwen35Runner, GraphedDecoder, build_packed_batch
from engine.cache import allocate_caches
from engine.paging import PagePool, SequencePages
import engine.runner as R
for name in ("gemm_2d", "qwen_rmsnorm", "lm_head_argmax", "gdn_recurrent_decode", "partial_rope"):
    fn = getattr(R, name)
    assert "b200attn" in fn.__module__ or "b200attn" in getattr(fn, "_init_fn", fn).__module__, (name, fn.__module__)
pool = PagePool(8)
pages = SequencePages(4, batch=2, device="cpu")
pages.reserve_all(33, pool)
assert pages.block_table.dtype == torch.int32 and pages.block_table.shape == (2, 4)
print("ok")
"""
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.strip().endswith("ok")

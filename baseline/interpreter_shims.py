"""Harness-side shims that let the reference's Triton kernels run on the CPU under ``TRITON_INTERPRET=1`` (Triton 3.6;
the reference files are not modified).  Used by tests/golden/make_golden.py (golden vectors) and by
baseline/run_reference.py (the interpreter leg of the CPU baseline).  Set ``TRITON_INTERPRET=1`` before importing triton.

1. every ``triton.runtime.autotuner.Autotuner`` is pinned to its first config, because the autotuner benchmarks on a
   GPU driver that a CPU run does not have;
2. ``InterpreterBuilder.create_dot`` is replaced by a version that widens bf16 operands to fp32 (the stock interpreter
   multiplies the raw uint16 bit patterns);
3. ``torch.library.wrap_triton`` passes ``InterpretedFunction`` objects through (two GDN chunk kernels have no autotune
   wrapper and would otherwise be rejected);
4. ``InterpreterBuilder.cast_impl`` rounds fp32 -> bf16 to nearest-even, as the GPU's ``cvt.rn.bf16.f32`` does for
   ``.to(tl.bfloat16)`` and for stores through a bf16 pointer (the stock interpreter truncates).
"""
from __future__ import annotations

import numpy as np
import torch


def install_shims() -> None:
    import triton
    import triton.language as tl
    from triton.runtime import interpreter as interp
    from triton.runtime.autotuner import Autotuner

    def create_dot(self, a, b, d, input_precision, max_num_imprecise_acc):
        def widen(h):
            data = h.data
            if h.dtype.scalar == tl.bfloat16 or data.dtype == np.uint16:
                data = (data.astype(np.uint32) << 16).view(np.float32)
            return data

        out = np.matmul(widen(a), widen(b), dtype=d.data.dtype) + d.data
        return interp.TensorHandle(out, d.dtype.scalar)

    interp.InterpreterBuilder.create_dot = create_dot

    original_cast = interp.InterpreterBuilder.cast_impl

    def cast_impl(self, src, dst_type):
        if src.dtype.scalar == tl.float32 and dst_type.scalar == tl.bfloat16:
            bits = np.ascontiguousarray(src.data).view(np.uint32).astype(np.uint64)
            rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
            return interp.TensorHandle(rounded, dst_type.scalar)
        return original_cast(self, src, dst_type)

    interp.InterpreterBuilder.cast_impl = cast_impl

    original_wrap = torch.library.wrap_triton

    def wrap_triton(fn):
        if isinstance(fn, interp.InterpretedFunction):
            return fn
        return original_wrap(fn)

    torch.library.wrap_triton = wrap_triton

    def pin_autotuners():
        import importlib
        import pkgutil

        import triton_kernels

        pinned = 0
        for info in pkgutil.iter_modules(triton_kernels.__path__):
            mod = importlib.import_module(f"triton_kernels.{info.name}")
            for name in dir(mod):
                obj = getattr(mod, name)
                if isinstance(obj, Autotuner) and len(obj.configs) > 1:
                    obj.configs = [obj.configs[0]]
                    pinned += 1
        return pinned

    return pin_autotuners

"""Calling a registered operator without the dispatcher.

Every operator of this package is registered with `torch.library.custom_op` under the reference's `wy_lib::*` name
and schema, which is what `torch.ops.wy_lib.*`, `torch.compile` and fake-tensor tracing need.  An eager caller gains
nothing from the dispatcher and pays about 10 us per call for it - as much as the ctypes call and the launch together,
and a packed prefill of the reference runner is ~400 such calls.  `rebind(namespace)` therefore replaces each operator
object in a module namespace by a function of the same name and signature that calls the implementation directly, and
goes through the registered operator only while `torch.compile` is tracing.
"""
from __future__ import annotations

import functools

import torch


def direct(op):
    """The plain-call form of a `custom_op` object (anything else is returned unchanged)."""
    raw = getattr(op, "_init_fn", None)
    if raw is None or not hasattr(op, "register_fake"):
        return op

    @functools.wraps(raw)
    def call(*args, **kwargs):
        if torch.compiler.is_compiling():
            return op(*args, **kwargs)
        return raw(*args, **kwargs)

    call.op = op           # the registered operator (schema, fake kernel)
    call._init_fn = raw    # the implementation, for callers that look it up the way they would on the operator
    return call


def rebind(namespace: dict) -> None:
    for name, value in list(namespace.items()):
        if hasattr(value, "_init_fn") and hasattr(value, "register_fake"):
            namespace[name] = direct(value)

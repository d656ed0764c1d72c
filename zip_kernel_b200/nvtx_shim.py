"""Environment-gated NVTX ranges around the operator entry points.

Counterpart of the reference's ``tools/profile/nvtx_shim.py:30-70`` (same
switch: ``HKUST_V9_PROFILE=1``; same range names as its call sites in
``cuda_kernel/ops.py:229,344,399,584,633,733``), so a timeline taken with this
library lines up with one taken with the reference.  With the switch off the
operators are returned undecorated: the hot path pays nothing.
"""

from __future__ import annotations

import functools
import os

ENABLED: bool = os.environ.get("HKUST_V9_PROFILE", "0") == "1"


class _Range:
    """``with nvtx_range(name):`` - a real range when profiling is on."""

    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch.cuda.nvtx as nvtx
        nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        import torch.cuda.nvtx as nvtx
        nvtx.range_pop()
        return False


class _NoRange:
    __slots__ = ()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_RANGE = _NoRange()


def nvtx_range(name: str):
    return _Range(name) if ENABLED else _NO_RANGE


def range_push(name: str) -> None:
    if ENABLED:
        import torch.cuda.nvtx as nvtx
        nvtx.range_push(name)


def range_pop() -> None:
    if ENABLED:
        import torch.cuda.nvtx as nvtx
        nvtx.range_pop()


def traced(name: str):
    """Decorator: run the function inside the NVTX range ``name`` when profiling
    is on; hand the function back untouched when it is off."""
    def wrap(fn):
        if not ENABLED:
            return fn

        @functools.wraps(fn)
        def inner(*a, **kw):
            with _Range(name):
                return fn(*a, **kw)
        return inner
    return wrap


__all__ = ["ENABLED", "nvtx_range", "range_push", "range_pop", "traced"]

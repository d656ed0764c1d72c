"""Backend policy shims.

The reference chooses between a Triton and a CUDA implementation per kernel and
shape (``backend/policy.py:71-155,194-254``).  This build has one backend, so the
policy only validates what it is given and reports status; the setters are kept
so that code written against the reference keeps working.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Union

from .registry import ALL_KERNELS, BackendKernel


@dataclass(frozen=True)
class ShapeContext:
    """Shape descriptor handed to custom policies (reference: policy.py:47-62)."""

    T: int = -1
    d_out: int = -1
    d_in: int = -1
    n_hp_blocks: int = 0
    n_groups: int = -1


PolicyFn = Callable[[str, ShapeContext], str]

_NAMES = ("auto", "cuda")
_active = "auto"


def set_backend_policy(policy: Union[str, PolicyFn, Dict[str, str]]) -> None:
    """Accepts the reference's forms.  ``'auto'`` and ``'cuda'`` select the only
    backend; asking for ``'triton'`` (by name or per kernel) raises."""
    global _active
    if isinstance(policy, str):
        key = policy.lower()
        if key == "triton":
            raise ValueError("this build has no Triton backend")
        if key not in _NAMES:
            raise ValueError(f"Unknown backend policy name {policy!r}; expected one of {sorted(_NAMES)}")
        _active = key
        return
    if isinstance(policy, dict):
        for k, v in policy.items():
            if k not in ALL_KERNELS:
                raise ValueError(f"Unknown kernel name {k!r} in policy dict")
            if v != "cuda":
                raise ValueError(f"Policy value for {k!r} must be 'cuda' in this build, got {v!r}")
        _active = "cuda"
        return
    if callable(policy):
        _active = getattr(policy, "__name__", "custom")
        return
    raise TypeError(f"Policy must be str, dict, or callable; got {type(policy).__name__}")


def current_policy() -> str:
    return _active


def get_backend_status() -> Dict[str, object]:
    """Diagnostic dict with the reference's keys (policy.py:262-273)."""
    return {
        "cuda_available": BackendKernel.cuda_available(),
        "cuda_import_error": BackendKernel.cuda_import_error(),
        "cuda_kernels": list(BackendKernel.cuda_available_kernels()),
        "active_policy": _active,
    }


__all__ = ["ShapeContext", "PolicyFn", "set_backend_policy", "current_policy", "get_backend_status"]

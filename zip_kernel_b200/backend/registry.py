"""Kernel registry of the W4A4 linear.

Interface of the reference's ``backend/registry.py`` (kernel names :34-44,
``BackendKernel`` facade :117-180): callers look kernels up by the canonical
names and get the callable ``<name>_cuda`` of the operator module.  There is a
single backend here (hand-written sm_100a CUDA behind the C ABI); nothing falls
back to Triton or to the CPU, so a missing library is an import error and not a
silent downgrade.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Optional

KERNEL_ACTIVATION_QUANT = "activation_quant"
KERNEL_DENSE_GEMM = "dense_gemm"
KERNEL_SPARSE_GEMM = "sparse_gemm"
KERNEL_FUSED_DENSE_SPARSE = "fused_dense_sparse"

ALL_KERNELS = (
    KERNEL_ACTIVATION_QUANT,
    KERNEL_DENSE_GEMM,
    KERNEL_SPARSE_GEMM,
    KERNEL_FUSED_DENSE_SPARSE,
)

_cuda_impls: Dict[str, Callable[..., Any]] = {}
_cuda_import_error: Optional[str] = None


def _load_cuda_backend() -> None:
    """Populate the table from ``zip_kernel_b200.ops`` by attribute name, as the
    reference does with ``cuda_kernel.ops`` (registry.py:88-97)."""
    global _cuda_import_error
    try:
        from .. import ops as cuda_ops
    except Exception as exc:  # the library is missing or does not load
        _cuda_import_error = f"{type(exc).__name__}: {exc}"
        return
    for name in ALL_KERNELS:
        fn = getattr(cuda_ops, f"{name}_cuda", None)
        if callable(fn):
            _cuda_impls[name] = fn


_load_cuda_backend()


class BackendKernel:
    """Static facade over the kernel table (reference: registry.py:117-180)."""

    @staticmethod
    def cuda_available() -> bool:
        return len(_cuda_impls) > 0

    @staticmethod
    def cuda_available_kernels() -> tuple:
        return tuple(sorted(_cuda_impls.keys()))

    @staticmethod
    def cuda_import_error() -> Optional[str]:
        return _cuda_import_error

    @staticmethod
    def cuda_impl(name: str) -> Optional[Callable[..., Any]]:
        return _cuda_impls.get(name)

    @staticmethod
    def triton_impl(name: str) -> Callable[..., Any]:
        raise RuntimeError("this build has no Triton backend; use BackendKernel.cuda_impl")

    @staticmethod
    def _require(name: str) -> Callable[..., Any]:
        fn = _cuda_impls.get(name)
        if fn is None:
            raise RuntimeError(
                f"kernel {name!r} is unavailable: {_cuda_import_error or 'not exported by the operator module'}"
            )
        return fn

    @staticmethod
    def activation_quant(*args, **kwargs):
        return BackendKernel._require(KERNEL_ACTIVATION_QUANT)(*args, **kwargs)

    @staticmethod
    def dense_gemm(*args, **kwargs):
        return BackendKernel._require(KERNEL_DENSE_GEMM)(*args, **kwargs)

    @staticmethod
    def sparse_gemm(*args, **kwargs):
        return BackendKernel._require(KERNEL_SPARSE_GEMM)(*args, **kwargs)

    @staticmethod
    def fused_dense_sparse(*args, **kwargs):
        return BackendKernel._require(KERNEL_FUSED_DENSE_SPARSE)(*args, **kwargs)


__all__ = [
    "BackendKernel",
    "ALL_KERNELS",
    "KERNEL_ACTIVATION_QUANT",
    "KERNEL_DENSE_GEMM",
    "KERNEL_SPARSE_GEMM",
    "KERNEL_FUSED_DENSE_SPARSE",
]

"""Public API of the W4A4 linear, with the names of the reference's
``backend/__init__.py`` (:102-121).  ``weight_loader`` is pure PyTorch and always
importable; the forward entry points need the CUDA library and raise at call
time if it is missing.
"""

from __future__ import annotations

from .weight_loader import (CutlassPackValidationError, CutlassV9Tensors,
                            pack_v9_weights_for_cutlass)
from .graph_cache import (clear_cuda_graph_cache, cuda_graph_cache_stats, get_cuda_graph_policy,
                          prewarm_cuda_graph_cache, set_cuda_graph_policy,
                          v9_linear_forward_cuda_graph, v9_linear_forward_host_graph,
                          v9_linear_forward_host_graph_many, v9_linear_host_batch_graph, HostBatchGraph)
from .policy import get_backend_status, set_backend_policy
from .registry import BackendKernel


def _forward_module():
    from .. import v9_linear
    return v9_linear


def v9_linear_forward(X_fp16, W):
    return _forward_module().v9_linear_forward(X_fp16, W)


def v9_linear_forward_decode(X_fp16, W):
    return _forward_module().v9_linear_forward_decode(X_fp16, W)


def v9_linear_forward_prefill(X_fp16, W):
    return _forward_module().v9_linear_forward_prefill(X_fp16, W)


def v9_linear_fakequant(X_fp16, W):
    return _forward_module().v9_linear_fakequant(X_fp16, W)


__all__ = [
    "v9_linear_forward",
    "v9_linear_forward_decode",
    "v9_linear_forward_prefill",
    "v9_linear_fakequant",
    "set_backend_policy",
    "get_backend_status",
    "BackendKernel",
    "v9_linear_forward_cuda_graph",
    "v9_linear_forward_host_graph",
    "v9_linear_forward_host_graph_many",
    "v9_linear_host_batch_graph",
    "HostBatchGraph",
    "set_cuda_graph_policy",
    "get_cuda_graph_policy",
    "prewarm_cuda_graph_cache",
    "cuda_graph_cache_stats",
    "clear_cuda_graph_cache",
    "pack_v9_weights_for_cutlass",
    "CutlassV9Tensors",
    "CutlassPackValidationError",
]

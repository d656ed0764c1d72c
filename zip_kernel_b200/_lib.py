"""ctypes binding of libw4a4_b200.so (the C ABI declared in include/w4a4_b200.h).

There is no fallback: if the library has not been built, importing the operator
layer raises.  ``python -m zip_kernel_b200.build`` (or ``__graft_entry__.build``)
produces it.
"""

from __future__ import annotations

import contextlib
import ctypes
import os
import threading
from typing import Dict, Tuple

import torch

from .build import LIB_PATH

_c = ctypes
_PTR = _c.c_void_p
_INT = _c.c_int
_LL = _c.c_longlong
_SZ = _c.c_size_t

# name -> (restype, argtypes); must list every symbol of include/w4a4_b200.h
SIGNATURES = {
    "w4a4_abi_version": (_INT, []),
    "w4a4_status_string": (_c.c_char_p, [_INT]),
    "w4a4_last_error": (_c.c_char_p, []),
    "w4a4_device_error": (_INT, [_c.POINTER(_INT), _PTR]),
    "w4a4_selftest_bounded_wait": (_INT, [_INT, _PTR]),
    "w4a4_activation_quant": (_INT, [_PTR, _LL, _PTR, _PTR, _PTR, _PTR, _INT, _INT, _PTR]),
    "w4a4_rmsnorm_quant": (_INT, [_PTR, _LL, _PTR, _c.c_float] + [_PTR] * 6 + [_INT, _INT, _INT, _PTR]),
    "w4a4_silu_mul_quant": (_INT, [_PTR, _LL] + [_PTR] * 6 + [_INT, _INT, _INT, _PTR]),
    "w4a4_peer_alloc": (_INT, [_SZ, _c.POINTER(_PTR)]),
    "w4a4_peer_free": (_INT, [_PTR]),
    "w4a4_peer_export": (_INT, [_PTR, _PTR]),
    "w4a4_peer_open": (_INT, [_PTR, _c.POINTER(_PTR)]),
    "w4a4_peer_close": (_INT, [_PTR]),
    "w4a4_peer_push_wait": (_INT, [_PTR, _LL, _c.POINTER(_PTR), _c.POINTER(_PTR), _LL, _LL, _INT, _INT, _INT, _INT, _PTR, _INT, _PTR]),
    "w4a4_workspace_bytes": (_SZ, [_INT, _INT, _INT, _INT]),
    "w4a4_fused_dense_sparse": (_INT, [_PTR] * 10 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_expanded_codes_bytes": (_SZ, [_INT, _INT]),
    "w4a4_expanded_sums_bytes": (_SZ, [_INT, _INT]),
    "w4a4_expand_activations": (_INT, [_PTR] * 4 + [_INT, _INT, _PTR]),
    "w4a4_fused_dense_sparse_expanded": (_INT, [_PTR] * 10 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_dense_gemm": (_INT, [_PTR] * 7 + [_INT] * 4 + [_PTR, _SZ, _PTR]),
    "w4a4_sparse_gemm": (_INT, [_PTR] * 7 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_fused_quant_dense_sparse": (_INT, [_PTR, _LL] + [_PTR] * 8 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_fused_dense_sparse_noalloc": (_INT, [_PTR] * 10 + [_INT] * 5 + [_PTR]),
    "w4a4_dump_accumulators": (_INT, [_PTR] * 7 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_dequant_weights_fp16": (_INT, [_PTR] * 4 + [_INT, _INT, _PTR]),
    "w4a4_prepared_weights_bytes": (_SZ, [_SZ]),
    "w4a4_prepare_weights": (_INT, [_PTR, _PTR, _SZ, _PTR]),
    "w4a4_fused_dense_sparse_prepared": (_INT, [_PTR] * 12 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_fused_quant_dense_sparse_prepared": (_INT, [_PTR, _LL] + [_PTR] * 10 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_expand_activations_fmt": (_INT, [_PTR] * 4 + [_INT, _INT, _INT, _PTR]),
    "w4a4_fused_dense_sparse_expanded_prepared": (_INT, [_PTR] * 12 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
    "w4a4_dump_accumulators_prepared": (_INT, [_PTR] * 9 + [_INT] * 5 + [_PTR, _SZ, _PTR]),
}

FLAG_OUT_TOKEN_MAJOR = 0x1
FLAG_FORCE_STREAM = 0x2
FLAG_FORCE_TENSOR = 0x4
FLAG_CODES_E4M3 = 0x8
FLAG_CODES_E4M3_PACKED = 0x10
CODES_S8, CODES_E4M3, CODES_E4M3_PACKED = 0, 1, 2

_lib = None


class W4A4Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, where: str, detail: str):
        self.status = status
        super().__init__(f"{where} failed with status {status}: {detail}")


def load() -> ctypes.CDLL:
    """Load the shared library once and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("W4A4_B200_LIB", LIB_PATH)
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m zip_kernel_b200.build` "
            "(needs nvcc; there is no CPU fallback)"
        )
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.w4a4_abi_version() != 1:
        raise RuntimeError("libw4a4_b200.so ABI version mismatch")
    _lib = lib
    return lib


def check(status: int, where: str) -> None:
    """Translate a status code into the exception class the reference raises:
    argument problems become ValueError, everything else RuntimeError."""
    if status == 0:
        return
    lib = load()
    detail = (lib.w4a4_last_error() or b"").decode() or lib.w4a4_status_string(status).decode()
    if status == 1:
        raise ValueError(f"{where}: {detail}")
    raise W4A4Error(status, where, detail)


def ptr(t) -> int:
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else t.data_ptr()


_raw_current_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_NO_SWITCH = contextlib.nullcontext()


def stream_ptr(device) -> int:
    """Handle of the current stream of ``device`` (the capture stream during a graph capture)."""
    if _raw_current_stream is not None:
        idx = getattr(device, "index", device)
        return _raw_current_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


def on_device(device):
    """Context that makes ``device`` current; free when it already is (a torch.cuda.device block costs
    several microseconds per eager call otherwise)."""
    idx = device.index
    if idx is None or idx == torch.cuda.current_device():
        return _NO_SWITCH
    return torch.cuda.device(device)


# ---------------------------------------------------------------------------
# workspace cache: one scratch buffer per (device, stream), grown on
# demand.  Calls issued on one stream are ordered, so they can share scratch.
#
# A captured CUDA graph bakes the scratch address into its kernel nodes, so a
# graph must own the scratch it was captured with: a buffer from the shared
# cache could be replaced (and freed) by a later, larger call on a stream that
# happens to reuse the same handle, and the graph would then replay into freed
# memory.  Code that captures wraps warm-up and capture in
# ``use_workspace(holder)`` and keeps ``holder`` alive next to the graph.
# ---------------------------------------------------------------------------
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_tls = threading.local()


class WorkspaceHolder:
    """Scratch buffers private to one captured graph (or one group of graphs that
    are never replayed concurrently).  Buffers are only ever added: a buffer that a
    captured kernel may reference is never freed or replaced while the holder lives."""

    def __init__(self):
        self.buffers: Dict[Tuple[int, int], list] = {}

    def get(self, key: Tuple[int, int], need: int, device: torch.device) -> torch.Tensor:
        bufs = self.buffers.setdefault(key, [])
        if bufs and bufs[-1].numel() >= need:
            return bufs[-1]
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                "the W4A4 workspace must be allocated before CUDA-graph capture: "
                "run the shape once eagerly inside use_workspace(holder) first"
            )
        buf = torch.empty(max(need, 256), dtype=torch.uint8, device=device)
        bufs.append(buf)
        return buf

    def nbytes(self) -> int:
        return sum(b.numel() for bufs in self.buffers.values() for b in bufs)


@contextlib.contextmanager
def use_workspace(holder: WorkspaceHolder):
    """Route this thread's workspace requests to ``holder`` for the duration of the block."""
    prev = getattr(_tls, "holder", None)
    _tls.holder = holder
    try:
        yield holder
    finally:
        _tls.holder = prev


def workspace(device: torch.device, T: int, K: int, N: int, nnz: int) -> torch.Tensor:
    lib = load()
    need = int(lib.w4a4_workspace_bytes(T, K, N, nnz))
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           stream_ptr(device))
    holder = getattr(_tls, "holder", None)
    if holder is not None:
        return holder.get(key, need, device)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < need:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError(
                "the W4A4 workspace must be allocated before CUDA-graph capture: "
                "run the shape once eagerly (or call zip_kernel_b200.ops.reserve_workspace)"
            )
        grow = max(need, int(buf.numel() * 1.5) if buf is not None else 0)
        buf = torch.empty(grow, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def device_error(device) -> int:
    """Read and clear the device error word (synchronises the current stream)."""
    lib = load()
    word = _INT(0)
    lib.w4a4_device_error(ctypes.byref(word), stream_ptr(device))
    return int(word.value)

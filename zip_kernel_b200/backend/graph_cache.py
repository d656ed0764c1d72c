"""CUDA-graph replay cache for the module-level forward.

Interface of the reference's ``backend/graph_cache.py``
(``v9_linear_forward_cuda_graph`` :355-407, ``set_cuda_graph_policy`` :566-582,
``get_cuda_graph_policy`` :585-587, ``prewarm_cuda_graph_cache`` :590-631,
``cuda_graph_cache_stats`` :634-636, ``clear_cuda_graph_cache`` :639-641): an
LRU cache of captured graphs keyed on the weight container's identity and the
activation's shape / dtype / strides / device, with weak-reference eviction when
a container dies and a sentinel entry after a failed capture so capture is not
retried on every call.

Decode-sized linears run for a few microseconds on a B200, so the Python and
launch overhead of the eager path dominates; replaying one graph per (shape,
weight) removes it.  The kernels behind the forward never allocate or
synchronise, and the scratch buffer is reserved before capture, so the eager
call is capturable as is.
"""

from __future__ import annotations

import logging
import threading
import time
import weakref
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..pack_utils import V9WeightContainer

logger = logging.getLogger(__name__)

DECODE_T_THRESHOLD = 128
_POLICY_LEGAL = ("off", "auto", "force")
_AUTO_T_BUCKETS = frozenset({1, 2, 4, 8, 16, 32, 64, 128})
_DEFAULT_CAPACITY = 64
_policy = "off"


@dataclass(frozen=True)
class _CacheKey:
    """Everything a captured graph bakes in (reference: graph_cache.py:142-188)."""
    w_id: int
    x_shape: Tuple[int, ...]
    x_dtype: str
    x_stride: Tuple[int, ...]
    x_contiguous: bool
    device_index: int


@dataclass
class _CacheEntry:
    key: _CacheKey
    T: int
    d_in: int
    d_out: int
    n_hp_blocks: int
    graph: Optional[Any] = None          # None after a failed capture (sentinel)
    x_static: Optional[torch.Tensor] = None
    y_static: Optional[torch.Tensor] = None
    scratch: Optional[Any] = None        # the scratch buffers the captured kernels write (owned by this entry)
    capture_us: float = 0.0
    replay_count: int = 0
    _finalizer: Optional[weakref.finalize] = None

    def release(self) -> None:
        self.graph = None
        self.x_static = None
        self.y_static = None
        self.scratch = None
        if self._finalizer is not None and self._finalizer.alive:
            self._finalizer.detach()


def _device_index(X) -> int:
    dev = getattr(X, "device", None)
    idx = getattr(dev, "index", None)
    return int(idx) if idx is not None else 0


def _build_cache_key(X, W) -> _CacheKey:
    return _CacheKey(
        w_id=id(W),
        x_shape=tuple(int(s) for s in X.shape),
        x_dtype=str(X.dtype),
        x_stride=tuple(int(s) for s in X.stride()),
        x_contiguous=bool(X.is_contiguous()),
        device_index=_device_index(X),
    )


class _GraphCache:
    """Thread-safe LRU of :class:`_CacheEntry` with hit/miss/eviction counters."""

    def __init__(self, capacity: int = _DEFAULT_CAPACITY):
        self.capacity = int(capacity)
        self._entries: "OrderedDict[_CacheKey, _CacheEntry]" = OrderedDict()
        self._lock = threading.RLock()
        self.hits = self.misses = self.evictions = self.capture_failures = self.weak_evictions = 0

    def get(self, key: _CacheKey) -> Optional[_CacheEntry]:
        with self._lock:
            e = self._entries.get(key)
            if e is None:
                self.misses += 1
                return None
            self._entries.move_to_end(key)
            self.hits += 1
            return e

    def put(self, key: _CacheKey, entry: _CacheEntry, weight_ref_target=None) -> None:
        with self._lock:
            old = self._entries.pop(key, None)
            if old is not None:
                old.release()
            self._entries[key] = entry
            if entry.graph is None:
                self.capture_failures += 1
            if weight_ref_target is not None:
                try:
                    entry._finalizer = weakref.finalize(weight_ref_target, _on_weight_dead,
                                                        weakref.ref(self), key)
                except TypeError:      # object without weak-reference support
                    entry._finalizer = None
            while len(self._entries) > self.capacity:
                _, victim = self._entries.popitem(last=False)
                victim.release()
                self.evictions += 1

    def drop(self, key: _CacheKey, weak: bool = False) -> None:
        with self._lock:
            e = self._entries.pop(key, None)
            if e is not None:
                e.release()
                if weak:
                    self.weak_evictions += 1

    def clear(self) -> None:
        with self._lock:
            for e in self._entries.values():
                e.release()
            self._entries.clear()

    def __len__(self) -> int:
        with self._lock:
            return len(self._entries)

    def stats(self) -> Dict[str, Any]:
        with self._lock:
            return {
                # the reference's key names (backend/graph_cache.py:278-288) ...
                "n_entries": len(self._entries), "max_entries": self.capacity, "n_hit": self.hits,
                "n_miss": self.misses, "n_evict": self.evictions, "n_capture_fail": self.capture_failures,
                # ... and this library's own
                "policy": _policy, "size": len(self._entries), "capacity": self.capacity,
                "hits": self.hits, "misses": self.misses, "evictions": self.evictions,
                "weak_evictions": self.weak_evictions, "capture_failures": self.capture_failures,
                "replays": sum(e.replay_count for e in self._entries.values()),
            }


def _on_weight_dead(cache_ref, key: _CacheKey) -> None:
    cache = cache_ref()
    if cache is not None:
        cache.drop(key, weak=True)


_cache = _GraphCache()


def _is_eligible(X, W, T: int) -> bool:
    """Whether the active policy lets this call use a graph; False is always safe."""
    if _policy == "off":
        return False
    if T < 1 or T > DECODE_T_THRESHOLD:
        return False
    if _policy == "force":
        return True
    return T in _AUTO_T_BUCKETS


def _eager(X, W):
    from ..v9_linear import v9_linear_forward
    return v9_linear_forward(X, W)


def _flat_T(X) -> Optional[int]:
    if X.dim() == 2:
        return int(X.shape[0])
    if X.dim() == 3:
        return int(X.shape[0] * X.shape[1])
    return None


def _capture_entry(X: torch.Tensor, W: V9WeightContainer, T: int, key: _CacheKey) -> _CacheEntry:
    """Warm up on a side stream, then capture one eager forward.  Any failure
    yields a sentinel entry (``graph is None``)."""
    entry = _CacheEntry(key=key, T=T, d_in=W.d_in, d_out=W.d_out, n_hp_blocks=W.n_hp_blocks)
    if torch.cuda.is_current_stream_capturing():
        return entry                    # nested capture is refused
    t0 = time.perf_counter()
    try:
        from .. import _lib, ops
        x_static = torch.empty_strided(tuple(X.shape), tuple(X.stride()), dtype=X.dtype, device=X.device)
        x_static.copy_(X)
        side = torch.cuda.Stream(device=X.device)
        side.wait_stream(torch.cuda.current_stream(X.device))
        # the graph bakes the scratch address in: it gets scratch of its own, kept alive by the entry
        scratch = _lib.WorkspaceHolder()
        with _lib.use_workspace(scratch), torch.cuda.stream(side):
            ops.reserve_workspace(X.device, T, W.d_in, W.d_out, W.n_hp_blocks)
            for _ in range(3):
                _eager(x_static, W)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                y_static = _eager(x_static, W)
        torch.cuda.current_stream(X.device).wait_stream(side)
        entry.graph, entry.x_static, entry.y_static, entry.scratch = graph, x_static, y_static, scratch
    except Exception as exc:  # noqa: BLE001 - capture may fail for many reasons; stay on eager
        logger.warning("cuda_graph_cache: capture failed for %s (%s); using eager", key, exc)
        entry.graph = entry.x_static = entry.y_static = entry.scratch = None
    entry.capture_us = (time.perf_counter() - t0) * 1e6
    return entry


def _replay(entry: _CacheEntry, X: torch.Tensor) -> torch.Tensor:
    entry.x_static.copy_(X)
    entry.graph.replay()
    entry.replay_count += 1
    return entry.y_static.clone()


def v9_linear_forward_cuda_graph(X_fp16: torch.Tensor, W: V9WeightContainer) -> torch.Tensor:
    """Same result as ``v9_linear_forward``; replays a cached graph when the
    policy and the shape allow it, otherwise (or after a failed capture) runs
    eagerly."""
    if not getattr(X_fp16, "is_cuda", False) or _policy == "off":
        return _eager(X_fp16, W)
    T = _flat_T(X_fp16)
    if T is None or not _is_eligible(X_fp16, W, T):
        return _eager(X_fp16, W)
    key = _build_cache_key(X_fp16, W)
    entry = _cache.get(key)
    if entry is None:
        entry = _capture_entry(X_fp16, W, T, key)
        _cache.put(key, entry, weight_ref_target=W)
    if entry.graph is None:
        return _eager(X_fp16, W)
    return _replay(entry, X_fp16)


# ---------------------------------------------------------------------------
# Host-staged forward: pinned host activations in, pinned host result out, one
# graph launch.  Not in the reference (its callers keep activations on the
# device); it serves callers whose activations arrive in pinned host memory -
# the copy in, the quantisation + GEMM and the copy out are captured together,
# so a call costs one graph launch instead of five launches and their Python.
# ---------------------------------------------------------------------------
_host_graphs: "OrderedDict[Tuple[int, int, int, Tuple[int, ...], int], Tuple[Any, torch.Tensor, torch.Tensor]]" = OrderedDict()
_HOST_GRAPH_CAPACITY = 256


def v9_linear_forward_host_graph(X_pinned: torch.Tensor, W: V9WeightContainer, Y_pinned: torch.Tensor,
                                 device: Optional[torch.device] = None) -> torch.Tensor:
    """``Y_pinned[...] = v9_linear_forward(X_pinned.to(device), W)`` as one replayed
    CUDA graph on the current stream of ``device`` (default: the weights' device).

    ``X_pinned (..., d_in)`` fp16 and ``Y_pinned (..., d_out)`` fp16 must be pinned
    host tensors whose storage stays where it is between calls: the graph bakes
    their addresses in (refill ``X_pinned`` in place before each call).  The
    result is complete once the stream has been synchronised.  The first call for
    a (weights, input buffer, output buffer, shape) combination captures."""
    if not (X_pinned.is_pinned() and Y_pinned.is_pinned()):
        raise ValueError("X_pinned and Y_pinned must be pinned host tensors")
    if X_pinned.dtype != torch.float16 or Y_pinned.dtype != torch.float16:
        raise ValueError("X_pinned and Y_pinned must be fp16")
    if tuple(Y_pinned.shape) != tuple(X_pinned.shape[:-1]) + (W.d_out,):
        raise ValueError(f"Y_pinned must have shape {tuple(X_pinned.shape[:-1]) + (W.d_out,)}")
    dev = device if device is not None else W.W_low_packed.device
    key = (id(W), X_pinned.data_ptr(), Y_pinned.data_ptr(), tuple(X_pinned.shape), _device_index(W.W_low_packed))
    hit = _host_graphs.get(key)
    if hit is None:
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("v9_linear_forward_host_graph cannot capture inside another capture")
        from .. import _lib, ops
        T = 1
        for s_ in X_pinned.shape[:-1]:
            T *= int(s_)
        x_static = torch.empty(tuple(X_pinned.shape), dtype=torch.float16, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        scratch = _lib.WorkspaceHolder()          # owned by the graph (kept in the cache tuple)
        with _lib.use_workspace(scratch), torch.cuda.stream(side):
            ops.reserve_workspace(dev, T, W.d_in, W.d_out, W.n_hp_blocks)
            for _ in range(2):
                x_static.copy_(X_pinned, non_blocking=True)
                Y_pinned.copy_(_eager(x_static, W), non_blocking=True)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                x_static.copy_(X_pinned, non_blocking=True)
                y_static = _eager(x_static, W)
                Y_pinned.copy_(y_static, non_blocking=True)
        torch.cuda.current_stream(dev).wait_stream(side)
        hit = (graph, x_static, y_static, scratch)
        _host_graphs[key] = hit
        weakref.finalize(W, _host_graphs.pop, key, None)
        while len(_host_graphs) > _HOST_GRAPH_CAPACITY:
            _host_graphs.popitem(last=False)
    else:
        _host_graphs.move_to_end(key)
    hit[0].replay()
    return Y_pinned


_host_batch_graphs: "OrderedDict[Tuple, HostBatchGraph]" = OrderedDict()
_HOST_BATCH_CAPACITY = 32


class HostBatchGraph:
    """A captured batch of host-staged linears (``v9_linear_host_batch_graph``): ``replay()`` issues
    copy in, quantisation + GEMM and copy out of every request as one graph launch on the current
    stream; the results are complete once that stream has been synchronised.  The object keeps the
    graph's device buffers, streams and scratch alive; the caller keeps the pinned host buffers and
    the weight containers alive and at their addresses."""

    __slots__ = ("_graph", "_keep", "n_requests")

    def __init__(self, graph, keep, n_requests):
        self._graph, self._keep, self.n_requests = graph, keep, n_requests

    def replay(self) -> None:
        self._graph.replay()

    __call__ = replay


def _host_batch_key(reqs, n_streams):
    return (int(n_streams),) + tuple((id(W), X.data_ptr(), Y.data_ptr(), tuple(X.shape), X.dtype, Y.dtype)
                                     for X, W, Y in reqs)


def v9_linear_host_batch_graph(requests, n_streams: int = 12,
                               device: Optional[torch.device] = None) -> HostBatchGraph:
    """Validate and capture (or fetch from the cache) the graph of a batch of host-staged linears.

    ``requests``: sequence of ``(X_pinned, W, Y_pinned)`` with the conventions of
    ``v9_linear_forward_host_graph``; every request needs buffers of its own.  Inside
    the graph the requests are dealt round-robin onto ``n_streams`` parallel branches,
    so one request's copies overlap another's kernels - and, the requests being independent, so do
    the kernels of different requests: twelve decode linears of a Llama-3-8B layer mix take 442 / 209 /
    157 / 152 us per batch on 1 / 3 / 6 / 12 branches - and the whole batch costs one
    graph launch on the host.  Each branch owns scratch for its largest request.  A serving loop holds the returned object and calls
    ``replay()`` per step: no per-step argument checks or cache look-ups."""
    reqs = list(requests)
    if not reqs:
        raise ValueError("empty batch")
    key = _host_batch_key(reqs, n_streams)
    hit = _host_batch_graphs.get(key)
    if hit is not None:
        _host_batch_graphs.move_to_end(key)
        return hit
    for X, W, Y in reqs:
        if not (X.is_pinned() and Y.is_pinned()):
            raise ValueError("X_pinned and Y_pinned must be pinned host tensors")
        if X.dtype != torch.float16 or Y.dtype != torch.float16:
            raise ValueError("X_pinned and Y_pinned must be fp16")
        if tuple(Y.shape) != tuple(X.shape[:-1]) + (W.d_out,):
            raise ValueError(f"Y_pinned must have shape {tuple(X.shape[:-1]) + (W.d_out,)}")
    dev = device if device is not None else reqs[0][1].W_low_packed.device
    if torch.cuda.is_current_stream_capturing():
        raise RuntimeError("v9_linear_forward_host_graph_many cannot capture inside another capture")
    from .. import _lib, ops
    scratch = _lib.WorkspaceHolder()          # one buffer per branch stream, owned by the graph
    statics = [torch.empty(tuple(X.shape), dtype=torch.float16, device=dev) for X, _, _ in reqs]
    main = torch.cuda.Stream(device=dev)
    branches = [torch.cuda.Stream(device=dev) for _ in range(max(1, min(int(n_streams), len(reqs))))]
    keep = []

    def issue():
        for b in branches:
            b.wait_stream(main)
        for i, (X, W, Y) in enumerate(reqs):
            with torch.cuda.stream(branches[i % len(branches)]):
                statics[i].copy_(X, non_blocking=True)
                y = _eager(statics[i], W)
                Y.copy_(y, non_blocking=True)
                keep.append(y)
        for b in branches:
            main.wait_stream(b)

    main.wait_stream(torch.cuda.current_stream(dev))
    with _lib.use_workspace(scratch), torch.cuda.stream(main):
        for i, (X, W, _) in enumerate(reqs):          # the scratch is per stream: size it on every branch first
            T = X.numel() // X.shape[-1]
            with torch.cuda.stream(branches[i % len(branches)]):
                ops.reserve_workspace(dev, T, W.d_in, W.d_out, W.n_hp_blocks)
        issue()
        main.synchronize()
        keep.clear()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=main):
            issue()
    torch.cuda.current_stream(dev).wait_stream(main)
    hit = HostBatchGraph(graph, [statics, keep, branches, scratch], len(reqs))
    _host_batch_graphs[key] = hit
    while len(_host_batch_graphs) > _HOST_BATCH_CAPACITY:
        _host_batch_graphs.popitem(last=False)
    return hit


def v9_linear_forward_host_graph_many(requests, n_streams: int = 12,
                                      device: Optional[torch.device] = None) -> None:
    """Several independent host-staged linears as ONE replayed CUDA graph: looks the batch up by its
    buffers' addresses and shapes (``v9_linear_host_batch_graph``; the first call for a given batch
    validates and captures) and replays it.  Results are complete once the current stream has been
    synchronised."""
    reqs = list(requests)
    if not reqs:
        return
    v9_linear_host_batch_graph(reqs, n_streams, device).replay()


def set_cuda_graph_policy(policy: str) -> str:
    """``'off'`` (eager), ``'auto'`` (power-of-two T up to 128) or ``'force'`` (every
    T up to 128).  Returns the previous policy."""
    global _policy
    if policy not in _POLICY_LEGAL:
        raise ValueError(f"Unknown CUDA Graph policy {policy!r}; legal values are {_POLICY_LEGAL}")
    previous, _policy = _policy, policy
    return previous


def get_cuda_graph_policy() -> str:
    return _policy


def prewarm_cuda_graph_cache(entries: List[Tuple[torch.Tensor, V9WeightContainer]]) -> Dict[str, int]:
    """Capture graphs ahead of time; never raises.  Returns attempted / captured /
    skipped counts."""
    attempted = captured = skipped = 0
    for X, W in entries:
        T = _flat_T(X)
        if T is None or not getattr(X, "is_cuda", False) or not _is_eligible(X, W, T):
            skipped += 1
            continue
        attempted += 1
        key = _build_cache_key(X, W)
        entry = _cache.get(key)
        if entry is None:
            entry = _capture_entry(X, W, T, key)
            _cache.put(key, entry, weight_ref_target=W)
        if entry.graph is not None:
            captured += 1
    return {"attempted": attempted, "captured": captured, "skipped": skipped}


def cuda_graph_cache_stats() -> Dict[str, Any]:
    return _cache.stats()


def clear_cuda_graph_cache() -> None:
    _host_graphs.clear()
    _host_batch_graphs.clear()
    _cache.clear()


__all__ = [
    "v9_linear_forward_cuda_graph",
    "set_cuda_graph_policy",
    "get_cuda_graph_policy",
    "prewarm_cuda_graph_cache",
    "cuda_graph_cache_stats",
    "clear_cuda_graph_cache",
    "v9_linear_host_batch_graph",
    "HostBatchGraph",
]

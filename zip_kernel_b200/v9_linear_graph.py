"""Per-weight CUDA-graph wrapper of the module forward.

Interface of the reference's ``triton_kernel/v9_linear_graph.py:73-153``
(``V9LinearCudaGraph(W, warmup_iters)``; calling it with ``X (..., d_in)`` fp16
returns ``(..., d_out)`` fp16): one graph per ``(T, dtype)`` for decode-sized
calls (``T <= DECODE_T_THRESHOLD``), eager above.  Each graph owns its input and
output buffers and the scratch its kernels write, so graphs of different shapes
never share memory.
"""

from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import _lib, ops
from .pack_utils import V9WeightContainer
from .v9_linear import DECODE_T_THRESHOLD, v9_linear_forward


class V9LinearCudaGraph:
    """Graph-replayed forward of one weight container.  Do not change the
    container's tensors after the first call: the graphs hold their addresses."""

    def __init__(self, W: V9WeightContainer, warmup_iters: int = 3):
        self.W = W
        self.d_in, self.d_out = int(W.d_in), int(W.d_out)
        self.warmup_iters = max(1, int(warmup_iters))
        self._graphs: Dict[Tuple[int, torch.dtype, int], tuple] = {}

    def _capture(self, T: int, device: torch.device):
        x_static = torch.zeros((T, self.d_in), dtype=torch.float16, device=device)
        scratch = _lib.WorkspaceHolder()
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with _lib.use_workspace(scratch), torch.cuda.stream(side):
            ops.reserve_workspace(device, T, self.d_in, self.d_out, self.W.n_hp_blocks)
            for _ in range(self.warmup_iters):
                v9_linear_forward(x_static, self.W)
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                y_static = v9_linear_forward(x_static, self.W)
        torch.cuda.current_stream(device).wait_stream(side)
        return graph, x_static, y_static, scratch

    def __call__(self, X_fp16: torch.Tensor) -> torch.Tensor:
        assert X_fp16.is_cuda and X_fp16.dtype == torch.float16
        if X_fp16.shape[-1] != self.d_in:
            raise ValueError(f"X last dim ({X_fp16.shape[-1]}) != d_in ({self.d_in})")
        X_2d = X_fp16.reshape(-1, self.d_in)
        T = int(X_2d.shape[0])
        if T > DECODE_T_THRESHOLD or T == 0 or torch.cuda.is_current_stream_capturing():
            return v9_linear_forward(X_fp16, self.W)      # many tokens are not launch-bound; never nest captures
        key = (T, X_fp16.dtype, X_fp16.device.index or 0)
        entry = self._graphs.get(key)
        if entry is None:
            entry = self._capture(T, X_fp16.device)
            self._graphs[key] = entry
        graph, x_static, y_static, _ = entry
        x_static.copy_(X_2d, non_blocking=True)
        graph.replay()
        return y_static.clone().reshape(X_fp16.shape[:-1] + (self.d_out,))

    def n_graphs(self) -> int:
        return len(self._graphs)


__all__ = ["V9LinearCudaGraph"]

"""Module-level forward of the W4A4 linear.

Interface of the reference's ``triton_kernel/v9_linear.py`` (``v9_linear_forward``
:374-436, ``v9_linear_forward_decode`` :439-465, ``v9_linear_forward_prefill``
:468-484, ``reconstruct_w_fakequant_fp16`` :491-534, ``v9_linear_fakequant``
:537-562, ``DECODE_T_THRESHOLD`` :206) and of ``backend/dispatcher.py:271-338``.

The reference runs quant -> dense (+ sparse) -> combine + transpose as separate
launches.  Here one C-ABI call chains the quantisation kernel and a fused GEMM
that writes the ``(T, d_out)`` layout directly, so there is no combine/transpose
pass; decode and prefill differ only in which GEMM kernel the library selects.
"""

from __future__ import annotations

import os

import torch

from . import ops
from .pack_utils import BCOL, V9WeightContainer, unpack_s4_le

DECODE_T_THRESHOLD = 128


# W4A16 route for long prompts (the reference's backend/dispatcher.py:228-238): a layer WITHOUT residual blocks at
# T >= 1024 (or T >= 512 on shapes up to 4096 x 4096) is dequantised to fp16 and multiplied by a library fp16 GEMM;
# activations are then not quantised at all, so results differ from the W4A4 arithmetic (the reference bounds the
# difference by 2e-2 of the output range).  "off" (default here: every call is W4A4 and matches the oracle) or "auto"
# (the reference's rule).  The dequantised copy (4 x the packed bytes) is cached on the container.
_w4a16_policy = os.environ.get("W4A4_W4A16_FALLBACK", "off")


def set_w4a16_fallback(policy: str) -> str:
    """``'off'`` or ``'auto'``; returns the previous policy."""
    global _w4a16_policy
    if policy not in ("off", "auto"):
        raise ValueError(f"unknown W4A16 fallback policy {policy!r}; legal values are ('off', 'auto')")
    previous, _w4a16_policy = _w4a16_policy, policy
    return previous


def w4a16_eligible(W: V9WeightContainer, T: int) -> bool:
    """The reference's eligibility rule (dispatcher.py:231-234)."""
    return W.n_hp_blocks == 0 and (T >= 1024 or (T >= 512 and W.d_out * W.d_in <= 4096 * 4096))


def dequant_u4_to_fp16(W: V9WeightContainer) -> torch.Tensor:
    """``(d_out, d_in)`` fp16 weight in permuted column order, cached on the container."""
    cached = getattr(W, "_fp16_cache", None)
    if cached is None or cached.device != W.W_low_packed.device:
        cached = ops.dequant_u4_to_fp16_cuda(W.W_low_packed, W.scale_u4, W.zero_u4)
        W._fp16_cache = cached
    return cached


def _forward(X_fp16: torch.Tensor, W: V9WeightContainer, force=None) -> torch.Tensor:
    assert X_fp16.is_cuda and X_fp16.dtype == torch.float16
    d_in, d_out = W.d_in, W.d_out
    if X_fp16.shape[-1] != d_in:
        raise ValueError(f"X last dim ({X_fp16.shape[-1]}) must match d_in ({d_in})")
    X_2d = X_fp16 if X_fp16.dim() == 2 else X_fp16.reshape(-1, d_in)
    if _w4a16_policy == "auto" and force is None and w4a16_eligible(W, int(X_2d.shape[0])):
        perm = ops.perm_or_none(W.perm, W)
        Xp = X_2d if perm is None else X_2d.index_select(1, perm.to(torch.long))
        return torch.nn.functional.linear(Xp, dequant_u4_to_fp16(W)).reshape(X_fp16.shape[:-1] + (d_out,))
    Y = ops.fused_dense_sparse_e2e_cuda(
        X_2d, W.perm, W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets,
        W.hp_col_indices, W.scale_u4, W.zero_u4, d_out, d_in, token_major=True, force=force,
        prepared=W.prepared)
    return Y if X_fp16.dim() == 2 else Y.reshape(X_fp16.shape[:-1] + (d_out,))


def _gemm_on_expanded(quantised, W: V9WeightContainer, lead_shape, e4m3) -> torch.Tensor:
    XE, sumxf, scale_x = quantised
    Y = ops.fused_dense_sparse_expanded_cuda(
        W.W_low_packed, W.W_high_blocks_packed, W.hp_row_offsets, W.hp_col_indices, XE, sumxf, W.scale_u4,
        W.zero_u4, scale_x, W.d_out, W.d_in, token_major=True, prepared=W.prepared if e4m3 is True else None, e4m3=e4m3)
    return Y.reshape(tuple(lead_shape) + (W.d_out,))


def _wants_e4m3(W: V9WeightContainer, T: int):
    # the many-token kernel runs fp8 MMAs: on the prepared copy when the container has one, else on the packed
    # arrays; below its threshold the packed arrays are streamed against s8 codes
    if T < 256:
        return False
    return True if W.prepared is not None else "packed"


def v9_linear_forward_rmsnorm(X_fp16: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                              W: V9WeightContainer) -> torch.Tensor:
    """``v9_linear_forward(rms_norm(X) * norm_weight, W)`` in two launches (normalise + quantise, GEMM):
    the normalised activations are never written out.  Same output bits as the unfused sequence when the
    RMSNorm is the fp16 one of :func:`oracle.w4a4_oracle.rmsnorm_fp16`."""
    if X_fp16.shape[-1] != W.d_in:
        raise ValueError(f"X last dim ({X_fp16.shape[-1]}) must match d_in ({W.d_in})")
    T = X_fp16.numel() // W.d_in
    e4m3 = _wants_e4m3(W, T)
    q = ops.rmsnorm_quant_cuda(X_fp16, norm_weight, eps, ops.perm_or_none(W.perm, W), expanded=True, e4m3=e4m3)
    return _gemm_on_expanded(q, W, X_fp16.shape[:-1], e4m3)


def v9_linear_forward_silu_mul(gate_up_fp16: torch.Tensor, W: V9WeightContainer) -> torch.Tensor:
    """``v9_linear_forward(silu(gate) * up, W)`` for ``gate_up (..., 2 * d_in)`` (gate first) in two launches:
    the gated activations are quantised as they are computed, with no fp16 round trip."""
    if gate_up_fp16.shape[-1] != 2 * W.d_in:
        raise ValueError(f"gate_up last dim ({gate_up_fp16.shape[-1]}) must be 2 * d_in ({2 * W.d_in})")
    T = gate_up_fp16.numel() // (2 * W.d_in)
    e4m3 = _wants_e4m3(W, T)
    q = ops.silu_mul_quant_cuda(gate_up_fp16, ops.perm_or_none(W.perm, W), expanded=True, e4m3=e4m3)
    return _gemm_on_expanded(q, W, gate_up_fp16.shape[:-1], e4m3)


def prepare_for_prefill(W: V9WeightContainer) -> V9WeightContainer:
    """Widen the container's packed weights once (2 x their bytes, kept next to them) so that
    many-token calls run the fp8 instantiation of the tensor-core kernel; few-token calls keep
    streaming the packed arrays.  Outputs are bit-identical either way.  A load-time step with no
    counterpart in the reference's forward; returns ``W``."""
    assert W.W_low_packed.is_cuda, "prepare the container after moving it to the GPU"
    W.prepared = (ops.prepare_weights_cuda(W.W_low_packed), ops.prepare_weights_cuda(W.W_high_blocks_packed))
    return W


def v9_linear_forward(X_fp16: torch.Tensor, W: V9WeightContainer) -> torch.Tensor:
    """``Y (..., d_out)`` fp16 for ``X (..., d_in)`` fp16."""
    return _forward(X_fp16, W)


def v9_linear_forward_decode(X_fp16: torch.Tensor, W: V9WeightContainer) -> torch.Tensor:
    """Explicit decode entry; any T is accepted (same result as the dispatcher)."""
    return _forward(X_fp16, W)


def v9_linear_forward_prefill(X_fp16: torch.Tensor, W: V9WeightContainer) -> torch.Tensor:
    """Explicit prefill entry; any T is accepted (same result as the dispatcher)."""
    return _forward(X_fp16, W)


def reconstruct_w_fakequant_fp16(W: V9WeightContainer) -> torch.Tensor:
    """Dequantised ``(d_out, d_in)`` fp16 weight in permuted column order:
    ``(w_low - zero) * scale + 16 * w_high * scale`` on the residual blocks."""
    d_out, d_in = W.d_out, W.d_in
    scale = W.scale_u4.to(torch.float32)
    w = (unpack_s4_le(W.W_low_packed).to(torch.float32)
         - W.zero_u4.to(torch.float32).repeat_interleave(BCOL, dim=1)) * scale.repeat_interleave(BCOL, dim=1)
    if W.n_hp_blocks > 0:
        tiles = unpack_s4_le(W.W_high_blocks_packed).to(torch.float32)
        offs = W.hp_row_offsets.cpu().tolist()
        cols = W.hp_col_indices.cpu().tolist()
        brow, bcol = W.block_shape
        for br in range(len(offs) - 1):
            r0, r1 = br * brow, min((br + 1) * brow, d_out)
            for b in range(offs[br], offs[br + 1]):
                c0 = cols[b] * bcol
                w[r0:r1, c0:c0 + bcol] += 16.0 * tiles[b, : r1 - r0] * scale[r0:r1, cols[b]:cols[b] + 1]
    return w.to(torch.float16)


def v9_linear_fakequant(X_fp16: torch.Tensor, W: V9WeightContainer) -> torch.Tensor:
    """fp16 reference forward on the dequantised weight with fake-quantised
    activations (a correctness cross-check, not a fast path)."""
    X_2d = X_fp16.reshape(-1, W.d_in)
    Xp = X_2d[:, W.perm.to(torch.long)]
    W_fp = reconstruct_w_fakequant_fp16(W)
    max_abs = Xp.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale_x = (max_abs / 7.0).to(torch.float16).to(torch.float32)
    q = torch.clamp(torch.round(Xp.to(torch.float32) / scale_x), -8.0, 7.0)
    Y = (q * scale_x).to(torch.float16) @ W_fp.t()
    return Y.reshape(X_fp16.shape[:-1] + (W.d_out,))


__all__ = [
    "v9_linear_forward",
    "v9_linear_forward_decode",
    "v9_linear_forward_prefill",
    "v9_linear_forward_rmsnorm",
    "v9_linear_forward_silu_mul",
    "v9_linear_fakequant",
    "reconstruct_w_fakequant_fp16",
    "set_w4a16_fallback",
    "w4a16_eligible",
    "dequant_u4_to_fp16",
    "DECODE_T_THRESHOLD",
]

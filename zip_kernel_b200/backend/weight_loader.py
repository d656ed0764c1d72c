"""Validated zero-copy view of a weight container.

Interface of the reference's ``backend/weight_loader.py``
(``CutlassPackValidationError`` :74-111, ``CutlassV9Tensors`` :114-156,
``pack_v9_weights_for_cutlass`` :158-228, rules :236-330).  The checks are the
layout rules the kernels here rely on as well: int8 row-major nibbles with a
unit inner stride, ``d_in`` a multiple of 128, fp16 ``(d_out, n_groups)`` scale
and zero tables, one device.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..pack_utils import V9WeightContainer

_GROUP_K = 128


class CutlassPackValidationError(ValueError):
    """Raised in strict mode; ``violations`` lists every broken rule."""

    def __init__(self, violations: List[str]):
        self.violations = list(violations)
        super().__init__(
            "V9WeightContainer does not satisfy the INT4 layout contract. "
            f"{len(violations)} violation(s):\n  - " + "\n  - ".join(violations)
        )


@dataclass(frozen=True)
class CutlassV9Tensors:
    """View sharing storage with the source container."""

    W_low_rowmajor: torch.Tensor  # (d_out, d_in // 2) int8, stride(1) == 1
    scale_u4: torch.Tensor        # (d_out, n_groups) fp16
    zero_u4: torch.Tensor         # (d_out, n_groups) fp16
    d_out: int
    d_in: int
    n_groups: int
    source: V9WeightContainer


def _check_table(t: Optional[torch.Tensor], tag: str, name: str, d_out: int, ng: int) -> List[str]:
    out: List[str] = []
    if not isinstance(t, torch.Tensor):
        return [f"{tag}: {name} is not a torch.Tensor (got {type(t)!r})"]
    if t.dtype != torch.float16:
        out.append(f"{tag}: {name}.dtype must be float16, got {t.dtype}")
    if t.dim() != 2:
        out.append(f"{tag}: {name} must be 2-D, got shape {tuple(t.shape)}")
        return out
    if int(t.shape[0]) != d_out:
        out.append(f"{tag}: {name}.shape[0]={int(t.shape[0])} disagrees with container.d_out={d_out}")
    if ng > 0 and int(t.shape[1]) != ng:
        out.append(f"{tag}: {name}.shape[1]={int(t.shape[1])} must equal d_in/GROUP_K={ng}")
    if t.stride(1) != 1:
        out.append(f"{tag}: {name}.stride(1)={t.stride(1)} must be 1")
    return out


def _collect_violations(container: V9WeightContainer) -> List[str]:
    """Every broken rule, never raises (the tests assert a complete list)."""
    v: List[str] = []
    W = container.W_low_packed
    d_out, d_in = int(container.d_out), int(container.d_in)
    if not isinstance(W, torch.Tensor):
        v.append(f"T1: W_low_packed is not a torch.Tensor (got {type(W)!r})")
    else:
        if W.dtype != torch.int8:
            v.append(f"T1: W_low_packed.dtype must be int8, got {W.dtype}")
        if W.dim() != 2:
            v.append(f"T1: W_low_packed must be 2-D, got shape {tuple(W.shape)}")
        else:
            if int(W.shape[0]) != d_out:
                v.append(f"T1: W_low_packed.shape[0]={int(W.shape[0])} disagrees with container.d_out={d_out}")
            if int(W.shape[1]) * 2 != d_in:
                v.append(f"T1: W_low_packed.shape[1]={int(W.shape[1])} must equal d_in/2={d_in // 2} (d_in={d_in})")
            if W.stride(1) != 1:
                v.append(f"T1: W_low_packed.stride(1)={W.stride(1)} must be 1")
    if d_in % _GROUP_K != 0:
        v.append(f"Alignment: d_in={d_in} not divisible by kAlignmentA={_GROUP_K}")
        v.append(f"Alignment: d_in={d_in} not divisible by GROUP_K={_GROUP_K}")
    ng = d_in // _GROUP_K if d_in > 0 else 0
    v += _check_table(container.scale_u4, "T5", "scale_u4", d_out, ng)
    v += _check_table(container.zero_u4, "T6", "zero_u4", d_out, ng)
    devs = [(n, t.device) for n, t in (("W_low_packed", W), ("scale_u4", container.scale_u4),
                                       ("zero_u4", container.zero_u4)) if isinstance(t, torch.Tensor)]
    if devs and len({d for _, d in devs}) > 1:
        v.append(f"Device: W_low_packed / scale_u4 / zero_u4 straddle multiple devices: {devs}")
    return v


def pack_v9_weights_for_cutlass(container: V9WeightContainer, *, strict: bool = True) -> CutlassV9Tensors:
    """Adapt a container to the dense-GEMM tensor view; raises
    :class:`CutlassPackValidationError` with all violations in strict mode."""
    violations = _collect_violations(container)
    if strict and violations:
        raise CutlassPackValidationError(violations)
    return CutlassV9Tensors(
        W_low_rowmajor=container.W_low_packed,
        scale_u4=container.scale_u4,
        zero_u4=container.zero_u4,
        d_out=int(container.d_out),
        d_in=int(container.d_in),
        n_groups=int(container.n_groups),
        source=container,
    )


__all__ = ["CutlassV9Tensors", "CutlassPackValidationError", "pack_v9_weights_for_cutlass"]

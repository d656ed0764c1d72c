"""Weight container and 4-bit packing contract of the W4A4 linear.

Mirrors the interface of the reference's ``triton_kernel/pack_utils.py``
(constants ``BROW``/``BCOL`` :24-25, ``pack_s4_le`` :32-56, ``unpack_s4_le``
:59-78, ``V9WeightContainer`` :85-106, ``pack_v9_weights`` :113-264) so that a
container packed by either project is consumed unchanged by the kernels here.

Layout facts the kernels rely on:

* ``W_low_packed  (d_out, d_in/2) int8`` - byte j of a row holds element 2j in
  its low nibble and 2j+1 in its high nibble; values are ``u4 - 8`` (signed).
* ``W_high_blocks_packed (nnz, 128, 64) int8`` - the high nibbles of the int8
  residual blocks, same nibble order, blocks sorted by (block-row, block-col).
* ``scale_u4, zero_u4 (d_out, d_in/128) fp16`` - ``zero_u4`` already shifted by -8.
* ``hp_row_offsets (d_out/128 + 1) int32``, ``hp_col_indices (nnz) int32`` - block-CSR.
* ``perm (d_in) int32`` - activation column gather applied before quantisation.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

BROW: int = 128
BCOL: int = 128


def pack_s4_le(tensor: torch.Tensor) -> torch.Tensor:
    """Pack 4-bit integers along the last dim, little-endian nibbles.

    ``byte[j] = (x[2j+1] << 4) | (x[2j] & 15)``; accepts u4 in [0, 15] and s4 in
    [-8, 7] alike (two's-complement nibble kept).  Returns int8 with the last
    dim halved.
    """
    if tensor.shape[-1] % 2 != 0:
        raise ValueError(
            f"pack_s4_le requires last dim to be even, got {tensor.shape[-1]}"
        )
    pairs = tensor.to(torch.int16).reshape(*tensor.shape[:-1], tensor.shape[-1] // 2, 2)
    byte = ((pairs[..., 1] & 0x0F) << 4) | (pairs[..., 0] & 0x0F)      # 0..255
    # wrap 128..255 onto the negative int8 range explicitly
    return (byte - ((byte & 0x80) << 1)).to(torch.int8)


def unpack_s4_le(packed: torch.Tensor, signed: bool = True) -> torch.Tensor:
    """Inverse of :func:`pack_s4_le`; returns int8 with the last dim doubled."""
    b = packed.to(torch.int16) & 0xFF
    nib = torch.stack((b & 0x0F, b >> 4), dim=-1).reshape(*packed.shape[:-1],
                                                         packed.shape[-1] * 2)
    if signed:
        nib = nib - ((nib & 0x8) << 1)
    return nib.to(torch.int8)


@dataclass
class V9WeightContainer:
    """Inference-ready weights of one W4A4 linear (field names as in the reference)."""

    W_low_packed: torch.Tensor          # (d_out, d_in // 2) int8
    W_high_blocks_packed: torch.Tensor  # (n_hp_blocks, 128, 64) int8
    scale_u4: torch.Tensor              # (d_out, n_groups) fp16
    zero_u4: torch.Tensor               # (d_out, n_groups) fp16, pre-shifted by -8
    hp_row_offsets: torch.Tensor        # (ceil(d_out/128) + 1,) int32
    hp_col_indices: torch.Tensor        # (n_hp_blocks,) int32
    perm: torch.Tensor                  # (d_in,) int32
    block_shape: Tuple[int, int]
    d_out: int
    d_in: int
    # optional (W_low, W_high) widened once for the many-token kernel (``prepare_for_prefill``); not part
    # of the reference's container and never serialised: a copy made by ``to`` starts without it
    prepared: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    @property
    def n_hp_blocks(self) -> int:
        return int(self.W_high_blocks_packed.shape[0])

    @property
    def n_groups(self) -> int:
        return int(self.scale_u4.shape[1])

    def to(self, device) -> "V9WeightContainer":
        """Copy of the container with every tensor moved to ``device``."""
        mv = lambda t: t.to(device)
        return V9WeightContainer(
            W_low_packed=mv(self.W_low_packed),
            W_high_blocks_packed=mv(self.W_high_blocks_packed),
            scale_u4=mv(self.scale_u4), zero_u4=mv(self.zero_u4),
            hp_row_offsets=mv(self.hp_row_offsets), hp_col_indices=mv(self.hp_col_indices),
            perm=mv(self.perm), block_shape=self.block_shape,
            d_out=self.d_out, d_in=self.d_in,
        )


def pack_v9_weights(
    gptq_outputs: Dict[str, torch.Tensor],
    brow: int = BROW,
    bcol: int = BCOL,
) -> V9WeightContainer:
    """Build a :class:`V9WeightContainer` from mixed-precision quantiser outputs.

    Keys (as in the reference, ``pack_utils.py:120-127``): ``Q_u4_permuted
    (d_out, d_in)`` in [0, 15]; ``scale_u4_raw``/``zero_u4_raw (d_out, n_groups)``;
    ``Q_s8_blocks (nnz, 128, 128)`` int8; ``scale_s8_per_block (nnz, 128)``;
    ``hp_block_indices (nnz, 2)`` as (block-row, block-col); ``perm (d_in,)``.

    Each int8 block is split losslessly as ``q = 16 * hi + lo``: ``lo`` replaces
    the dense u4 codes of that block, ``hi`` goes to the residual, the block's
    row scale overwrites ``scale_u4[rows, bc]`` and its zero becomes 0.  Dense
    codes and zeros are then shifted by -8, and residual blocks are ordered by
    (block-row, block-col) into block-CSR.
    """
    if brow != BROW or bcol != BCOL:
        raise ValueError(
            f"V9 pack requires brow == bcol == 128, got brow={brow}, bcol={bcol}"
        )
    q_u4 = gptq_outputs["Q_u4_permuted"]
    d_out, d_in = int(q_u4.shape[0]), int(q_u4.shape[1])
    if d_in % bcol != 0:
        raise ValueError(f"V9 pack requires d_in ({d_in}) divisible by bcol ({bcol})")
    n_groups = d_in // bcol
    nrow = (d_out + brow - 1) // brow
    for key in ("scale_u4_raw", "zero_u4_raw"):
        if tuple(gptq_outputs[key].shape) != (d_out, n_groups):
            raise ValueError(
                f"{key} expected shape ({d_out}, {n_groups}), "
                f"got {tuple(gptq_outputs[key].shape)}"
            )
    device = q_u4.device
    low = q_u4.to(torch.int32).clone()
    scale = gptq_outputs["scale_u4_raw"].to(torch.float16).clone()
    zero = gptq_outputs["zero_u4_raw"].to(torch.float16).clone()

    idx = gptq_outputs["hp_block_indices"]
    n_hp = int(idx.shape[0]) if idx.numel() > 0 else 0
    if n_hp > 0:
        idx = idx.reshape(n_hp, 2).to(torch.int64).cpu()
        # block-CSR order: by block-row, ties by block-col (stable for duplicates)
        order = sorted(range(n_hp), key=lambda i: (int(idx[i, 0]), int(idx[i, 1])))
        slot = {src: dst for dst, src in enumerate(order)}
        blocks = gptq_outputs["Q_s8_blocks"]
        blk_scale = gptq_outputs["scale_s8_per_block"]
        high = torch.zeros((n_hp, brow, bcol), dtype=torch.int8, device=device)
        # writes into `low`/`scale` happen in the caller's order so that a
        # duplicated block index resolves exactly as in the reference packer
        for i in range(n_hp):
            br, bc = int(idx[i, 0]), int(idx[i, 1])
            r0, r1 = br * brow, min((br + 1) * brow, d_out)
            c0, c1 = bc * bcol, min((bc + 1) * bcol, d_in)
            q8 = blocks[i, : r1 - r0, : c1 - c0].to(torch.int32)
            hi = q8 >> 4                       # arithmetic shift: [-8, 7]
            lo = q8 & 0x0F                     # [0, 15]
            if not torch.equal(hi * 16 + lo, q8):
                raise AssertionError(f"bit-split mismatch at block idx={i} (br={br}, bc={bc})")
            low[r0:r1, c0:c1] = lo
            high[slot[i], : r1 - r0, : c1 - c0] = hi.to(torch.int8)
            scale[r0:r1, bc] = blk_scale[i, : r1 - r0].to(torch.float16)
            zero[r0:r1, bc] = 0.0
        brs = torch.tensor([int(idx[i, 0]) for i in order], dtype=torch.int64)
        cols = torch.tensor([int(idx[i, 1]) for i in order], dtype=torch.int32, device=device)
        row_offsets = torch.zeros(nrow + 1, dtype=torch.int32, device=device)
        row_offsets[1:] = torch.cumsum(torch.bincount(brs, minlength=nrow), 0).to(torch.int32)
    else:
        high = torch.zeros((0, brow, bcol), dtype=torch.int8, device=device)
        cols = torch.zeros((0,), dtype=torch.int32, device=device)
        row_offsets = torch.zeros(nrow + 1, dtype=torch.int32, device=device)

    return V9WeightContainer(
        W_low_packed=pack_s4_le((low - 8).to(torch.int8)),
        W_high_blocks_packed=pack_s4_le(high),
        scale_u4=scale,
        zero_u4=(zero - 8.0).to(torch.float16),
        hp_row_offsets=row_offsets,
        hp_col_indices=cols,
        perm=gptq_outputs["perm"].to(torch.int32).to(device),
        block_shape=(brow, bcol),
        d_out=d_out,
        d_in=d_in,
    )


__all__ = [
    "BROW",
    "BCOL",
    "pack_s4_le",
    "unpack_s4_le",
    "V9WeightContainer",
    "pack_v9_weights",
]

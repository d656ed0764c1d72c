"""Seeded synthetic inputs for the W4A4 linear (no checkpoints, no datasets).

The reference measures and tests on seeded random tensors only
(``cuda_kernel/tests/test_parity.py:30-79``, ``bench_qwen3_shapes.py``).  The
recipes here follow those distributions and the benchmark description:
activations ``N(0, 1)`` with 1 % of the K channels scaled by 20 (outlier
channels), s4 weights uniform in [-8, 7], ``scale_u4 ~ U(0,1) * 0.05 + 0.001``,
``zero_u4 ~ N(0, 0.2^2)``, and a Bernoulli mask of 128x128 residual blocks.
Everything is generated on the CPU with an explicit ``torch.Generator`` so that
a seed gives the same tensors on every machine.
"""

from __future__ import annotations

from typing import Optional

import torch

from .pack_utils import BCOL, BROW, V9WeightContainer, pack_s4_le


def shape_seed(M: int, K: int, N: int) -> int:
    """Seed convention of the reference's shape sweeps: ``0xBEEF + M + K + N``."""
    return 0xBEEF + int(M) + int(K) + int(N)


def make_activations(M: int, K: int, seed: int, outlier_frac: float = 0.01,
                     outlier_scale: float = 20.0, std: float = 1.0) -> torch.Tensor:
    """``X (M, K)`` fp16: ``N(0, std)`` with ``round(outlier_frac * K)`` channels x20."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    x = torch.randn(M, K, generator=g, dtype=torch.float32) * std
    n_out = int(round(outlier_frac * K))
    if n_out > 0:
        ch = torch.randperm(K, generator=g)[:n_out]
        x[:, ch] *= outlier_scale
    return x.to(torch.float16)


def make_perm(K: int, seed: Optional[int]) -> torch.Tensor:
    """Identity when ``seed`` is None, else a seeded random permutation (int32)."""
    if seed is None:
        return torch.arange(K, dtype=torch.int32)
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    return torch.randperm(K, generator=g).to(torch.int32)


def make_container(N: int, K: int, density: float, seed: int, perm_seed: Optional[int] = None,
                   per_channel_scale: bool = False, force_block_per_row: bool = False,
                   ) -> V9WeightContainer:
    """Random packed weights with a Bernoulli(density) residual-block mask.

    ``per_channel_scale`` gives the special case ``scale_u4[n, :] = s[n]``,
    ``zero_u4 = 0`` (symmetric per-output-channel weights).  ``N`` need not be a
    multiple of 128; the last block-row is then ragged (its residual blocks are
    still stored as full 128x128 tiles with zero padding, as the packer does).
    """
    if K % BCOL != 0:
        raise ValueError(f"K ({K}) must be a multiple of {BCOL}")
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    ng = K // BCOL
    nbr = (N + BROW - 1) // BROW
    w = torch.randint(-8, 8, (N, K), generator=g, dtype=torch.int8)
    if per_channel_scale:
        s = (torch.rand(N, 1, generator=g) * 0.05 + 0.001).expand(N, ng).contiguous()
        z = torch.zeros(N, ng)
    else:
        s = torch.rand(N, ng, generator=g) * 0.05 + 0.001
        z = torch.randn(N, ng, generator=g) * 0.2
    mask = torch.rand(nbr, ng, generator=g) < density
    if force_block_per_row and density > 0:
        for br in range(nbr):
            if not bool(mask[br].any()):
                mask[br, int(torch.randint(0, ng, (1,), generator=g))] = True
    coords = mask.nonzero()                      # sorted by (br, bc)
    nnz = int(coords.shape[0])
    wh = torch.randint(-8, 8, (nnz, BROW, BCOL), generator=g, dtype=torch.int8)
    if N % BROW != 0 and nnz > 0:
        last = coords[:, 0] == nbr - 1
        wh[last, N - (nbr - 1) * BROW:, :] = 0
    row_offsets = torch.zeros(nbr + 1, dtype=torch.int32)
    if nnz > 0:
        row_offsets[1:] = torch.cumsum(torch.bincount(coords[:, 0], minlength=nbr), 0).to(torch.int32)
    return V9WeightContainer(
        W_low_packed=pack_s4_le(w),
        W_high_blocks_packed=pack_s4_le(wh) if nnz > 0 else torch.zeros((0, BROW, BCOL // 2), dtype=torch.int8),
        scale_u4=s.to(torch.float16),
        zero_u4=z.to(torch.float16),
        hp_row_offsets=row_offsets,
        hp_col_indices=coords[:, 1].to(torch.int32).contiguous() if nnz > 0 else torch.zeros((0,), dtype=torch.int32),
        perm=make_perm(K, perm_seed),
        block_shape=(BROW, BCOL),
        d_out=N,
        d_in=K,
    )


def make_container_like(base: V9WeightContainer, density: float, seed: int) -> V9WeightContainer:
    """A container with ``base``'s dense weights, scales, zeros and permutation and a NEW residual part
    (Bernoulli(density) mask, uniform s4 blocks) - for sweeps over the residual density, where drawing
    the dense matrix again for every point would only cost time."""
    N, K = base.d_out, base.d_in
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    ng, nbr = K // BCOL, (N + BROW - 1) // BROW
    mask = torch.rand(nbr, ng, generator=g) < density
    coords = mask.nonzero()
    nnz = int(coords.shape[0])
    wh = torch.randint(-8, 8, (nnz, BROW, BCOL), generator=g, dtype=torch.int8)
    if N % BROW != 0 and nnz > 0:
        wh[coords[:, 0] == nbr - 1, N - (nbr - 1) * BROW:, :] = 0
    row_offsets = torch.zeros(nbr + 1, dtype=torch.int32)
    if nnz > 0:
        row_offsets[1:] = torch.cumsum(torch.bincount(coords[:, 0], minlength=nbr), 0).to(torch.int32)
    return V9WeightContainer(
        W_low_packed=base.W_low_packed, scale_u4=base.scale_u4, zero_u4=base.zero_u4, perm=base.perm,
        W_high_blocks_packed=pack_s4_le(wh) if nnz > 0 else torch.zeros((0, BROW, BCOL // 2), dtype=torch.int8),
        hp_row_offsets=row_offsets,
        hp_col_indices=coords[:, 1].to(torch.int32).contiguous() if nnz > 0 else torch.zeros((0,), dtype=torch.int32),
        block_shape=(BROW, BCOL), d_out=N, d_in=K)


def algorithmic_bytes(M: int, K: int, N: int, nnz: int, fused_quant: bool = True) -> int:
    """Bytes one fused linear must move at least once.

    Weights ``0.5*K*N`` nibbles + ``4*N*ng`` fp16 scale and zero + ``8192*nnz``
    residual nibbles + the block-CSR index; activations ``2*M*K`` fp16 plus the
    permutation; output ``2*M*N``.  With a separate quantisation kernel the
    packed codes, scales and group sums are written once and read once more.
    """
    ng = K // BCOL
    nbr = (N + BROW - 1) // BROW
    b_w = K * N // 2 + 4 * N * ng + 8192 * nnz + 4 * (nbr + 1) + 4 * nnz
    b_x = 2 * M * K + 4 * K
    if not fused_quant:
        b_x += 2 * (M * K // 2 + 2 * M + 4 * M * ng)
    return int(b_w + b_x + 2 * M * N)


def algorithmic_ops(M: int, K: int, N: int, nnz: int = 0) -> int:
    """Integer multiply-adds counted as 2 ops: dense ``2*M*K*N`` (+ residual blocks)."""
    return int(2 * M * K * N + 2 * M * BROW * BCOL * nnz)

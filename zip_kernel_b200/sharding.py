"""Column-parallel sharding of a W4A4 linear over the GPUs of one node.

The reference is single-GPU.  Each output row of the linear depends only on its
own row of the packed weights, its row of scales/zeros and the residual blocks
of its block-row, so the layer splits over ``d_out`` with no reduction: rank r
of g owns a contiguous range of 128-row block-rows (a residual block never
straddles two ranks), activations and ``perm`` are replicated and every rank
quantises them itself.  The only exchange is an all-gather of the fp16 output
shards where the caller needs the full output; it goes through
``torch.distributed`` (NCCL over NVLink on GPUs, gloo in the CPU tests).
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .pack_utils import BCOL, BROW, V9WeightContainer


def block_row_range(n_block_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Balanced contiguous split of the block-rows: the first ``n % world`` ranks
    get one more."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, rem = divmod(n_block_rows, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_rows(d_out: int, rank: int, world: int) -> Tuple[int, int]:
    """Output-row range ``[lo, hi)`` of a rank."""
    nbr = (d_out + BROW - 1) // BROW
    b0, b1 = block_row_range(nbr, rank, world)
    return min(b0 * BROW, d_out), min(b1 * BROW, d_out)


def shard_container(W: V9WeightContainer, rank: int, world: int) -> V9WeightContainer:
    """The rank's slice of a container: rows ``shard_rows`` of the dense nibbles
    and of the scale/zero tables, the residual blocks of its block-rows with the
    row offsets re-based to zero (column indices address K and stay as they are).
    Tensors are views where slicing allows."""
    nbr = (W.d_out + BROW - 1) // BROW
    b0, b1 = block_row_range(nbr, rank, world)
    r0, r1 = min(b0 * BROW, W.d_out), min(b1 * BROW, W.d_out)
    offs = W.hp_row_offsets
    k0, k1 = int(offs[b0]), int(offs[b1])
    return V9WeightContainer(
        W_low_packed=W.W_low_packed[r0:r1],
        W_high_blocks_packed=W.W_high_blocks_packed[k0:k1],
        scale_u4=W.scale_u4[r0:r1],
        zero_u4=W.zero_u4[r0:r1],
        hp_row_offsets=(offs[b0:b1 + 1] - offs[b0]).to(torch.int32).contiguous(),
        hp_col_indices=W.hp_col_indices[k0:k1],
        perm=W.perm,
        block_shape=W.block_shape,
        d_out=r1 - r0,
        d_in=W.d_in,
    )


def shard_sizes(d_out: int, world: int) -> List[int]:
    return [shard_rows(d_out, r, world)[1] - shard_rows(d_out, r, world)[0] for r in range(world)]


def check_shard_metadata(d_out: int, d_in: int, shard: V9WeightContainer, rank: int, world: int) -> None:
    """Reject a shard that does not belong to (d_out, d_in, rank, world) before any
    kernel is launched with it."""
    lo, hi = shard_rows(d_out, rank, world)
    if shard.d_in != d_in or d_in % BCOL != 0:
        raise ValueError(f"shard d_in={shard.d_in} does not match layer d_in={d_in}")
    if shard.d_out != hi - lo:
        raise ValueError(f"rank {rank}/{world} must own {hi - lo} rows of {d_out}, shard has {shard.d_out}")
    nbr = (shard.d_out + BROW - 1) // BROW
    if shard.hp_row_offsets.numel() != nbr + 1 or int(shard.hp_row_offsets[0]) != 0:
        raise ValueError("shard block-row offsets are not re-based to its own rows")
    if int(shard.hp_row_offsets[-1]) != shard.n_hp_blocks:
        raise ValueError("shard block-row offsets disagree with its number of residual blocks")


def gather_output(y_local: torch.Tensor, d_out: int, group=None, token_major: bool = True) -> torch.Tensor:
    """All-gather the per-rank outputs into the full output.

    ``token_major``: shards are ``(T, d_out_r)`` and the result ``(T, d_out)``;
    otherwise shards are ``(d_out_r, T)`` (contiguous row ranges of the result, so
    equal shards are gathered in place with no repack) and the result
    ``(d_out, T)``.  Unequal shards are padded to the largest for the exchange.
    """
    import torch.distributed as dist

    world = dist.get_world_size(group)
    sizes = shard_sizes(d_out, world)
    rows_axis = 1 if token_major else 0
    T = y_local.shape[0] if token_major else y_local.shape[1]
    if y_local.shape[rows_axis] != sizes[dist.get_rank(group)]:
        raise ValueError("local output does not have this rank's shard size")
    biggest = max(sizes)
    if not token_major and len(set(sizes)) == 1:
        out = torch.empty((d_out, T), dtype=y_local.dtype, device=y_local.device)
        dist.all_gather_into_tensor(out, y_local.contiguous(), group=group)
        return out
    # (world, rows, T) staging with rows leading, padded to the largest shard
    rows_first = y_local.t() if token_major else y_local
    send = torch.zeros((biggest, T), dtype=y_local.dtype, device=y_local.device)
    send[: rows_first.shape[0]] = rows_first
    recv = torch.empty((world * biggest, T), dtype=y_local.dtype, device=y_local.device)
    dist.all_gather_into_tensor(recv, send, group=group)
    full = torch.cat([recv[r * biggest: r * biggest + sizes[r]] for r in range(world)], dim=0)      # (d_out, T)
    return full.t().contiguous() if token_major else full


def column_parallel_forward(X_fp16: torch.Tensor, shard: V9WeightContainer, d_out: int, group=None,
                            gather: bool = True) -> torch.Tensor:
    """Forward of one rank's shard; with ``gather`` the full ``(..., d_out)``
    output is assembled on every rank, otherwise the local ``(..., d_out_r)``
    slice is returned (the consumer stays shard-aware)."""
    from .v9_linear import v9_linear_forward

    y = v9_linear_forward(X_fp16, shard)
    if not gather:
        return y
    lead = y.shape[:-1]
    full = gather_output(y.reshape(-1, y.shape[-1]), d_out, group=group, token_major=True)
    return full.reshape(lead + (d_out,))


__all__ = ["block_row_range", "shard_rows", "shard_sizes", "shard_container", "check_shard_metadata",
           "gather_output", "column_parallel_forward"]

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


class _DeviceArray:
    """Raw device memory exposed through the CUDA array interface, so that torch can view it."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 2, "strides": None}


class PeerGather:
    """All-gather of the output shards WITHOUT a collective library call: every rank's kernel stores its
    shard straight into every rank's copy of the full output over NVLink (plain stores to peer-mapped
    memory) and waits, with a bound, for the other ranks' flags (``w4a4_peer_push_wait``).  One kernel
    launch per exchange - for decode-sized outputs the launch and protocol cost of a library all-gather
    (~20 us) is more than the sharded GEMM itself.  One process per GPU, one node.

    Two buffer sets alternate, so the tensor a call returns stays valid until the second next call.  Every
    rank must make the same sequence of calls.  Capturable in a CUDA graph (no host-side state changes per
    call except the alternation, which a replayed graph repeats consistently on all ranks)."""

    FLAG_BYTES = 256

    def __init__(self, max_bytes: int, group=None, device=None, poll_limit: int = 2_000_000):
        import ctypes
        import torch.distributed as dist
        from . import _lib
        self._lib = _lib.load()
        self._check = _lib.check
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > 16:
            raise ValueError("PeerGather supports up to 16 ranks")
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.max_bytes = (int(max_bytes) + 255) // 256 * 256
        self.poll_limit = int(poll_limit)
        self.sets, self._next = [], 0
        with torch.cuda.device(self.device):
            for _ in range(2):
                own = ctypes.c_void_p()
                self._check(self._lib.w4a4_peer_alloc(self.FLAG_BYTES + self.max_bytes, ctypes.byref(own)), "peer_alloc")
                handle = ctypes.create_string_buffer(64)
                self._check(self._lib.w4a4_peer_export(own, handle), "peer_export")
                handles = [None] * self.world
                dist.all_gather_object(handles, bytes(handle.raw), group=group)
                ptrs, opened = [], []
                for r in range(self.world):
                    if r == self.rank:
                        ptrs.append(own.value)
                        continue
                    peer = ctypes.c_void_p()
                    self._check(self._lib.w4a4_peer_open(ctypes.create_string_buffer(handles[r], 64), ctypes.byref(peer)), "peer_open")
                    ptrs.append(peer.value)
                    opened.append(peer.value)
                PtrArr = ctypes.c_void_p * self.world
                self.sets.append(dict(own=own.value, opened=opened, flags=PtrArr(*ptrs),
                                      data=PtrArr(*[p + self.FLAG_BYTES for p in ptrs]),
                                      state=torch.zeros(1 + 2 * self.world, dtype=torch.int32, device=self.device)))
        dist.barrier(group=group)         # nobody pushes before everyone has mapped everything

    def gather(self, y_local: torch.Tensor, d_out: int, token_major: bool = True) -> torch.Tensor:
        """``y_local``: this rank's ``(T, d_out_r)`` (``token_major``) or ``(d_out_r, T)`` fp16 shard.  Returns the
        full ``(T, d_out)`` / ``(d_out, T)`` output as a view of this rank's exchange buffer; it is complete when
        the current stream has executed the call."""
        assert y_local.is_cuda and y_local.dtype == torch.float16 and y_local.dim() == 2
        sizes = shard_sizes(d_out, self.world)
        row_off = sum(sizes[: self.rank])
        n_r = sizes[self.rank]
        T = int(y_local.shape[0] if token_major else y_local.shape[1])
        if int(y_local.shape[1 if token_major else 0]) != n_r:
            raise ValueError("local output does not have this rank's shard size")
        if 2 * T * d_out > self.max_bytes:
            raise ValueError(f"full output of {2 * T * d_out} bytes exceeds the exchange buffer ({self.max_bytes})")
        if y_local.stride(1) != 1:
            y_local = y_local.contiguous()
        st = self.sets[self._next]
        self._next ^= 1
        return self._exchange(st, y_local, d_out, T, n_r, row_off, token_major)

    def gather_band(self, y_band: torch.Tensor, d_out: int, T_total: int, t0: int) -> torch.Tensor:
        """Token-major exchange of a BAND of tokens: ``y_band (T_b, d_out_r)`` goes to rows ``t0 .. t0 + T_b`` of the
        full ``(T_total, d_out)`` output in the CURRENT buffer set, which stays current until :meth:`advance` - so a
        long prompt can be exchanged band by band on a side stream while the next band is computed.  Returns the
        full output view (complete for the bands exchanged so far)."""
        assert y_band.is_cuda and y_band.dtype == torch.float16 and y_band.dim() == 2 and y_band.stride(1) == 1
        sizes = shard_sizes(d_out, self.world)
        if int(y_band.shape[1]) != sizes[self.rank] or 2 * T_total * d_out > self.max_bytes:
            raise ValueError("band does not fit this rank's shard or the exchange buffer")
        st = self.sets[self._next]
        Tb = int(y_band.shape[0])
        if Tb > 0 and sizes[self.rank] > 0:
            self._push(st, y_band, Tb, 2 * sizes[self.rank], 2 * int(y_band.stride(0)), 2 * d_out,
                       2 * (t0 * d_out + sum(sizes[: self.rank])))
        return torch.as_tensor(_DeviceArray(st["own"] + self.FLAG_BYTES, (T_total, d_out), "<f2"), device=self.device)

    def advance(self) -> None:
        """Make the other buffer set current (after the last band of a step)."""
        self._next ^= 1

    def _push(self, st, y, rows, row_bytes, src_pitch, dst_pitch, dst_off) -> None:
        with torch.cuda.device(self.device):
            self._check(self._lib.w4a4_peer_push_wait(
                y.data_ptr(), src_pitch, st["data"], st["flags"], dst_pitch, dst_off, rows, row_bytes,
                self.world, self.rank, st["state"].data_ptr(), self.poll_limit,
                torch.cuda.current_stream(self.device).cuda_stream), "peer_push_wait")

    def _exchange(self, st, y_local, d_out, T, n_r, row_off, token_major):
        if token_major:
            rows, row_bytes, src_pitch = T, 2 * n_r, 2 * int(y_local.stride(0))
            dst_pitch, dst_off = 2 * d_out, 2 * row_off
            shape = (T, d_out)
        else:
            if y_local.stride(0) == T:       # contiguous rows of the full output: one long row
                rows, row_bytes, src_pitch, dst_pitch = 1, 2 * n_r * T, 2 * n_r * T, 2 * d_out * T
            else:
                rows, row_bytes, src_pitch, dst_pitch = n_r, 2 * T, 2 * int(y_local.stride(0)), 2 * T
            dst_off = 2 * T * row_off
            shape = (d_out, T)
        if n_r > 0 and T > 0:
            self._push(st, y_local, rows, row_bytes, src_pitch, dst_pitch, dst_off)
        return torch.as_tensor(_DeviceArray(st["own"] + self.FLAG_BYTES, shape, "<f2"), device=self.device)

    def close(self) -> None:
        """Unmap the peers' buffers and free this rank's (call on every rank, after a barrier)."""
        import torch.distributed as dist
        if not self.sets:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for st in self.sets:
                for p in st["opened"]:
                    self._lib.w4a4_peer_close(p)
            dist.barrier(group=self.group)
            for st in self.sets:
                self._lib.w4a4_peer_free(st["own"])
        self.sets = []


def column_parallel_forward(X_fp16: torch.Tensor, shard: V9WeightContainer, d_out: int, group=None,
                            gather: bool = True, exchange: Optional[PeerGather] = None) -> torch.Tensor:
    """Forward of one rank's shard; with ``gather`` the full ``(..., d_out)``
    output is assembled on every rank - through ``exchange`` (peer-memory stores, one
    kernel) when given, else by an NCCL all-gather - otherwise the local
    ``(..., d_out_r)`` slice is returned (the consumer stays shard-aware)."""
    from .v9_linear import v9_linear_forward

    y = v9_linear_forward(X_fp16, shard)
    if not gather:
        return y
    lead = y.shape[:-1]
    if exchange is not None:
        full = exchange.gather(y.reshape(-1, y.shape[-1]), d_out, token_major=True)
    else:
        full = gather_output(y.reshape(-1, y.shape[-1]), d_out, group=group, token_major=True)
    return full.reshape(lead + (d_out,))


__all__ = ["block_row_range", "shard_rows", "shard_sizes", "shard_container", "check_shard_metadata",
           "gather_output", "column_parallel_forward", "PeerGather"]

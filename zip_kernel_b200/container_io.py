"""On-disk format of a W4A4 weight container, and its loader.

The reference keeps its weights only as in-memory ``V9WeightContainer`` objects
(``triton_kernel/pack_utils.py:85-106``) and validates them when they are handed
to a kernel (``backend/weight_loader.py:169-261``); it has no file format.  This
module adds one, so that a packed layer is written once and mapped straight into
pinned memory and onto the GPU afterwards:

    file = magic "W4A4V9C\\0" | u32 version | u32 header bytes | JSON header | padding | tensor data

The JSON header carries ``d_out``, ``d_in``, ``block_shape`` and, per tensor (the
seven container fields), dtype, shape, byte offset, byte count and CRC-32.  Tensor
data starts at a multiple of 4096 bytes and every tensor at a multiple of 256, so
a memory map of the file gives aligned row-major arrays without a copy.  All
integers are little-endian.  The load path is ``mmap -> pinned host -> device``
with every layout rule checked BEFORE anything reaches a kernel: the rules of the
reference's validated view (int8 nibbles, fp16 tables of shape ``(d_out,
d_in/128)``, ``d_in`` a multiple of 128) plus those of the block-CSR index
(offset count, monotonic offsets, column indices inside ``d_in/128``, sorted
inside a block-row, block count).  ``prepare=True`` also builds the e4m3 copy the
many-token kernel can use (it is derived data and is never stored).
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import zlib
from typing import Dict, List, Optional

import numpy as np
import torch

from .backend.weight_loader import CutlassPackValidationError, _collect_violations
from .pack_utils import BCOL, BROW, V9WeightContainer

MAGIC = b"W4A4V9C\x00"
VERSION = 1
DATA_ALIGN = 4096
TENSOR_ALIGN = 256

_FIELDS = ("W_low_packed", "W_high_blocks_packed", "scale_u4", "zero_u4", "hp_row_offsets", "hp_col_indices", "perm")
_DTYPES = {"int8": (torch.int8, np.int8), "float16": (torch.float16, np.float16), "int32": (torch.int32, np.int32)}
_EXPECT = {"W_low_packed": "int8", "W_high_blocks_packed": "int8", "scale_u4": "float16", "zero_u4": "float16",
           "hp_row_offsets": "int32", "hp_col_indices": "int32", "perm": "int32"}


class ContainerFormatError(ValueError):
    """The file is not a container of this format, is truncated or corrupt, or breaks a layout rule."""


def _round_up(v: int, a: int) -> int:
    return (v + a - 1) // a * a


def index_violations(W: V9WeightContainer) -> List[str]:
    """Rules of the block-CSR residual index and of the permutation (complements the dense-tensor rules
    of ``backend.weight_loader``).  Never raises; returns every broken rule."""
    v: List[str] = []
    d_out, d_in = int(W.d_out), int(W.d_in)
    nbr, ng = (d_out + BROW - 1) // BROW, d_in // BCOL if d_in > 0 else 0
    if tuple(W.block_shape) != (BROW, BCOL):
        v.append(f"block_shape must be ({BROW}, {BCOL}), got {tuple(W.block_shape)}")
    ro, ci, wh = W.hp_row_offsets, W.hp_col_indices, W.W_high_blocks_packed
    nnz = int(wh.shape[0]) if wh.dim() == 3 else -1
    if wh.dtype != torch.int8 or wh.dim() != 3 or tuple(wh.shape[1:]) != (BROW, BCOL // 2):
        v.append(f"W_high_blocks_packed must be int8 (nnz, {BROW}, {BCOL // 2}), got {wh.dtype} {tuple(wh.shape)}")
    if ro.dtype != torch.int32 or ro.dim() != 1 or int(ro.numel()) != nbr + 1:
        v.append(f"hp_row_offsets must be int32 with ceil(d_out/128)+1 = {nbr + 1} entries, got {ro.dtype} {tuple(ro.shape)}")
    else:
        r = ro.cpu().to(torch.int64)
        if int(r[0]) != 0:
            v.append(f"hp_row_offsets[0] must be 0, got {int(r[0])}")
        if bool((r[1:] < r[:-1]).any()):
            v.append("hp_row_offsets must be non-decreasing")
        if nnz >= 0 and int(r[-1]) != nnz:
            v.append(f"hp_row_offsets[-1]={int(r[-1])} disagrees with the number of residual blocks {nnz}")
    if ci.dtype != torch.int32 or ci.dim() != 1 or (nnz >= 0 and int(ci.numel()) != nnz):
        v.append(f"hp_col_indices must be int32 with one entry per residual block ({nnz}), got {ci.dtype} {tuple(ci.shape)}")
    elif nnz > 0:
        c = ci.cpu().to(torch.int64)
        if int(c.min()) < 0 or int(c.max()) >= ng:
            v.append(f"hp_col_indices must lie in [0, d_in/128 = {ng}), got [{int(c.min())}, {int(c.max())}]")
        elif ro.dtype == torch.int32 and int(ro.numel()) == nbr + 1 and not v:
            r = ro.cpu().to(torch.int64)
            row_of = torch.repeat_interleave(torch.arange(nbr), (r[1:] - r[:-1]).clamp(min=0))
            key = row_of * max(ng, 1) + c
            if bool((key[1:] <= key[:-1]).any()):
                v.append("residual blocks must be sorted by (block-row, block-col) without duplicates")
    p = W.perm
    if p.dtype != torch.int32 or p.dim() != 1 or int(p.numel()) != d_in:
        v.append(f"perm must be int32 with d_in = {d_in} entries, got {p.dtype} {tuple(p.shape)}")
    elif d_in > 0:
        pc = p.cpu().to(torch.int64)
        if int(pc.min()) < 0 or int(pc.max()) >= d_in:
            v.append(f"perm entries must lie in [0, {d_in})")
    return v


def validate_container(W: V9WeightContainer) -> None:
    """Raises :class:`CutlassPackValidationError` (the reference's exception for a broken layout) listing
    every violated rule of the dense tensors, the residual index and the permutation."""
    violations = _collect_violations(W) + index_violations(W)
    if violations:
        raise CutlassPackValidationError(violations)


def save_container(W: V9WeightContainer, path: str) -> int:
    """Writes ``W`` (any device) to ``path``; returns the file size.  The container is validated first:
    a file of this format always holds a layout the kernels accept."""
    validate_container(W)
    arrays: Dict[str, np.ndarray] = {}
    for name in _FIELDS:
        t = getattr(W, name).detach().cpu().contiguous()
        arrays[name] = t.numpy() if t.numel() else np.zeros(tuple(t.shape), dtype=_DTYPES[_EXPECT[name]][1])
    entries, off = {}, 0
    for name in _FIELDS:
        a = arrays[name]
        off = _round_up(off, TENSOR_ALIGN)
        entries[name] = {"dtype": _EXPECT[name], "shape": [int(s) for s in a.shape], "offset": off,
                         "nbytes": int(a.nbytes), "crc32": zlib.crc32(a.tobytes()) & 0xFFFFFFFF}
        off += a.nbytes
    header = json.dumps({"format": "w4a4-v9-container", "version": VERSION, "d_out": int(W.d_out), "d_in": int(W.d_in),
                         "block_shape": [int(b) for b in W.block_shape], "tensors": entries, "data_bytes": off},
                        sort_keys=True).encode()
    data_start = _round_up(len(MAGIC) + 8 + len(header), DATA_ALIGN)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(MAGIC)
        f.write(struct.pack("<II", VERSION, len(header)))
        f.write(header)
        f.write(b"\0" * (data_start - f.tell()))
        for name in _FIELDS:
            f.write(b"\0" * (data_start + entries[name]["offset"] - f.tell()))
            f.write(arrays[name].tobytes())
    os.replace(tmp, path)            # a reader never sees a half-written file
    return data_start + off


def read_header(path: str) -> dict:
    """Parses and checks the header (magic, version, sizes against the file length); returns it with
    ``data_start`` added."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(len(MAGIC) + 8)
        if len(head) < len(MAGIC) + 8 or head[:len(MAGIC)] != MAGIC:
            raise ContainerFormatError(f"{path}: not a W4A4 container file (bad magic)")
        version, hlen = struct.unpack("<II", head[len(MAGIC):])
        if version != VERSION:
            raise ContainerFormatError(f"{path}: format version {version} is not supported (this reader: {VERSION})")
        if hlen <= 0 or len(MAGIC) + 8 + hlen > size:
            raise ContainerFormatError(f"{path}: header length {hlen} exceeds the file")
        try:
            h = json.loads(f.read(hlen).decode())
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ContainerFormatError(f"{path}: unreadable header ({exc})") from None
    h["data_start"] = _round_up(len(MAGIC) + 8 + hlen, DATA_ALIGN)
    tensors = h.get("tensors", {})
    if set(tensors) != set(_FIELDS):
        raise ContainerFormatError(f"{path}: header lists tensors {sorted(tensors)}, expected {sorted(_FIELDS)}")
    for name, e in tensors.items():
        if e.get("dtype") != _EXPECT[name]:
            raise ContainerFormatError(f"{path}: {name} has dtype {e.get('dtype')}, expected {_EXPECT[name]}")
        n = int(np.prod(e["shape"])) * np.dtype(_DTYPES[e["dtype"]][1]).itemsize if e["shape"] else 0
        if n != int(e["nbytes"]) or int(e["offset"]) % TENSOR_ALIGN != 0:
            raise ContainerFormatError(f"{path}: {name} byte count / alignment disagrees with its shape")
        if h["data_start"] + int(e["offset"]) + int(e["nbytes"]) > size:
            raise ContainerFormatError(f"{path}: truncated ({name} ends beyond the file)")
    return h


def load_container(path: str, device: Optional[torch.device] = None, *, prepare: bool = False,
                   verify_crc: bool = True, pin: bool = True) -> V9WeightContainer:
    """Maps ``path``, checks it (header, sizes, CRC-32 per tensor, every layout rule) and returns the
    container on ``device`` (``None`` or ``"cpu"``: host tensors that own their memory).  For a CUDA
    device the tensors go ``mmap -> pinned host buffer -> device``; ``prepare=True`` then also builds
    the e4m3 copy for the many-token kernel (``prepare_for_prefill``)."""
    h = read_header(path)
    dev = torch.device(device) if device is not None else torch.device("cpu")
    out = {}
    problem = None
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        for name in _FIELDS:
            e = h["tensors"][name]
            tdt, ndt = _DTYPES[e["dtype"]]
            start = h["data_start"] + int(e["offset"])
            view = np.frombuffer(mm, dtype=ndt, count=int(np.prod(e["shape"])) if e["shape"] else 0, offset=start)
            if verify_crc and (zlib.crc32(view) & 0xFFFFFFFF) != int(e["crc32"]):
                problem = f"{path}: checksum mismatch in {name}"
            else:
                host = torch.empty(tuple(e["shape"]), dtype=tdt, pin_memory=bool(pin and dev.type == "cuda" and view.size))
                if view.size:
                    host.view(-1).numpy()[:] = view        # the one host copy: mapped pages -> (pinned) buffer
                out[name] = host
            del view                                       # the map cannot be closed while an array still exports it
            if problem:
                break
        mm.close()
    if problem:
        raise ContainerFormatError(problem)
    W = V9WeightContainer(block_shape=tuple(int(b) for b in h["block_shape"]), d_out=int(h["d_out"]), d_in=int(h["d_in"]),
                          **out)
    try:
        validate_container(W)
    except CutlassPackValidationError as exc:
        raise ContainerFormatError(f"{path}: {exc}") from None
    if dev.type == "cuda":
        W = V9WeightContainer(block_shape=W.block_shape, d_out=W.d_out, d_in=W.d_in,
                              **{n: getattr(W, n).to(dev, non_blocking=True) for n in _FIELDS})
        torch.cuda.current_stream(dev).synchronize()       # the pinned staging buffers may be freed now
        if prepare:
            from .v9_linear import prepare_for_prefill
            prepare_for_prefill(W)
    elif prepare:
        raise ValueError("prepare=True needs a CUDA device")
    return W


__all__ = ["ContainerFormatError", "save_container", "load_container", "read_header", "validate_container",
           "index_violations", "MAGIC", "VERSION"]

"""CPU oracle for the W4A4 fused-linear path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the GPU path is compared against.  It is imported
by the test-suite, by the smoke check and by the benchmark's CPU-baseline leg,
and by nothing else: the product (``zip_kernel_b200``) never imports it and
has no CPU fallback.

Everything here is plain numpy (torch is used only by ``cpu_reference_path``,
the timed dequant->matmul baseline).  Each function restates one piece of the
reference project (HuYangjia/Zip_kernel); the file:line it follows is cited in
its docstring.  Paths are relative to the reference repository root.

Parity pinning: the reference holds no stored golden files, only seeded
synthetic self-consistency tests.  The oracle is therefore pinned against
outputs of the reference's own CPU functions (``tools/parity/*`` and
``triton_kernel/pack_utils.py``) executed on seeded inputs; those outputs are
committed under ``tests/golden/`` together with the generating script, and
``tests/test_oracle_golden.py`` replays them bit for bit.

Contract summary (all sizes: T tokens, K = d_in, N = d_out, ng = K/128):

* activation  : signed int4, symmetric, one fp16 scale per token, codes
                gathered through ``perm``; per-token per-group int32 ``sum_X``.
* dense weight: stored as s4 nibbles (u4 - 8), fp16 ``scale_u4``/``zero_u4`` per
                (row, group-128); ``zero_u4`` already shifted by -8.
* residual    : 128x128 s4 blocks in block-CSR, scaled by ``scale_u4[row, bc]``
                and weighted by 16.
* output      : ``Y[n, t]`` fp16, d_out-major.
"""

from __future__ import annotations

import numpy as np

BROW = 128
BCOL = 128


# ---------------------------------------------------------------------------
# nibble packing  (triton_kernel/pack_utils.py:32-78)
# ---------------------------------------------------------------------------

def pack_s4_le(x: np.ndarray) -> np.ndarray:
    """Pack 4-bit integers two per byte, element 2j in the low nibble.

    Follows triton_kernel/pack_utils.py:32-56: ``byte = (x[2j+1] << 4) |
    (x[2j] & 15)`` stored as signed int8.
    """
    x = np.asarray(x)
    if x.shape[-1] % 2 != 0:
        raise ValueError(f"pack_s4_le requires an even last dim, got {x.shape[-1]}")
    v = x.astype(np.int32)
    lo = v[..., 0::2] & 0x0F
    hi = v[..., 1::2] & 0x0F
    return ((hi << 4) | lo).astype(np.uint8).view(np.int8)


def unpack_s4_le(packed: np.ndarray, signed: bool = True) -> np.ndarray:
    """Inverse of :func:`pack_s4_le` (triton_kernel/pack_utils.py:59-78)."""
    p = np.asarray(packed).view(np.uint8).astype(np.int32)
    out = np.empty(p.shape[:-1] + (p.shape[-1] * 2,), dtype=np.int32)
    out[..., 0::2] = p & 0x0F
    out[..., 1::2] = (p >> 4) & 0x0F
    if signed:
        out = np.where(out >= 8, out - 16, out)
    return out.astype(np.int8)


# ---------------------------------------------------------------------------
# activation quantisation  (tools/parity/quant_reference.py:82-112)
# ---------------------------------------------------------------------------

def quantize_activation_s4(X_fp16: np.ndarray, perm: np.ndarray, bcol: int = BCOL):
    """Per-token symmetric s4 quantisation with per-group code sums.

    Restates tools/parity/quant_reference.py:82-112 (kernel contract:
    cuda_kernel/csrc/activation_quant/activation_quant.cu:6-12):

    ``Xp = X[:, perm]``; ``scale_x = fp16(max|Xp| / 7)``; ``s = fp32(scale_x)``
    (1 when 0); ``q = clamp(rint(Xp / s), -8, 7)`` with IEEE division and
    round-half-even, all-zero codes for a zero-scale row; ``sum_X[t, g]`` is the
    int32 sum of the 128 codes of group g.

    Returns ``(X_s4 (T, K/2) int8, scale_x (T,) fp16, sum_X (T, ng) int32)``.
    """
    X = np.asarray(X_fp16)
    if X.dtype != np.float16:
        raise TypeError(f"X must be fp16, got {X.dtype}")
    if X.ndim == 3:
        X = X.reshape(-1, X.shape[-1])
    elif X.ndim != 2:
        raise ValueError(f"X must be 2D or 3D, got shape {X.shape}")
    T, D = X.shape
    if D % bcol != 0:
        raise ValueError(f"d_in ({D}) must be divisible by bcol ({bcol})")
    Xp = X[:, np.asarray(perm).astype(np.int64)].astype(np.float32)
    max_abs = np.abs(Xp).max(axis=1) if D > 0 else np.zeros((T,), np.float32)
    scale32 = (max_abs / np.float32(7.0)).astype(np.float32)
    scale16 = scale32.astype(np.float16)
    s = scale16.astype(np.float32)
    is_zero = s <= 0.0
    s_safe = np.where(is_zero, np.float32(1.0), s).astype(np.float32)
    q = np.rint(Xp / s_safe[:, None]).clip(-8.0, 7.0).astype(np.int32)
    q[is_zero, :] = 0
    sum_X = q.reshape(T, D // bcol, bcol).sum(axis=-1).astype(np.int32)
    return pack_s4_le(q.astype(np.int8)), scale16, sum_X


# ---------------------------------------------------------------------------
# integer stage: exact int32 accumulators
# ---------------------------------------------------------------------------

def group_accumulators(W_low_packed: np.ndarray, X_s4: np.ndarray) -> np.ndarray:
    """``acc[g, n, t] = sum_{k in group g} W_s4[n, k] * X_s4[t, k]`` as int32.

    This is the ``(n_groups, d_out, T)`` int32 workspace the reference defines
    in cuda_kernel/csrc/fused_dense_sparse/cutlass_dequant.cu:7-16 and the
    per-group accumulator of fused_dense_sparse_mma_int4.cu:595-601.  Products
    and sums stay below 2**24 in magnitude, so a float32 BLAS matmul of the
    small integers is exact.
    """
    W = unpack_s4_le(W_low_packed).astype(np.float32)
    X = unpack_s4_le(X_s4).astype(np.float32)
    N, K = W.shape
    T = X.shape[0]
    ng = K // BCOL
    acc = np.empty((ng, N, T), dtype=np.int32)
    for g in range(ng):
        sl = slice(g * BCOL, (g + 1) * BCOL)
        acc[g] = (W[:, sl] @ X[:, sl].T).astype(np.int32)
    return acc


def block_accumulators(W_high_blocks_packed: np.ndarray, hp_col_indices: np.ndarray,
                       X_s4: np.ndarray) -> np.ndarray:
    """``acc_hi[b, r, t] = sum_c Whigh_s4[b, r, c] * X_s4[t, 128*bc_b + c]`` int32.

    The residual-block accumulator of
    fused_dense_sparse_mma_int4.cu:1021-1115 before its scale fold.
    """
    nnz = int(W_high_blocks_packed.shape[0])
    X = unpack_s4_le(X_s4).astype(np.float32)
    T = X.shape[0]
    out = np.zeros((nnz, BROW, T), dtype=np.int32)
    if nnz == 0:
        return out
    Wh = unpack_s4_le(W_high_blocks_packed).astype(np.float32)
    for b in range(nnz):
        bc = int(hp_col_indices[b])
        out[b] = (Wh[b] @ X[:, bc * BCOL:(bc + 1) * BCOL].T).astype(np.int32)
    return out


# ---------------------------------------------------------------------------
# floating-point stage in the kernel's order
# ---------------------------------------------------------------------------

def _row_block_of(nnz, hp_row_offsets):
    ro = np.asarray(hp_row_offsets).astype(np.int64)
    br = np.zeros((nnz,), dtype=np.int64)
    for r in range(len(ro) - 1):
        br[ro[r]:ro[r + 1]] = r
    return br


def fused_kernel_order(W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
                       X_s4, scale_u4, zero_u4, sum_X, scale_x, d_out, d_in,
                       dtype=np.float32, dense=True, sparse=True, sparse_weight=16.0):
    """Fused linear in the arithmetic order of the reference CUDA kernels.

    Per output ``(n, t)``: for each group g in increasing order
    ``y += (float(acc[g]) - z[n,g] * float(sum_X[t,g])) * s[n,g]``
    (csrc_naive/dense_gemm_naive.cu:277-286; fused_dense_sparse_mma_int4.cu:966-972),
    then for each residual block of the row's block-row in (br, bc) order
    ``y += 16 * float(acc_hi) * s[n, bc]`` (fused_dense_sparse_mma_int4.cu:1099-1104),
    finally ``y *= float(scale_x[t])`` and one round-to-nearest fp16 cast
    (fused_dense_sparse_mma_int4.cu:1120-1129,1176-1178).

    ``dtype=np.float64`` gives the high-precision truth the fp32 kernels are
    measured against; ``dense``/``sparse`` select the two partial products
    (``sparse_weight=1`` reproduces ``sparse_gemm_cuda``, which leaves the
    factor 16 to its caller, cuda_kernel/ops.py:394-408).
    Returns ``Y (d_out, T)`` fp16.
    """
    N, K = int(d_out), int(d_in)
    ng = K // BCOL
    T = int(np.asarray(X_s4).shape[0])
    s = np.asarray(scale_u4).astype(dtype)
    z = np.asarray(zero_u4).astype(dtype) if zero_u4 is not None else None
    y = np.zeros((N, T), dtype=dtype)
    if dense:
        acc = group_accumulators(W_low_packed, X_s4)
        sx = np.asarray(sum_X).astype(dtype)                # (T, ng)
        for g in range(ng):
            corrected = acc[g].astype(dtype) - z[:, g:g + 1] * sx[None, :, g]
            y += corrected * s[:, g:g + 1]
    nnz = int(np.asarray(W_high_blocks_packed).shape[0]) if W_high_blocks_packed is not None else 0
    if sparse and nnz > 0:
        acc_hi = block_accumulators(W_high_blocks_packed, hp_col_indices, X_s4)
        br = _row_block_of(nnz, hp_row_offsets)
        w = dtype(sparse_weight)
        for b in range(nnz):
            r0 = int(br[b]) * BROW
            r1 = min(r0 + BROW, N)
            bc = int(hp_col_indices[b])
            y[r0:r1] += w * acc_hi[b, :r1 - r0].astype(dtype) * s[r0:r1, bc:bc + 1]
    y *= np.asarray(scale_x).astype(dtype)[None, :]
    return y.astype(np.float16)


# ---------------------------------------------------------------------------
# "loose truth": dequantise to fp16, fp32 matmul  (tools/parity/fp16_reference.py)
# ---------------------------------------------------------------------------

def _dequant_w_low_fp16(W_low_packed, scale_u4, zero_u4):
    """tools/parity/fp16_reference.py:71-106."""
    W = unpack_s4_le(W_low_packed).astype(np.float32)
    s = np.repeat(np.asarray(scale_u4).astype(np.float32), BCOL, axis=1)
    z = np.repeat(np.asarray(zero_u4).astype(np.float32), BCOL, axis=1)
    return ((W - z) * s).astype(np.float16)


def _dequant_x_fp16(X_s4, scale_x):
    """tools/parity/fp16_reference.py:109-130."""
    X = unpack_s4_le(X_s4).astype(np.float32)
    return (X * np.asarray(scale_x).astype(np.float32)[:, None]).astype(np.float16)


def _dequant_w_high_fp16(W_high_blocks_packed, hp_row_offsets, hp_col_indices, scale_u4,
                         d_out, d_in):
    """tools/parity/fp16_reference.py:160-217."""
    nnz = int(np.asarray(W_high_blocks_packed).shape[0])
    Wh = np.zeros((d_out, d_in), dtype=np.float32)
    if nnz == 0:
        return Wh.astype(np.float16)
    tiles = unpack_s4_le(W_high_blocks_packed).astype(np.float32)
    s = np.asarray(scale_u4).astype(np.float32)
    br = _row_block_of(nnz, hp_row_offsets)
    for b in range(nnz):
        r0 = int(br[b]) * BROW
        r1 = min(r0 + BROW, d_out)
        bc = int(hp_col_indices[b])
        Wh[r0:r1, bc * BCOL:(bc + 1) * BCOL] = tiles[b, :r1 - r0] * s[r0:r1, bc:bc + 1]
    return Wh.astype(np.float16)


def fp16_dense_reference(W_low_packed, X_s4, scale_u4, zero_u4, scale_x, d_out, d_in):
    """tools/parity/fp16_reference.py:133-157; returns ``Y_low (d_out, T)`` fp16."""
    Wf = _dequant_w_low_fp16(W_low_packed, scale_u4, zero_u4).astype(np.float32)
    Xf = _dequant_x_fp16(X_s4, scale_x).astype(np.float32)
    return np.ascontiguousarray((Xf @ Wf.T).astype(np.float16).T)


def fp16_sparse_reference(W_high_blocks_packed, hp_row_offsets, hp_col_indices, X_s4,
                          scale_u4, scale_x, d_out, d_in):
    """tools/parity/fp16_reference.py:220-243; returns ``Y_high`` without the x16."""
    Wh = _dequant_w_high_fp16(W_high_blocks_packed, hp_row_offsets, hp_col_indices,
                              scale_u4, d_out, d_in).astype(np.float32)
    Xf = _dequant_x_fp16(X_s4, scale_x).astype(np.float32)
    return np.ascontiguousarray((Xf @ Wh.T).astype(np.float16).T)


def fp16_fused_reference(W_low_packed, W_high_blocks_packed, hp_row_offsets, hp_col_indices,
                         X_s4, scale_u4, zero_u4, scale_x, d_out, d_in):
    """tools/parity/fp16_reference.py:246-279: ``fp16(Y_low + 16 * Y_high)``."""
    yl = fp16_dense_reference(W_low_packed, X_s4, scale_u4, zero_u4, scale_x, d_out, d_in)
    yh = fp16_sparse_reference(W_high_blocks_packed, hp_row_offsets, hp_col_indices, X_s4,
                               scale_u4, scale_x, d_out, d_in)
    return (yl.astype(np.float32) + np.float32(16.0) * yh.astype(np.float32)).astype(np.float16)


# ---------------------------------------------------------------------------
# offline packer  (triton_kernel/pack_utils.py:113-264)
# ---------------------------------------------------------------------------

def pack_v9_weights(Q_u4_permuted, scale_u4_raw, zero_u4_raw, Q_s8_blocks, scale_s8_per_block,
                    hp_block_indices, perm):
    """Restates triton_kernel/pack_utils.py:113-264 on numpy arrays.

    Returns a dict with the container fields (``W_low_packed``,
    ``W_high_blocks_packed``, ``scale_u4``, ``zero_u4``, ``hp_row_offsets``,
    ``hp_col_indices``, ``perm``, ``d_out``, ``d_in``).
    """
    Q = np.asarray(Q_u4_permuted).astype(np.int32).copy()
    d_out, d_in = Q.shape
    if d_in % BCOL != 0:
        raise ValueError(f"V9 pack requires d_in ({d_in}) divisible by bcol ({BCOL})")
    ng = d_in // BCOL
    nrow = (d_out + BROW - 1) // BROW
    scale = np.asarray(scale_u4_raw).astype(np.float16).copy()
    zero = np.asarray(zero_u4_raw).astype(np.float16).copy()
    if scale.shape != (d_out, ng) or zero.shape != (d_out, ng):
        raise ValueError("scale_u4_raw / zero_u4_raw must have shape (d_out, n_groups)")
    idx = np.asarray(hp_block_indices).reshape(-1, 2).astype(np.int64)
    n_hp = idx.shape[0]
    tiles = []
    for i in range(n_hp):
        br, bc = int(idx[i, 0]), int(idx[i, 1])
        r0, r1 = br * BROW, min((br + 1) * BROW, d_out)
        c0, c1 = bc * BCOL, min((bc + 1) * BCOL, d_in)
        q8 = np.asarray(Q_s8_blocks[i])[:r1 - r0, :c1 - c0].astype(np.int32)
        qh, ql = q8 >> 4, q8 & 0x0F
        assert np.array_equal(qh * 16 + ql, q8)
        Q[r0:r1, c0:c1] = ql
        t = np.zeros((BROW, BCOL), dtype=np.int32)
        t[:r1 - r0, :c1 - c0] = qh
        tiles.append((br, bc, t))
        scale[r0:r1, bc] = np.asarray(scale_s8_per_block[i])[:r1 - r0].astype(np.float16)
        zero[r0:r1, bc] = 0.0
    W_low_s4 = (Q - 8).astype(np.int8)
    zero = (zero.astype(np.float16) - np.float16(8.0)).astype(np.float16)
    row_offsets = np.zeros((nrow + 1,), dtype=np.int32)
    if n_hp > 0:
        tiles.sort(key=lambda t: (t[0], t[1]))
        brs = np.array([t[0] for t in tiles], dtype=np.int64)
        cols = np.array([t[1] for t in tiles], dtype=np.int32)
        Wh = np.stack([t[2].astype(np.int8) for t in tiles], axis=0)
        row_offsets[1:] = np.cumsum(np.bincount(brs, minlength=nrow)).astype(np.int32)
    else:
        cols = np.zeros((0,), dtype=np.int32)
        Wh = np.zeros((0, BROW, BCOL), dtype=np.int8)
    return {
        "W_low_packed": pack_s4_le(W_low_s4),
        "W_high_blocks_packed": pack_s4_le(Wh),
        "scale_u4": scale,
        "zero_u4": zero,
        "hp_row_offsets": row_offsets,
        "hp_col_indices": cols,
        "perm": np.asarray(perm).astype(np.int32),
        "d_out": d_out,
        "d_in": d_in,
    }


# ---------------------------------------------------------------------------
# module-level fake-quant forward  (triton_kernel/v9_linear.py:491-562)
# ---------------------------------------------------------------------------

def v9_linear_fakequant(X_fp16, W: dict):
    """Restates triton_kernel/v9_linear.py:491-562 (fp16 dequantised weights,
    fake-quantised activations, ``X_dq @ W_fp16.T``); returns ``(..., d_out)``."""
    d_in, d_out = int(W["d_in"]), int(W["d_out"])
    X = np.asarray(X_fp16)
    X2 = X.reshape(-1, d_in)
    Xp = X2[:, np.asarray(W["perm"]).astype(np.int64)]
    w_low = unpack_s4_le(W["W_low_packed"]).astype(np.float32)
    s = np.repeat(np.asarray(W["scale_u4"]).astype(np.float32), BCOL, axis=1)
    z = np.repeat(np.asarray(W["zero_u4"]).astype(np.float32), BCOL, axis=1)
    w = (w_low - z) * s
    nnz = int(W["W_high_blocks_packed"].shape[0])
    if nnz > 0:
        tiles = unpack_s4_le(W["W_high_blocks_packed"]).astype(np.float32)
        br = _row_block_of(nnz, W["hp_row_offsets"])
        sc = np.asarray(W["scale_u4"]).astype(np.float32)
        for b in range(nnz):
            r0 = int(br[b]) * BROW
            r1 = min(r0 + BROW, d_out)
            bc = int(W["hp_col_indices"][b])
            w[r0:r1, bc * BCOL:(bc + 1) * BCOL] += 16.0 * tiles[b, :r1 - r0] * sc[r0:r1, bc:bc + 1]
    w16 = w.astype(np.float16)
    max_abs = np.maximum(np.abs(Xp).max(axis=-1, keepdims=True).astype(np.float16),
                         np.float16(1e-12))
    sx = (max_abs.astype(np.float32) / np.float32(7.0)).astype(np.float16).astype(np.float32)
    sx = np.where(sx > 0, sx, np.float32(1.0))
    q = np.clip(np.rint(Xp.astype(np.float32) / sx), -8.0, 7.0)
    xdq = (q * sx).astype(np.float16)
    y = (xdq.astype(np.float32) @ w16.astype(np.float32).T).astype(np.float16)
    return y.reshape(X.shape[:-1] + (d_out,))


# ---------------------------------------------------------------------------
# the timed CPU baseline: the reference's own CPU path, multi-threaded
# ---------------------------------------------------------------------------

def dequant_u4_to_fp16(W_low_packed: np.ndarray, scale_u4: np.ndarray, zero_u4: np.ndarray) -> np.ndarray:
    """``(d_out, d_in)`` fp16 weight of the reference's W4A16 route: ``(fp16(code) - zero) * scale`` with both
    operations rounded to half precision (triton_kernel/dequant_w4_to_fp16.py:97-121)."""
    codes = unpack_s4_le(np.asarray(W_low_packed)).astype(np.float16)
    z = np.repeat(np.asarray(zero_u4, dtype=np.float16), BCOL, axis=1)
    s = np.repeat(np.asarray(scale_u4, dtype=np.float16), BCOL, axis=1)
    d = (codes.astype(np.float32) - z.astype(np.float32)).astype(np.float16)
    return (d.astype(np.float32) * s.astype(np.float32)).astype(np.float16)


def rmsnorm_fp16(X_fp16: np.ndarray, weight_fp16: np.ndarray, eps: float) -> np.ndarray:
    """fp16 RMSNorm as a decoder layer applies it before a quantised linear:
    ``y = fp16(fp16(x * r) * w)`` with ``r = 1 / sqrt(fp32(mean(x^2)) + eps)`` in fp32 (the PyTorch
    composition ``(x.float() * rsqrt(x.float().pow(2).mean(-1) + eps)).half() * w`` with the mean taken
    exactly and IEEE square root / division).  The reference has no fused form of this step; this is
    the definition the fused RMSNorm + quantisation kernel is checked against, bit for bit."""
    X = np.asarray(X_fp16, dtype=np.float16)
    x64 = X.astype(np.float64)
    ms = ((x64 * x64).sum(axis=-1) / X.shape[-1]).astype(np.float32)
    r = (np.float32(1.0) / np.sqrt(ms + np.float32(eps), dtype=np.float32)).astype(np.float32)
    xn = (X.astype(np.float32) * r[..., None]).astype(np.float16)
    return (xn.astype(np.float32) * np.asarray(weight_fp16, dtype=np.float16).astype(np.float32)).astype(np.float16)


def silu_mul_fp16(gate_fp16: np.ndarray, up_fp16: np.ndarray) -> np.ndarray:
    """The gated activation ahead of the down projection, ``fp16(fp16(silu(gate)) * up)`` with
    ``silu(g) = g / (1 + exp(-g))`` evaluated in double precision and rounded to fp32, then fp16 (the
    PyTorch composition ``F.silu(gate) * up`` on fp16 tensors, made independent of the accuracy of a
    single-precision exponential)."""
    g = np.asarray(gate_fp16, dtype=np.float16).astype(np.float64)
    with np.errstate(over="ignore"):
        s = (g / (1.0 + np.exp(-g))).astype(np.float32).astype(np.float16)
    return (s.astype(np.float32) * np.asarray(up_fp16, dtype=np.float16).astype(np.float32)).astype(np.float16)


def cpu_reference_path(X_fp16_t, perm_t, Wt: dict):
    """The reference's CPU route for one linear, on torch CPU tensors with all
    host threads: ``quantize_activation_s4_reference`` followed by
    ``fp16_fused_reference`` (dequantise both operands to fp16, fp32 matmul,
    fp16 cast; tools/parity/quant_reference.py:82-112 and
    tools/parity/fp16_reference.py:133-279).  Used only for timing; returns
    ``Y (d_out, T)`` fp16 as a torch tensor.
    """
    import torch

    d_out, d_in = int(Wt["d_out"]), int(Wt["d_in"])
    X2 = X_fp16_t.reshape(-1, d_in)
    Xp = X2.index_select(1, perm_t.to(torch.int64)).to(torch.float32)
    s16 = (Xp.abs().amax(dim=1) / 7.0).to(torch.float16)
    s = s16.to(torch.float32)
    zero_row = s <= 0
    s_safe = torch.where(zero_row, torch.ones_like(s), s)
    q = torch.round(Xp / s_safe[:, None]).clamp(-8.0, 7.0)
    q = torch.where(zero_row[:, None], torch.zeros_like(q), q)
    x16 = (q * s[:, None]).to(torch.float16)

    def unpack(p):
        v = p.to(torch.int32) & 0xFF
        out = torch.empty(*v.shape[:-1], v.shape[-1] * 2, dtype=torch.int32)
        out[..., 0::2] = v & 15
        out[..., 1::2] = (v >> 4) & 15
        return torch.where(out >= 8, out - 16, out).to(torch.float32)

    sc = Wt["scale_u4"].to(torch.float32)
    w = ((unpack(Wt["W_low_packed"]) - Wt["zero_u4"].to(torch.float32).repeat_interleave(BCOL, 1))
         * sc.repeat_interleave(BCOL, 1)).to(torch.float16)
    y_low = (x16.to(torch.float32) @ w.to(torch.float32).T).to(torch.float16)
    nnz = int(Wt["W_high_blocks_packed"].shape[0])
    wh = torch.zeros((d_out, d_in), dtype=torch.float32)
    if nnz > 0:
        tiles = unpack(Wt["W_high_blocks_packed"])
        ro = Wt["hp_row_offsets"].tolist()
        ci = Wt["hp_col_indices"].tolist()
        for br in range(len(ro) - 1):
            r0 = br * BROW
            r1 = min(r0 + BROW, d_out)
            for b in range(ro[br], ro[br + 1]):
                bc = ci[b]
                wh[r0:r1, bc * BCOL:(bc + 1) * BCOL] = tiles[b, :r1 - r0] * sc[r0:r1, bc:bc + 1]
    y_high = (x16.to(torch.float32) @ wh.to(torch.float16).to(torch.float32).T).to(torch.float16)
    y = (y_low.to(torch.float32) + 16.0 * y_high.to(torch.float32)).to(torch.float16)
    return y.T.contiguous()

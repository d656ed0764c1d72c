"""Shared helpers of the GPU parity tests."""

import numpy as np
import torch

from oracle import w4a4_oracle as O
from zip_kernel_b200 import synth

ATOL = 1e-2      # fp16 output tolerance stated for the path: max-abs 1e-2 ...
RTOL = 1e-3      # ... plus 1e-3 relative


def np_(t):
    return t.detach().cpu().numpy()


def container_np(W):
    return dict(W_low_packed=np_(W.W_low_packed), W_high_blocks_packed=np_(W.W_high_blocks_packed),
                scale_u4=np_(W.scale_u4), zero_u4=np_(W.zero_u4), hp_row_offsets=np_(W.hp_row_offsets),
                hp_col_indices=np_(W.hp_col_indices), perm=np_(W.perm), d_out=W.d_out, d_in=W.d_in)


def oracle_fused(Wn, xs4, sumx, sx, dtype=np.float32, **kw):
    return O.fused_kernel_order(Wn["W_low_packed"], Wn["W_high_blocks_packed"], Wn["hp_row_offsets"],
                                Wn["hp_col_indices"], xs4, Wn["scale_u4"], Wn["zero_u4"], sumx, sx,
                                Wn["d_out"], Wn["d_in"], dtype=dtype, **kw)


def assert_close_fp16(got, ref, what=""):
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    err = np.abs(got - ref)
    tol = ATOL + RTOL * np.abs(ref)
    bad = err > tol
    assert not bad.any(), (
        f"{what}: {int(bad.sum())} of {bad.size} outside max-abs {ATOL} + rel {RTOL}; "
        f"worst |d|={err.max():.4g} at ref={ref.flat[int(err.argmax())]:.4g}")


def make_case(T, N, K, density, perm_seed=None, seed_offset=0, **kw):
    seed = synth.shape_seed(T, K, N) + seed_offset
    W = synth.make_container(N, K, density, seed=seed, perm_seed=perm_seed, **kw)
    X = synth.make_activations(T, K, seed=seed + 1)
    return W, X


def cuda_container(W):
    return W.to(torch.device("cuda"))


def assert_kernels_agree(Y_a, Y_b, what, W=None, q=None, names=("first", "second")):
    """Two kernels' outputs ``(N, T)`` of the same problem within the fp16 tolerance of each other.  When they
    are not, the message says where they differ, what the device error word holds, and - given the CPU container
    ``W`` and the quantised activations ``q`` - how far each of them is from the oracle on the block-rows
    concerned, so that a failure names the kernel at fault."""
    a, b = np_(Y_a).astype(np.float32), np_(Y_b).astype(np.float32)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    bad = np.abs(a - b) > ATOL + RTOL * np.abs(b)
    if not bad.any():
        return
    from zip_kernel_b200 import _lib
    from zip_kernel_b200.pack_utils import BROW, V9WeightContainer
    rows, toks = np.nonzero(bad)
    lines = [f"{what}: {int(bad.sum())} of {bad.size} outside max-abs {ATOL} + rel {RTOL}; worst |d|={np.abs(a - b).max():.4g}",
             f"  device error word {_lib.device_error(torch.device('cuda')):#x}",
             f"  rows {sorted(set(rows.tolist()))[:48]} tokens {sorted(set(toks.tolist()))[:48]}"]
    if W is not None and q is not None:
        xs4, sx, sumx = (np_(t) for t in q)
        for br in sorted(set((rows // BROW).tolist()))[:4]:
            r0, r1 = br * BROW, min((br + 1) * BROW, W.d_out)
            off = W.hp_row_offsets[br:br + 2].clone()
            b0, b1 = int(off[0]), int(off[1])
            Ws = V9WeightContainer(
                W_low_packed=W.W_low_packed[r0:r1].contiguous(), W_high_blocks_packed=W.W_high_blocks_packed[b0:b1].contiguous(),
                scale_u4=W.scale_u4[r0:r1].contiguous(), zero_u4=W.zero_u4[r0:r1].contiguous(),
                hp_row_offsets=(off - b0).to(torch.int32), hp_col_indices=W.hp_col_indices[b0:b1].contiguous(),
                perm=W.perm, block_shape=W.block_shape, d_out=r1 - r0, d_in=W.d_in)
            ref = oracle_fused(container_np(Ws), xs4, sumx, sx)
            for nm, y in zip(names, (a, b)):
                d = np.abs(y[r0:r1] - ref)
                lines.append(f"  block-row {br}: {nm} kernel vs oracle: worst {d.max():.4g}, {int((d > ATOL + RTOL * np.abs(ref)).sum())} outside")
    raise AssertionError("\n".join(lines))

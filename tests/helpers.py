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

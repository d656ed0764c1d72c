"""The paired-CTA instantiation of the many-token kernel (tcgen05 cta_group::2, selected with
W4A4_PREFILL_PAIR=1): integer accumulators bit-exact against the oracle, outputs bit-identical to the
one-CTA-per-tile kernel (same fold order), on shapes with an odd number of block-rows (a pair with a
phantom second row), ragged rows and tokens, residual columns that the two rows of a pair share, have
alone, or lack, and on prepared weights."""

import os

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import assert_close_fp16, container_np, make_case, np_, oracle_fused

pytestmark = pytest.mark.gpu


@pytest.fixture()
def pair_env():
    old = os.environ.get("W4A4_PREFILL_PAIR")

    def set_(v):
        os.environ["W4A4_PREFILL_PAIR"] = v
    yield set_
    if old is None:
        os.environ.pop("W4A4_PREFILL_PAIR", None)
    else:
        os.environ["W4A4_PREFILL_PAIR"] = old


@pytest.mark.parametrize("T,N,K,density,prepared", [
    (128, 256, 128, 0.0, False), (64, 128, 256, 0.0, False), (128, 256, 512, 1.0, False), (300, 640, 1024, 0.3, False),
    (129, 384, 2048, 0.1, False), (40, 200, 384, 0.5, False), (300, 640, 1024, 0.3, True), (129, 384, 2048, 0.1, True),
    (2048, 1024, 4096, 0.05, False), (700, 1152, 14336, 0.05, True),
])
def test_pair_kernel_equals_single_cta_kernel_and_oracle(pair_env, T, N, K, density, prepared):
    from zip_kernel_b200 import _lib, ops
    dev = torch.device("cuda")
    W, X = make_case(T, N, K, density, perm_seed=3)
    Wd = W.to(dev)
    Wn = container_np(W)
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    prep = (ops.prepare_weights_cuda(Wd.W_low_packed), ops.prepare_weights_cuda(Wd.W_high_blocks_packed)) if prepared else None
    args = (Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices)

    def fused():
        return ops.fused_dense_sparse_cuda(*args, q[0], Wd.scale_u4, Wd.zero_u4, q[2], q[1], N, K, force="tensor", prepared=prep)

    pair_env("1")
    Yp = fused()
    small = T * N * K <= 2 ** 28
    if small:
        acc, acc_hi = ops.dump_accumulators(*args, q[0], N, K, force="tensor", prepared=prep)
    pair_env("0")
    Y1 = fused()
    assert torch.equal(Yp, Y1)
    assert _lib.device_error(dev) == 0
    if small:
        xs4, sx, sumx = (np_(t) for t in q)
        assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], xs4))
        assert np.array_equal(np_(acc_hi), O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4))
        if T * N * K <= 2 ** 27:
            assert_close_fp16(np_(Yp), oracle_fused(Wn, xs4, sumx, sx), "pair kernel vs oracle")

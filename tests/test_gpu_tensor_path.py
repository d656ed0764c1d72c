"""GPU parity of the tcgen05 tensor-core kernel (forced with force="tensor"),
against the CPU oracle: int32 accumulators bit-exact, fp16 outputs within
max-abs 1e-2 + rel 1e-3, and agreement with the weight-streaming kernel."""

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from tests.helpers import assert_close_fp16, container_np, cuda_container, make_case, np_, oracle_fused

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from zip_kernel_b200 import ops as _ops
    return _ops


@pytest.fixture(autouse=True)
def _no_device_error():
    yield
    from zip_kernel_b200 import _lib
    assert _lib.device_error(torch.device("cuda")) == 0, "a bounded device-side wait gave up"


@pytest.mark.parametrize("T,N,K,density", [(128, 128, 128, 0.0), (128, 256, 512, 0.3), (40, 128, 384, 1.0),
                                           (200, 200, 256, 0.5), (1, 256, 256, 0.5)])
def test_tensor_accumulators_bit_exact(ops, T, N, K, density):
    W, X = make_case(T, N, K, density)
    Wn, Wc = container_np(W), cuda_container(W)
    xs4, _, _ = O.quantize_activation_s4(np_(X), Wn["perm"])
    acc, acc_hi = ops.dump_accumulators(Wc.W_low_packed, Wc.W_high_blocks_packed, Wc.hp_row_offsets,
                                        Wc.hp_col_indices, torch.from_numpy(xs4).cuda(), N, K, force="tensor")
    assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], xs4))
    ref_hi = O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4)
    got = np_(acc_hi)
    if N % 128:
        counts = np.diff(Wn["hp_row_offsets"])
        br = np.repeat(np.arange(len(counts)), counts)
        pad = (br[:, None] * 128 + np.arange(128)[None, :]) >= N
        got, ref_hi = got.copy(), ref_hi.copy()
        got[pad] = 0
        ref_hi[pad] = 0
    assert np.array_equal(got, ref_hi)


CASES = [(128, 128, 128, 0.0, None), (256, 256, 256, 0.3, 2), (129, 384, 512, 0.2, None), (17, 128, 256, 0.5, None),
         (300, 200, 384, 0.3, 5), (512, 1024, 1024, 0.05, None), (64, 512, 2048, 0.1, 3), (130, 256, 17408, 0.02, None)]


@pytest.mark.parametrize("T,N,K,density,perm_seed", CASES)
def test_tensor_path_vs_oracle(ops, T, N, K, density, perm_seed):
    W, X = make_case(T, N, K, density, perm_seed)
    Wn, Wc = container_np(W), cuda_container(W)
    xs4, sx, sumx = O.quantize_activation_s4(np_(X), Wn["perm"])
    ref = oracle_fused(Wn, xs4, sumx, sx)
    q4, qs, qsum = ops.activation_quant_cuda(X.cuda(), Wc.perm)
    args = (Wc.W_low_packed, Wc.W_high_blocks_packed, Wc.hp_row_offsets, Wc.hp_col_indices, q4, Wc.scale_u4,
            Wc.zero_u4, qsum, qs, N, K)
    Y = ops.fused_dense_sparse_cuda(*args, force="tensor")
    assert_close_fp16(np_(Y), ref, "tensor fused")
    Ys = ops.fused_dense_sparse_cuda(*args, force="stream")
    assert_close_fp16(np_(Y), np_(Ys), "tensor vs streaming kernel")
    Yt = ops.fused_dense_sparse_cuda(*args, force="tensor", token_major=True)
    assert Yt.shape == (T, N) and torch.equal(Yt.t().contiguous(), Y)
    Yd = ops.dense_gemm_cuda(Wc.W_low_packed, q4, Wc.scale_u4, Wc.zero_u4, qsum, qs, force="tensor")
    assert_close_fp16(np_(Yd), oracle_fused(Wn, xs4, sumx, sx, sparse=False), "tensor dense")
    Yh = ops.sparse_gemm_cuda(Wc.W_high_blocks_packed, Wc.hp_row_offsets, Wc.hp_col_indices, q4, Wc.scale_u4, qs,
                              N, K, force="tensor")
    assert_close_fp16(np_(Yh), oracle_fused(Wn, xs4, sumx, sx, dense=False, sparse_weight=1.0), "tensor sparse")
    Ye = ops.fused_dense_sparse_e2e_cuda(X.cuda(), Wc.perm, Wc.W_low_packed, Wc.W_high_blocks_packed,
                                         Wc.hp_row_offsets, Wc.hp_col_indices, Wc.scale_u4, Wc.zero_u4, N, K,
                                         force="tensor")
    assert torch.equal(Ye, Y)


def test_tensor_path_run_to_run(ops):
    W, X = make_case(256, 512, 1024, 0.1)
    Wc = cuda_container(W)
    outs = [ops.fused_dense_sparse_e2e_cuda(X.cuda(), Wc.perm, Wc.W_low_packed, Wc.W_high_blocks_packed,
                                            Wc.hp_row_offsets, Wc.hp_col_indices, Wc.scale_u4, Wc.zero_u4, 512, 1024,
                                            force="tensor") for _ in range(3)]
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])

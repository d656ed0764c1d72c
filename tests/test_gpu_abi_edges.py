"""Edges of the C ABI that the operator layer does not reach by itself: strided and
misaligned activation rows, the fused-quant wrappers with their token-count checks, and a
bounded device-side wait that is made to run out."""

import ctypes

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import assert_close_fp16, container_np, make_case, np_, oracle_fused

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from zip_kernel_b200 import ops as _ops
    return _ops


@pytest.mark.parametrize("T,K,ldx_extra,x_off,perm_off,use_perm", [
    (5, 512, 24, 0, 0, True),      # ldx > K, rows still 16-byte aligned
    (5, 512, 3, 0, 0, True),       # ldx not a multiple of 8: rows lose the alignment of 128-bit loads
    (3, 1024, 0, 1, 0, False),     # base pointer 2 bytes off, identity order
    (3, 1024, 5, 1, 1, True),      # everything at once, permutation array 4 bytes off
    (40, 256, 8, 0, 1, True),      # one CTA per token and a misaligned permutation
])
def test_quant_strided_and_misaligned_through_the_c_abi(ops, T, K, ldx_extra, x_off, perm_off, use_perm):
    from zip_kernel_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(T * 1000 + K + ldx_extra)
    ldx = K + ldx_extra
    backing = torch.randn(T * ldx + 8, generator=g).half().to(dev)
    X = backing[x_off:x_off + T * ldx].view(T, ldx)[:, :K]            # rows ldx apart, start x_off halfs in
    assert X.data_ptr() % 16 == (2 * x_off) % 16
    perm_full = torch.randperm(K, generator=g).to(torch.int32)
    perm_buf = torch.zeros(K + 4, dtype=torch.int32, device=dev)
    perm_buf[perm_off:perm_off + K] = perm_full.to(dev)
    perm = perm_buf[perm_off:perm_off + K]
    X_s4 = torch.empty((T, K // 2), dtype=torch.int8, device=dev)
    sx = torch.empty((T,), dtype=torch.float16, device=dev)
    sumx = torch.empty((T, K // 128), dtype=torch.int32, device=dev)
    rc = lib.w4a4_activation_quant(X.data_ptr(), ldx, perm.data_ptr() if use_perm else None, X_s4.data_ptr(),
                                   sx.data_ptr(), sumx.data_ptr(), T, K, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.w4a4_last_error()
    r4, rs, rsum = O.quantize_activation_s4(np_(X), np_(perm_full) if use_perm else np.arange(K, dtype=np.int32))
    assert np.array_equal(np_(X_s4), r4)
    assert np.array_equal(np_(sx).view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(np_(sumx), rsum)
    # the operator wrapper hands a row-strided view to the kernel as it is
    if x_off == 0:
        q = ops.activation_quant_cuda(X, perm_full.to(dev) if use_perm else torch.arange(K, dtype=torch.int32, device=dev))
        assert np.array_equal(np_(q[0]), r4)


def test_fused_quant_strided_rows_through_the_c_abi(ops):
    from zip_kernel_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    T, N, K = 6, 384, 1024
    W, Xc = make_case(T, N, K, 0.2, perm_seed=21)
    Wd = W.to(dev)
    ldx = K + 11
    backing = torch.zeros(T * ldx + 8, dtype=torch.float16, device=dev)
    X = backing[1:1 + T * ldx].view(T, ldx)[:, :K]
    X.copy_(Xc.to(dev))
    Y = torch.empty((N, T), dtype=torch.float16, device=dev)
    ws = _lib.workspace(dev, T, K, N, Wd.n_hp_blocks)
    rc = lib.w4a4_fused_quant_dense_sparse(
        X.data_ptr(), ldx, Wd.perm.data_ptr(), Wd.W_low_packed.data_ptr(), Wd.W_high_blocks_packed.data_ptr(),
        Wd.hp_row_offsets.data_ptr(), Wd.hp_col_indices.data_ptr(), Wd.scale_u4.data_ptr(), Wd.zero_u4.data_ptr(),
        Y.data_ptr(), T, K, N, Wd.n_hp_blocks, 0, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.w4a4_last_error()
    r4, rs, rsum = O.quantize_activation_s4(Xc.numpy(), W.perm.numpy())
    assert_close_fp16(np_(Y), oracle_fused(container_np(W), r4, rsum, rs), "fused quant, strided rows")


def test_fused_quant_wrappers(ops):
    """fused_quant_gemv_cuda (exactly one token) and fused_quant_dense_sparse_cuda_int4 (two or more), with
    the ValueErrors the reference raises for the wrong token count (cuda_kernel/ops.py:500-501,591-595)."""
    dev = torch.device("cuda")
    N, K = 640, 1536
    W, X = make_case(5, N, K, 0.25, perm_seed=22)
    Wd = W.to(dev)
    args = (Wd.perm, Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
            Wd.scale_u4, Wd.zero_u4, N, K)
    Wn = container_np(W)
    Xd = X.to(dev)
    y1 = ops.fused_quant_gemv_cuda(Xd[:1], *args)
    assert y1.shape == (N, 1)
    r4, rs, rsum = O.quantize_activation_s4(X[:1].numpy(), W.perm.numpy())
    assert_close_fp16(np_(y1), oracle_fused(Wn, r4, rsum, rs), "fused_quant_gemv")
    y5 = ops.fused_quant_dense_sparse_cuda_int4(Xd, *args)
    assert y5.shape == (N, 5)
    r4, rs, rsum = O.quantize_activation_s4(X.numpy(), W.perm.numpy())
    assert_close_fp16(np_(y5), oracle_fused(Wn, r4, rsum, rs), "fused_quant_dense_sparse")
    y3d = ops.fused_quant_dense_sparse_cuda_int4(Xd[:4].reshape(2, 2, K), *args)
    assert torch.equal(y3d, y5[:, :4])
    with pytest.raises(ValueError):
        ops.fused_quant_gemv_cuda(Xd[:2], *args)
    with pytest.raises(ValueError):
        ops.fused_quant_dense_sparse_cuda_int4(Xd[:1], *args)


def test_bounded_wait_gives_up_and_the_context_survives(ops):
    """A wait on a barrier nobody arrives on runs out after its poll limit, the kernel records the error
    word and returns; the host reads W4A4_ERR_DEVICE once, the word is cleared, and the next call works."""
    from zip_kernel_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda")
    assert _lib.device_error(dev) == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.w4a4_selftest_bounded_wait(3000, stream) == 0
    word = ctypes.c_int(0)
    rc = lib.w4a4_device_error(ctypes.byref(word), stream)
    assert rc == 5                                             # W4A4_ERR_DEVICE
    assert word.value & 0x40000000 and (word.value >> 8) & 0xff == 0x7e
    assert lib.w4a4_device_error(ctypes.byref(word), stream) == 0 and word.value == 0
    assert lib.w4a4_selftest_bounded_wait(0, stream) == 1      # argument check
    W, X = make_case(4, 256, 512, 0.2)
    Wd = W.to(dev)
    q = ops.activation_quant_cuda(X.to(dev), Wd.perm)
    Y = ops.fused_dense_sparse_cuda(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
                                    q[0], Wd.scale_u4, Wd.zero_u4, q[2], q[1], 256, 512)
    xs4, sx, sumx = (np_(t) for t in q)
    assert_close_fp16(np_(Y), oracle_fused(container_np(W), xs4, sumx, sx), "call after a timed-out wait")
    assert _lib.device_error(dev) == 0


def test_last_error_is_cleared_by_a_successful_call(ops):
    from zip_kernel_b200 import _lib
    lib = _lib.load()
    assert lib.w4a4_selftest_bounded_wait(0, None) == 1 and lib.w4a4_last_error()
    word = ctypes.c_int(0)
    assert lib.w4a4_device_error(ctypes.byref(word), torch.cuda.current_stream().cuda_stream) == 0
    assert lib.w4a4_last_error() == b""

"""The many-token kernel's third instantiation: fp8 MMAs on PACKED weights.  A nibble with bit 3 flipped,
alone in its byte, is the e4m3 number (code + 8) * 2^-9 (subnormals and the first binade are one linear
ramp), so the weights are widened with the same three logic operations as for the integer MMAs and the
accumulators hold 2^-9 * (acc + 8 * sumX) exactly; the offset leaves with the zero-point term.  Opt-in
(W4A4_PREFILL_F8=1, or activation codes expanded as ``e4m3="packed"``)."""

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


def base(Wd):
    return (Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices)


@pytest.mark.parametrize("T,N,K,density", [(300, 200, 384, 0.3), (129, 384, 1024, 0.1), (64, 128, 128, 1.0), (40, 256, 2176, 0.0)])
def test_accumulators_bit_exact(ops, T, N, K, density):
    """Subnormal e4m3 operands are exact on the tensor core: with the offset taken out the accumulators are
    the integers of the oracle, dense groups and residual blocks alike."""
    W, X = make_case(T, N, K, density, perm_seed=6)
    Wd = W.to(torch.device("cuda"))
    Wn = container_np(W)
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    acc, acc_hi = ops.dump_accumulators(*base(Wd), q[0], N, K, force="tensor", e4m3_packed=True)
    xs4 = np_(q[0])
    assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], xs4))
    assert np.array_equal(np_(acc_hi), O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4))


@pytest.mark.parametrize("T,N,K,density", [(300, 200, 384, 0.3), (257, 640, 2048, 0.0), (512, 384, 4096, 0.15)])
def test_outputs_against_oracle_and_between_entry_points(ops, monkeypatch, T, N, K, density):
    W, X = make_case(T, N, K, density, perm_seed=8)
    Wd = W.to(torch.device("cuda"))
    Xd = X.cuda()
    q = ops.activation_quant_cuda(Xd, Wd.perm)
    tail = (Wd.scale_u4, Wd.zero_u4, q[1], N, K)
    XE, sumxf = ops.expand_activations_cuda(q[0], q[2], e4m3="packed")
    Yx = ops.fused_dense_sparse_expanded_cuda(*base(Wd), XE, sumxf, *tail, e4m3="packed")
    xs4, sx, sumx = (np_(t) for t in q)
    assert_close_fp16(np_(Yx), oracle_fused(container_np(W), xs4, sumx, sx), "fp8 on packed weights vs oracle")
    monkeypatch.setenv("W4A4_PREFILL_F8", "1")
    Yo = ops.fused_dense_sparse_cuda(*base(Wd), q[0], Wd.scale_u4, Wd.zero_u4, q[2], q[1], N, K, force="tensor")
    Ye = ops.fused_dense_sparse_e2e_cuda(Xd, Wd.perm, *base(Wd), Wd.scale_u4, Wd.zero_u4, N, K, force="tensor")
    assert torch.equal(Yo, Yx) and torch.equal(Ye, Yx)
    monkeypatch.setenv("W4A4_PREFILL_F8", "0")
    Yi = ops.fused_dense_sparse_cuda(*base(Wd), q[0], Wd.scale_u4, Wd.zero_u4, q[2], q[1], N, K, force="tensor")
    # the integer instantiation folds acc * s, this one (acc + 8 sumX) * s - (8 s) sumX: same value, other rounding
    assert_close_fp16(np_(Yx), np_(Yi).astype(np.float32), "fp8 on packed weights vs integer MMAs")


def test_code_formats_are_not_mixed(ops):
    T, N, K = 192, 256, 512
    W, X = make_case(T, N, K, 0.1)
    Wd = W.to(torch.device("cuda"))
    prep = (ops.prepare_weights_cuda(Wd.W_low_packed), ops.prepare_weights_cuda(Wd.W_high_blocks_packed))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    tail = (Wd.scale_u4, Wd.zero_u4, q[1], N, K)
    XEp, sp = ops.expand_activations_cuda(q[0], q[2], e4m3="packed")
    XEn, sn = ops.expand_activations_cuda(q[0], q[2], e4m3=True)
    assert not torch.equal(XEp, XEn)                                   # another byte order inside every packed word
    with pytest.raises(ValueError):                                    # codes for packed weights + prepared weights
        ops.fused_dense_sparse_expanded_cuda(*base(Wd), XEp, sp, *tail, prepared=prep, e4m3="packed")
    with pytest.raises(ValueError):                                    # codes for prepared weights, none given
        ops.fused_dense_sparse_expanded_cuda(*base(Wd), XEn, sn, *tail, e4m3=True)
    with pytest.raises(ValueError):                                    # e4m3 codes cannot be streamed
        ops.fused_dense_sparse_expanded_cuda(*base(Wd), XEp, sp, *tail, e4m3="packed", force="stream")
    with pytest.raises(ValueError):
        ops.expand_activations_cuda(q[0], q[2], e4m3="natural")


def test_full_size_qkv(ops):
    T, K, N = 2048, 4096, 6144
    W, X = make_case(T, N, K, 0.05, perm_seed=9)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    tail = (Wd.scale_u4, Wd.zero_u4, q[1], N, K)
    XE, sumxf = ops.expand_activations_cuda(q[0], q[2], e4m3="packed")
    Yx = ops.fused_dense_sparse_expanded_cuda(*base(Wd), XE, sumxf, *tail, e4m3="packed")
    XE8, sumxf8 = ops.expand_activations_cuda(q[0], q[2])
    Yi = ops.fused_dense_sparse_expanded_cuda(*base(Wd), XE8, sumxf8, *tail, force="tensor")
    assert_close_fp16(np_(Yx), np_(Yi).astype(np.float32), "fp8 on packed weights vs integer MMAs, full size")
    from zip_kernel_b200 import _lib
    assert _lib.device_error(torch.device("cuda")) == 0

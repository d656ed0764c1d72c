"""The many-token kernel's two instantiations - integer MMAs on s8 codes against the packed
nibbles, and fp8 MMAs (tcgen05 kind::f8f6f4, fp32 accumulation) on weights prepared once as e4m3
bytes - must give the same accumulators and the same output bits: the products and sums are small
integers, exact in fp32."""

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import assert_close_fp16, assert_kernels_agree, container_np, make_case, np_, oracle_fused

pytestmark = pytest.mark.gpu

# e4m3 encodings (sign, 4 exponent bits of bias 7, 3 mantissa bits) of the integers -8..7
E4M3 = {0: 0x00, 1: 0x38, 2: 0x40, 3: 0x44, 4: 0x48, 5: 0x4A, 6: 0x4C, 7: 0x4E, 8: 0x50}


def e4m3_of_codes(codes):
    table = np.array([(0x80 | E4M3[-v]) if v < 0 else E4M3[v] for v in range(-8, 8)], dtype=np.uint8)
    return table[np.asarray(codes, dtype=np.int64) + 8]


def prepared_reference(packed):
    """One e4m3 byte per code, codes in their natural order (byte b of the packed array holds codes 2b, 2b + 1)."""
    b = np.ascontiguousarray(packed).view(np.uint8)
    lo = (b & 0xF).astype(np.int8)
    hi = (b >> 4).astype(np.int8)
    lo = np.where(lo >= 8, lo - 16, lo)
    hi = np.where(hi >= 8, hi - 16, hi)
    out = np.stack([e4m3_of_codes(lo), e4m3_of_codes(hi)], axis=-1)                 # (..., bytes, 2)
    return out.reshape(packed.shape[:-1] + (packed.shape[-1] * 2,))


@pytest.fixture(scope="module")
def ops():
    from zip_kernel_b200 import ops as _ops
    return _ops


def prepare(ops, Wd):
    return ops.prepare_weights_cuda(Wd.W_low_packed), ops.prepare_weights_cuda(Wd.W_high_blocks_packed)


def fused(ops, Wd, q, **kw):
    return ops.fused_dense_sparse_cuda(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
                                       q[0], Wd.scale_u4, Wd.zero_u4, q[2], q[1], Wd.d_out, Wd.d_in, **kw)


def test_prepared_bytes(ops):
    W, _ = make_case(4, 300, 512, 0.2)
    Wd = W.to(torch.device("cuda"))
    lo, hi = prepare(ops, Wd)
    assert lo.shape == (300, 512) and hi.shape == (W.W_high_blocks_packed.shape[0], 128, 128)
    assert np.array_equal(np_(lo), prepared_reference(np_(W.W_low_packed)))
    assert np.array_equal(np_(hi), prepared_reference(np_(W.W_high_blocks_packed)))
    # every code value in every nibble position
    allv = torch.arange(256, dtype=torch.uint8).view(torch.int8).repeat(4).reshape(8, 128).cuda()
    assert np.array_equal(np_(ops.prepare_weights_cuda(allv)), prepared_reference(np_(allv)))


@pytest.mark.parametrize("T,N,K,density", [(300, 200, 384, 0.3), (129, 384, 1024, 0.1), (64, 128, 128, 1.0)])
def test_prepared_accumulators_bit_exact(ops, T, N, K, density):
    W, X = make_case(T, N, K, density, perm_seed=6)
    Wd = W.to(torch.device("cuda"))
    Wn = container_np(W)
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    acc, acc_hi = ops.dump_accumulators(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
                                        q[0], N, K, force="tensor", prepared=prepare(ops, Wd))
    xs4 = np_(q[0])
    assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], xs4))
    assert np.array_equal(np_(acc_hi), O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4))


@pytest.mark.parametrize("T,N,K,density", [(300, 200, 384, 0.3), (2048, 1024, 4096, 0.05), (257, 6144, 2048, 0.0)])
def test_prepared_outputs_equal_packed(ops, T, N, K, density):
    W, X = make_case(T, N, K, density, perm_seed=8)
    Wd = W.to(torch.device("cuda"))
    prep = prepare(ops, Wd)
    Xd = X.cuda()
    q = ops.activation_quant_cuda(Xd, Wd.perm)
    Yp = fused(ops, Wd, q, force="tensor")                       # packed weights, integer MMAs
    Yf = fused(ops, Wd, q, force="tensor", prepared=prep)        # prepared weights, fp8 MMAs
    assert torch.equal(Yf, Yp)
    XE8, sumxf8 = ops.expand_activations_cuda(q[0], q[2])        # the same through caller-expanded s8 codes
    Yi = ops.fused_dense_sparse_expanded_cuda(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets,
                                              Wd.hp_col_indices, XE8, sumxf8, Wd.scale_u4, Wd.zero_u4, q[1], N, K,
                                              force="tensor")
    assert torch.equal(Yi, Yp)
    args = (Xd, Wd.perm, Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
            Wd.scale_u4, Wd.zero_u4, N, K)
    Ye = ops.fused_dense_sparse_e2e_cuda(*args, force="tensor", prepared=prep)
    assert torch.equal(Ye, Yp)
    Yt = ops.fused_dense_sparse_e2e_cuda(*args, force="tensor", prepared=prep, token_major=True)
    assert torch.equal(Yt.t(), Yp)
    XE, sumxf = ops.expand_activations_cuda(q[0], q[2], e4m3=True)
    Yx = ops.fused_dense_sparse_expanded_cuda(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets,
                                              Wd.hp_col_indices, XE, sumxf, Wd.scale_u4, Wd.zero_u4, q[1], N, K,
                                              force="tensor", prepared=prep, e4m3=True)
    assert torch.equal(Yx, Yp)
    if T <= 512:
        xs4, sx, sumx = (np_(t) for t in q)
        assert_close_fp16(np_(Yf), oracle_fused(container_np(W), xs4, sumx, sx), "prepared vs oracle")


def test_prepared_few_tokens_take_the_packed_stream(ops):
    T, N, K = 8, 512, 1024
    W, X = make_case(T, N, K, 0.1, perm_seed=1)
    Wd = W.to(torch.device("cuda"))
    prep = prepare(ops, Wd)
    args = (X.cuda(), Wd.perm, Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
            Wd.scale_u4, Wd.zero_u4, N, K)
    assert torch.equal(ops.fused_dense_sparse_e2e_cuda(*args, prepared=prep), ops.fused_dense_sparse_e2e_cuda(*args))


def test_prepared_full_size_gate_up(ops):
    T, K, N = 2048, 4096, 28672
    W, X = make_case(T, N, K, 0.05, perm_seed=9)
    Wd = W.to(torch.device("cuda"))
    prep = prepare(ops, Wd)
    args = (X.cuda(), Wd.perm, Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
            Wd.scale_u4, Wd.zero_u4, N, K)
    assert torch.equal(ops.fused_dense_sparse_e2e_cuda(*args, prepared=prep), ops.fused_dense_sparse_e2e_cuda(*args))
    from zip_kernel_b200 import _lib
    assert _lib.device_error(torch.device("cuda")) == 0


def test_expanded_code_format_is_what_the_flag_says(ops):
    """The flag alone tells the library which bytes XE holds.  Prepared weights with s8 codes, e4m3 codes
    without prepared weights, and e4m3 codes forced onto the streaming kernel are argument errors; e4m3
    codes with prepared weights run the tensor-core kernel at any token count (64..255 included, where the
    cost model may prefer the streaming kernel for s8 codes)."""
    for T, N, K in ((8, 256, 512), (100, 28672, 512), (192, 4096, 4096)):
        W, X = make_case(T, N, K, 0.1)
        Wd = W.to(torch.device("cuda"))
        prep = prepare(ops, Wd)
        q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
        XE, sumxf = ops.expand_activations_cuda(q[0], q[2], e4m3=True)
        XE8, sumxf8 = ops.expand_activations_cuda(q[0], q[2])
        base = (Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices)
        tail = (Wd.scale_u4, Wd.zero_u4, q[1], N, K)
        with pytest.raises(ValueError):          # s8 codes + prepared weights
            ops.fused_dense_sparse_expanded_cuda(*base, XE8, sumxf8, *tail, prepared=prep)
        with pytest.raises(ValueError):          # e4m3 codes, no prepared weights
            ops.fused_dense_sparse_expanded_cuda(*base, XE, sumxf, *tail, e4m3=True)
        with pytest.raises(ValueError):          # e4m3 codes cannot be streamed
            ops.fused_dense_sparse_expanded_cuda(*base, XE, sumxf, *tail, prepared=prep, e4m3=True, force="stream")
        Yx = ops.fused_dense_sparse_expanded_cuda(*base, XE, sumxf, *tail, prepared=prep, e4m3=True)
        Yt = fused(ops, Wd, q, force="tensor")
        assert torch.equal(Yx, Yt)


def test_prepared_container_forward(ops):
    from zip_kernel_b200 import v9_linear
    T, N, K = 384, 640, 1024
    W, X = make_case(T, N, K, 0.1, perm_seed=2)
    Wd = W.to(torch.device("cuda"))
    Y0 = v9_linear.v9_linear_forward(X.cuda(), Wd)
    v9_linear.prepare_for_prefill(Wd)
    assert Wd.prepared is not None and Wd.to(torch.device("cuda")).prepared is None
    assert torch.equal(v9_linear.v9_linear_forward(X.cuda(), Wd), Y0)


@pytest.mark.parametrize("T,N,K", [(64, 6144, 4096), (96, 6144, 4096), (128, 6144, 4096), (192, 4096, 4096),
                                   (128, 4096, 14336), (255, 384, 1024), (100, 28672, 512)])
def test_automatic_kernel_choice_between_64_and_255_tokens(ops, T, N, K):
    """Whichever kernel the library's cost model picks, with or without prepared weights, the result is that of
    one of the two kernels bit for bit (they agree with each other within the fp16 tolerance)."""
    W, X = make_case(T, N, K, 0.05, perm_seed=4)
    Wd = W.to(torch.device("cuda"))
    prep = prepare(ops, Wd)
    args = (X.cuda(), Wd.perm, Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
            Wd.scale_u4, Wd.zero_u4, N, K)
    Ys = ops.fused_dense_sparse_e2e_cuda(*args, force="stream")
    Yt = ops.fused_dense_sparse_e2e_cuda(*args, force="tensor")
    assert_kernels_agree(Yt, Ys, "tensor vs stream", W, ops.activation_quant_cuda(X.cuda(), Wd.perm), ("tensor-core", "streaming"))
    for pr in (None, prep):
        Ya = ops.fused_dense_sparse_e2e_cuda(*args, prepared=pr)
        assert torch.equal(Ya, Ys) or torch.equal(Ya, Yt)
        q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
        Yb = fused(ops, Wd, q, prepared=pr)
        assert torch.equal(Yb, Ys) or torch.equal(Yb, Yt)

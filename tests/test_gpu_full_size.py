"""Full-size shapes (Llama-2-70B linears, long prompts) checked through properties
that do not need the oracle to chew through the whole problem:

* a slice of output rows against the oracle (rows of a linear are independent, so
  a two-block-row sub-container is an exact sub-problem);
* the weight-streaming kernel against the tensor-core kernel (two independent MMA
  paths: mma.sync s8 vs tcgen05 kind::i8 with different tilings and fold order);
* exact homogeneity: doubling every weight scale doubles the fp16 output bit for
  bit (powers of two commute with every rounding on the path, fp16 subnormals aside);
* integer accumulators: the dump of the full-size run equals the integer matmul on
  the sliced rows.
"""

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import assert_close_fp16, container_np, make_case, np_, oracle_fused
from zip_kernel_b200.pack_utils import BROW, V9WeightContainer

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from zip_kernel_b200 import ops as _ops
    return _ops


def row_slice(W, br0, nbr):
    """The sub-container of block-rows [br0, br0 + nbr): an exact sub-problem."""
    r0, r1 = br0 * BROW, min((br0 + nbr) * BROW, W.d_out)
    off = W.hp_row_offsets[br0:br0 + nbr + 1].clone()
    b0, b1 = int(off[0]), int(off[-1])
    return V9WeightContainer(
        W_low_packed=W.W_low_packed[r0:r1].contiguous(), W_high_blocks_packed=W.W_high_blocks_packed[b0:b1].contiguous(),
        scale_u4=W.scale_u4[r0:r1].contiguous(), zero_u4=W.zero_u4[r0:r1].contiguous(),
        hp_row_offsets=(off - b0).to(torch.int32), hp_col_indices=W.hp_col_indices[b0:b1].contiguous(),
        perm=W.perm, block_shape=W.block_shape, d_out=r1 - r0, d_in=W.d_in), r0, r1


def fused(ops, Wd, q, **kw):
    return ops.fused_dense_sparse_cuda(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets, Wd.hp_col_indices,
                                       q[0], Wd.scale_u4, Wd.zero_u4, q[2], q[1], Wd.d_out, Wd.d_in, **kw)


# Llama-2-70B linears (the 8192 -> 57344 one as the 1/8 column shard a rank of 8 holds)
SHAPES_70B = [(8192, 10240), (8192, 8192), (8192, 7168), (28672, 8192)]


@pytest.mark.parametrize("K,N", SHAPES_70B)
@pytest.mark.parametrize("T", [1, 16])
def test_70b_decode_rows_vs_oracle(ops, K, N, T):
    W, X = make_case(T, N, K, 0.05, perm_seed=11)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Y = fused(ops, Wd, q)
    assert Y.shape == (N, T)
    xs4, sx, sumx = (np_(t) for t in q)
    # first, a middle and the last pair of block-rows
    nbr = (N + BROW - 1) // BROW
    for br0 in (0, nbr // 2, nbr - 2):
        Ws, r0, r1 = row_slice(W, br0, 2)
        ref = oracle_fused(container_np(Ws), xs4, sumx, sx)
        assert_close_fp16(np_(Y[r0:r1]), ref, f"{K}->{N} T={T} rows {r0}:{r1}")


@pytest.mark.parametrize("K,N", [(8192, 10240), (28672, 8192)])
def test_70b_stream_vs_tensor_kernel(ops, K, N):
    T = 40            # ragged against both kernels' token tiles
    W, X = make_case(T, N, K, 0.05, perm_seed=5)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Ys = fused(ops, Wd, q, force="stream")
    Yt = fused(ops, Wd, q, force="tensor")
    assert_close_fp16(np_(Yt), np_(Ys), f"tensor vs stream {K}->{N}")


@pytest.mark.parametrize("T,force", [(4, None), (2048, "tensor")])
def test_scale_homogeneity_is_exact(ops, T, force):
    K, N = 4096, 6144
    W, X = make_case(T, N, K, 0.05, perm_seed=3)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Y1 = fused(ops, Wd, q, force=force)
    W2 = Wd.to(torch.device("cuda"))
    W2.scale_u4 = (Wd.scale_u4.float() * 2).half()
    Y2 = fused(ops, W2, q, force=force)
    # fp16 subnormals (|y| < 6.1e-5) round on a fixed grid, so 2*round(y) != round(2*y) there
    normal = Y1.abs() >= 1.25e-4
    assert torch.equal(Y2[normal], (Y1.float() * 2).half()[normal])
    assert (Y2.float() - 2 * Y1.float()).abs().max().item() <= 1.3e-7


def test_prefill_2048_rows_vs_oracle_and_first_tokens_vs_stream(ops):
    T, K, N = 2048, 4096, 28672
    W, X = make_case(T, N, K, 0.05, perm_seed=9)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Y = fused(ops, Wd, q)                          # tensor-core kernel by shape
    xs4, sx, sumx = (np_(t) for t in q)
    Ws, r0, r1 = row_slice(W, 100, 1)
    # the oracle on one block-row and every 16th token
    sel = np.arange(0, T, 16)
    ref = oracle_fused(container_np(Ws), xs4[sel], sumx[sel], sx[sel])
    assert_close_fp16(np_(Y[r0:r1])[:, sel], ref, "prefill rows vs oracle")
    # the first 16 tokens through the streaming kernel
    q16 = tuple(t[:16].contiguous() for t in q)
    Y16 = fused(ops, Wd, q16, force="stream")
    assert_close_fp16(np_(Y[:, :16]), np_(Y16), "prefill vs stream, first tokens")


def test_full_size_accumulators_on_row_slice(ops):
    T, K, N = 16, 14336, 4096
    W, X = make_case(T, N, K, 0.05, perm_seed=2)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    acc, acc_hi = ops.dump_accumulators(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets,
                                        Wd.hp_col_indices, q[0], N, K)
    Ws, r0, r1 = row_slice(W, 7, 1)
    Wn = container_np(Ws)
    xs4 = np_(q[0])
    ref = O.group_accumulators(Wn["W_low_packed"], xs4)
    assert np.array_equal(np_(acc)[:, r0:r1, :], ref)
    b0 = int(W.hp_row_offsets[7])
    ref_hi = O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4)
    assert np.array_equal(np_(acc_hi)[b0:b0 + ref_hi.shape[0]], ref_hi)


@pytest.mark.parametrize("T", [17, 20, 32])
def test_32_token_pass_of_the_streaming_kernel(ops, T):
    """17..32 tokens on a long-K shape take one 32-token pass per CTA (four MMA tiles):
    outputs against the oracle, accumulators bit for bit."""
    K, N = 8192, 384
    W, X = make_case(T, N, K, 0.1, perm_seed=4)
    Wd = W.to(torch.device("cuda"))
    Wn = container_np(W)
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    xs4, sx, sumx = (np_(t) for t in q)
    Y = fused(ops, Wd, q, force="stream")
    assert_close_fp16(np_(Y), oracle_fused(Wn, xs4, sumx, sx), f"T={T} one 32-token pass")
    acc, acc_hi = ops.dump_accumulators(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets,
                                        Wd.hp_col_indices, q[0], N, K, force="stream")
    assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], xs4))
    assert np.array_equal(np_(acc_hi), O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4))
    # the split over a cluster and the 32-token pass together: a shape with few block-rows
    Ye = ops.fused_dense_sparse_e2e_cuda(X.cuda(), Wd.perm, Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets,
                                         Wd.hp_col_indices, Wd.scale_u4, Wd.zero_u4, N, K)
    assert torch.equal(Ye, Y)

"""The benchmark configurations at their full sizes, checked through exact sub-problems:

* prompt lengths 2048 and 8192 on Llama-3-8B linears, residual densities 0 %, 5 % and 15 %;
* the four Llama-2-70B linears at 4096 tokens, the 8192 -> 57344 one whole;
* the cluster split of a block-row at every size 1, 2, 4, 8 on one shape.

Rows of a linear are independent, so a block-row sub-container is an exact sub-problem for the
oracle (a subset of the tokens keeps it cheap); the first 16 tokens of a many-token run are also
compared with the weight-streaming kernel, an independent MMA path."""

import os

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import assert_close_fp16, assert_kernels_agree, container_np, make_case, np_, oracle_fused
from test_gpu_full_size import fused, row_slice
from zip_kernel_b200.pack_utils import BROW

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from zip_kernel_b200 import ops as _ops
    return _ops


def check_rows_and_first_tokens(ops, W, Wd, q, Y, block_rows, tok_step, what):
    """Y (N, T) of a many-token run: selected block-rows on every tok_step-th token against the
    oracle, the first 16 tokens of every row against the streaming kernel."""
    xs4, sx, sumx = (np_(t) for t in q)
    T = xs4.shape[0]
    sel = np.arange(0, T, tok_step)
    for br in block_rows:
        Ws, r0, r1 = row_slice(W, br, 1)
        ref = oracle_fused(container_np(Ws), xs4[sel], sumx[sel], sx[sel])
        assert_close_fp16(np_(Y[r0:r1])[:, sel], ref, f"{what}: block-row {br} vs oracle")
    q16 = tuple(t[:16].contiguous() for t in q)
    Y16 = fused(ops, Wd, q16, force="stream")
    assert_kernels_agree(Y[:, :16], Y16, f"{what}: first tokens vs streaming kernel", W, q16, ("tensor-core", "streaming"))


@pytest.mark.parametrize("name,K,N", [("gate_up", 4096, 28672), ("down", 14336, 4096)])
def test_prefill_8192_tokens(ops, name, K, N):
    T = 8192
    W, X = make_case(T, N, K, 0.05, perm_seed=12)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Y = fused(ops, Wd, q)
    assert Y.shape == (N, T)
    nbr = N // BROW
    check_rows_and_first_tokens(ops, W, Wd, q, Y, (0, nbr // 2 + 1, nbr - 1), 64, f"{name} M=8192")
    # the last token tile and a token in the middle, one block-row, against the oracle
    xs4, sx, sumx = (np_(t) for t in q)
    sel = np.array([4095, 4096, 8064, 8191])
    Ws, r0, r1 = row_slice(W, 3, 1)
    assert_close_fp16(np_(Y[r0:r1])[:, sel], oracle_fused(container_np(Ws), xs4[sel], sumx[sel], sx[sel]),
                      f"{name} M=8192 tile edges")


@pytest.mark.parametrize("density", [0.0, 0.15])
@pytest.mark.parametrize("prepared", [False, True])
def test_prefill_2048_density_sweep(ops, density, prepared):
    T, K, N = 2048, 4096, 6144
    W, X = make_case(T, N, K, density, perm_seed=13)
    Wd = W.to(torch.device("cuda"))
    assert (W.n_hp_blocks == 0) == (density == 0.0)
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    prep = (ops.prepare_weights_cuda(Wd.W_low_packed), ops.prepare_weights_cuda(Wd.W_high_blocks_packed)) if prepared else None
    Y = fused(ops, Wd, q, prepared=prep)
    check_rows_and_first_tokens(ops, W, Wd, q, Y, (0, 17, 47), 32, f"qkv M=2048 density {density} prepared={prepared}")
    if prepared:
        assert torch.equal(Y, fused(ops, Wd, q))       # the two instantiations agree bit for bit
    # integer accumulators of one token tile of this run against the integer matmul
    sub = tuple(t[1024:1152].contiguous() for t in q)
    acc, acc_hi = ops.dump_accumulators(Wd.W_low_packed[:256], Wd.W_high_blocks_packed[:int(W.hp_row_offsets[2])],
                                        Wd.hp_row_offsets[:3], Wd.hp_col_indices[:int(W.hp_row_offsets[2])], sub[0],
                                        256, K, force="tensor")
    Wn = container_np(row_slice(W, 0, 2)[0])
    assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], np_(sub[0])))
    if density > 0:
        assert np.array_equal(np_(acc_hi), O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], np_(sub[0])))


SHAPES_70B_FULL = [("qkv", 8192, 10240), ("o", 8192, 8192), ("gate_up", 8192, 57344), ("down", 28672, 8192)]


@pytest.mark.parametrize("name,K,N", SHAPES_70B_FULL)
def test_70b_4096_tokens(ops, name, K, N):
    T = 4096
    W, X = make_case(T, N, K, 0.05, perm_seed=14)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Y = fused(ops, Wd, q)
    nbr = N // BROW
    check_rows_and_first_tokens(ops, W, Wd, q, Y, (0, nbr // 3, nbr - 1), 128, f"70B {name} M=4096")
    from zip_kernel_b200 import _lib
    assert _lib.device_error(torch.device("cuda")) == 0


def test_70b_whole_gate_up_one_token(ops):
    """The 8192 -> 57344 linear whole (the 1-GPU point of the sharded configuration) at one token."""
    K, N = 8192, 57344
    W, X = make_case(1, N, K, 0.05, perm_seed=15)
    Wd = W.to(torch.device("cuda"))
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    Y = fused(ops, Wd, q)
    xs4, sx, sumx = (np_(t) for t in q)
    nbr = N // BROW
    for br0 in (0, 100, 223, 224, nbr - 2):
        Ws, r0, r1 = row_slice(W, br0, 2)
        assert_close_fp16(np_(Y[r0:r1]), oracle_fused(container_np(Ws), xs4, sumx, sx), f"70B gate_up rows {r0}:{r1}")


@pytest.mark.parametrize("T", [1, 16])
def test_cluster_split_sizes_agree(ops, T):
    """One shape with residual blocks at cluster sizes 1, 2, 4, 8 of a block-row: integer accumulators
    identical, outputs within the tolerance of the oracle (the fp32 partial sums of a split differ
    from the unsplit order in rounding only).  The reference pins the same trap for its split-K
    path (cuda_kernel/tests/test_splitk_parity.py:36-46)."""
    K, N = 4096, 512
    W, X = make_case(T, N, K, 0.3, perm_seed=16, force_block_per_row=True)
    Wd = W.to(torch.device("cuda"))
    Wn = container_np(W)
    q = ops.activation_quant_cuda(X.cuda(), Wd.perm)
    xs4, sx, sumx = (np_(t) for t in q)
    ref = oracle_fused(Wn, xs4, sumx, sx)
    ref_acc = O.group_accumulators(Wn["W_low_packed"], xs4)
    ref_hi = O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4)
    outs = {}
    old = os.environ.get("W4A4_DECODE_SPLIT")
    try:
        for split in (1, 2, 4, 8):
            os.environ["W4A4_DECODE_SPLIT"] = str(split)
            Y = fused(ops, Wd, q, force="stream")
            assert_close_fp16(np_(Y), ref, f"split {split}")
            acc, acc_hi = ops.dump_accumulators(Wd.W_low_packed, Wd.W_high_blocks_packed, Wd.hp_row_offsets,
                                                Wd.hp_col_indices, q[0], N, K, force="stream")
            assert np.array_equal(np_(acc), ref_acc) and np.array_equal(np_(acc_hi), ref_hi), f"split {split}"
            outs[split] = Y
            assert torch.equal(fused(ops, Wd, q, force="stream"), Y), "a split must be deterministic"
    finally:
        if old is None:
            os.environ.pop("W4A4_DECODE_SPLIT", None)
        else:
            os.environ["W4A4_DECODE_SPLIT"] = old
    worst = max((outs[a].float() - outs[b].float()).abs().max().item() for a in outs for b in outs)
    assert worst <= 2e-2

"""RMSNorm -> quantisation and SiLU * mul -> quantisation as single launches: codes, scales and group sums
bit-exact against the oracle's composition (fp16 RMSNorm / gated activation, then
``quantize_activation_s4``), in the packed and in the expanded output form, and the module-level
forwards built on them equal to the unfused sequence bit for bit."""

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import assert_close_fp16, container_np, make_case, np_, oracle_fused
from zip_kernel_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from zip_kernel_b200 import ops as _ops
    return _ops


def perm_of(K, seed):
    return synth.make_perm(K, seed)


CASES = [(1, 4096, None), (4, 4096, 3), (16, 512, None), (33, 1024, 5), (300, 256, None), (700, 384, 7), (2, 14336, None)]


@pytest.mark.parametrize("T,K,perm_seed", CASES)
def test_rmsnorm_quant_bit_exact(ops, T, K, perm_seed):
    g = torch.Generator().manual_seed(T * 31 + K)
    X = synth.make_activations(T, K, seed=T + K)
    X[0, : K // 2] = 0                                   # a row with many exact zeros
    if T > 2:
        X[2] = 0                                         # an all-zero row: scale 0, codes 0
    w = (torch.randn(K, generator=g) * 0.5 + 1.0).half()
    eps = 1e-5
    perm = perm_of(K, perm_seed)
    y = O.rmsnorm_fp16(X.numpy(), w.numpy(), eps)
    r4, rs, rsum = O.quantize_activation_s4(y, perm.numpy())
    pd = None if perm_seed is None else perm.cuda()
    q4, qs, qsum = ops.rmsnorm_quant_cuda(X.cuda(), w.cuda(), eps, pd)
    assert np.array_equal(np_(q4), r4)
    assert np.array_equal(np_(qs).view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(np_(qsum), rsum)
    # the expanded form equals the expansion of the packed form
    XE, sumxf, sx = ops.rmsnorm_quant_cuda(X.cuda(), w.cuda(), eps, pd, expanded=True)
    XE_ref, sumxf_ref = ops.expand_activations_cuda(q4, qsum)
    assert _live_lines_equal(XE, XE_ref, T, K)
    assert torch.equal(sumxf, sumxf_ref) and torch.equal(sx, qs)
    # identical to the unfused sequence on the torch composition of the same definition
    yt = torch.from_numpy(y).cuda()
    u4, us, usum = ops.activation_quant_cuda(yt, perm.cuda())
    assert torch.equal(u4, q4) and torch.equal(us, qs) and torch.equal(usum, qsum)


def _live_lines_equal(XE, XE_ref, T, K):
    """Compare only the lines of live tokens (rows of the padding up to 16 tokens are never written)."""
    t_pad = (T + 15) // 16 * 16
    a = XE[: (K // 128) * t_pad * 128].view(K // 128, t_pad, 128)[:, :T]
    b = XE_ref[: (K // 128) * t_pad * 128].view(K // 128, t_pad, 128)[:, :T]
    return bool(torch.equal(a, b))


@pytest.mark.parametrize("T,K,perm_seed", CASES)
def test_silu_mul_quant_bit_exact(ops, T, K, perm_seed):
    GU = synth.make_activations(T, 2 * K, seed=T * 3 + K, outlier_frac=0.0, std=2.0)
    GU[0, :8] = torch.tensor([0.0, -0.0, 65504.0, -65504.0, 1e-4, -1e-4, 20.0, -20.0]).half()
    GU[0, K:K + 8] = 0.25                                  # keeps the products of the extreme gates finite
    perm = perm_of(K, perm_seed)
    y = O.silu_mul_fp16(GU[:, :K].numpy(), GU[:, K:].numpy())
    r4, rs, rsum = O.quantize_activation_s4(y, perm.numpy())
    pd = None if perm_seed is None else perm.cuda()
    q4, qs, qsum = ops.silu_mul_quant_cuda(GU.cuda(), pd)
    assert np.array_equal(np_(qs).view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(np_(q4), r4)
    assert np.array_equal(np_(qsum), rsum)
    XE, sumxf, sx = ops.silu_mul_quant_cuda(GU.cuda(), pd, expanded=True)
    XE_ref, sumxf_ref = ops.expand_activations_cuda(q4, qsum)
    assert _live_lines_equal(XE, XE_ref, T, K) and torch.equal(sumxf, sumxf_ref) and torch.equal(sx, qs)


def test_fused_prologue_rows_strided_and_misaligned(ops):
    """Row-strided views go to the kernel as they are; a base 2 bytes off takes the scalar path."""
    T, K = 5, 512
    big = synth.make_activations(T, 2 * K + 24, seed=9)
    w = torch.ones(K).half()
    Xv = big.cuda()[:, 8:8 + K]                           # stride 2K+24, 16-byte aligned start
    q = ops.rmsnorm_quant_cuda(Xv, w.cuda(), 1e-6, None)
    r = O.quantize_activation_s4(O.rmsnorm_fp16(big[:, 8:8 + K].numpy(), w.numpy(), 1e-6), np.arange(K, dtype=np.int32))
    assert np.array_equal(np_(q[0]), r[0]) and np.array_equal(np_(q[2]), r[2])
    Xo = big.cuda()[:, 1:1 + K]                           # 2 bytes off
    q = ops.rmsnorm_quant_cuda(Xo, w.cuda(), 1e-6, None)
    r = O.quantize_activation_s4(O.rmsnorm_fp16(big[:, 1:1 + K].numpy(), w.numpy(), 1e-6), np.arange(K, dtype=np.int32))
    assert np.array_equal(np_(q[0]), r[0]) and np.array_equal(np_(q[2]), r[2])
    GUo = big.cuda()[:, 3:3 + 2 * K]
    q = ops.silu_mul_quant_cuda(GUo, None)
    h = big[:, 3:3 + 2 * K]
    r = O.quantize_activation_s4(O.silu_mul_fp16(h[:, :K].numpy(), h[:, K:].numpy()), np.arange(K, dtype=np.int32))
    assert np.array_equal(np_(q[0]), r[0]) and np.array_equal(np_(q[2]), r[2])
    with pytest.raises(ValueError):
        ops.silu_mul_quant_cuda(big.cuda()[:, : K + 128], None)


@pytest.mark.parametrize("T", [1, 32, 300])
def test_module_forwards_equal_the_unfused_sequence(ops, T):
    from zip_kernel_b200 import v9_linear
    dev = torch.device("cuda")
    K, N = 1024, 640
    W, X = make_case(T, N, K, 0.2, perm_seed=None if T != 32 else 4)
    Wd = W.to(dev)
    if T >= 256:
        v9_linear.prepare_for_prefill(Wd)
    w = (torch.rand(K) + 0.5).half()
    eps = 1e-5
    Xd = X.to(dev)
    y_norm = torch.from_numpy(O.rmsnorm_fp16(X.numpy(), w.numpy(), eps)).to(dev)
    assert torch.equal(v9_linear.v9_linear_forward_rmsnorm(Xd.reshape(1, T, K), w.to(dev), eps, Wd),
                       v9_linear.v9_linear_forward(y_norm, Wd).reshape(1, T, N))
    GU = synth.make_activations(T, 2 * K, seed=T + 5, outlier_frac=0.0, std=1.5)
    h = torch.from_numpy(O.silu_mul_fp16(GU[:, :K].numpy(), GU[:, K:].numpy())).to(dev)
    Yf = v9_linear.v9_linear_forward_silu_mul(GU.to(dev), Wd)
    assert torch.equal(Yf, v9_linear.v9_linear_forward(h, Wd))
    # and against the oracle end to end
    r4, rs, rsum = O.quantize_activation_s4(h.cpu().numpy(), W.perm.numpy())
    assert_close_fp16(np_(Yf).T, oracle_fused(container_np(W), r4, rsum, rs), "silu*mul -> linear vs oracle")

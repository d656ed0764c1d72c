"""The W4A16 route for long prompts without residual blocks (the reference's dispatcher takes it automatically,
backend/dispatcher.py:228-238; here it is a policy that is off by default): dequantisation bit-exact against the
oracle's restatement of the reference's formula; the route within 2e-2 of the output range (the bound of
triton_kernel/tests/test_w4a16_fallback.py:44-81) of what it computes by definition - the fp16 GEMM of the
UNQUANTISED permuted activations with the dequantised weight, dispatcher.py:236-238 - and the W4A4 kernels
within the same bound of the fake-quant forward; and the eligibility rule."""

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from helpers import make_case, np_

pytestmark = pytest.mark.gpu


def test_dequantised_weights_bit_exact():
    from zip_kernel_b200 import ops
    W, _ = make_case(1, 300, 512, 0.0)
    Wd = W.to(torch.device("cuda"))
    got = ops.dequant_u4_to_fp16_cuda(Wd.W_low_packed, Wd.scale_u4, Wd.zero_u4)
    ref = O.dequant_u4_to_fp16(np_(W.W_low_packed), np_(W.scale_u4), np_(W.zero_u4))
    assert got.shape == (300, 512)
    assert np.array_equal(np_(got).view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("T,K,N", [(512, 1024, 1024), (1024, 1024, 2752), (2048, 4096, 4096)])
def test_w4a16_route_matches_fakequant_and_rule(T, K, N):
    from zip_kernel_b200 import v9_linear
    dev = torch.device("cuda")
    W, _ = make_case(T, N, K, 0.0, perm_seed=5)
    Wd = W.to(dev)
    X = torch.randn(T, K, generator=torch.Generator().manual_seed(0)).half().to(dev)
    assert v9_linear.w4a16_eligible(Wd, T)
    Y_w4a4 = v9_linear.v9_linear_forward(X, Wd)                   # policy off: the W4A4 kernels
    prev = v9_linear.set_w4a16_fallback("auto")
    try:
        Y = v9_linear.v9_linear_forward(X, Wd)
        assert getattr(Wd, "_fp16_cache", None) is not None       # the route ran and cached its weight
    finally:
        v9_linear.set_w4a16_fallback(prev)
    # the route leaves the activations as they are: its reference is the plain forward on the dequantised weight
    W_fp = v9_linear.reconstruct_w_fakequant_fp16(Wd).float()
    ref16 = X[:, Wd.perm.to(torch.long)].float() @ W_fp.t()
    rng16 = ref16.abs().max().clamp(min=1e-6)
    assert ((Y.float() - ref16).abs().max() / rng16).item() <= 2e-2
    # the W4A4 kernels quantise them to 4 bits: their reference is the fake-quant forward
    ref = v9_linear.v9_linear_fakequant(X, Wd).float()
    rng = ref.abs().max().clamp(min=1e-6)
    assert ((Y_w4a4.float() - ref).abs().max() / rng).item() <= 2e-2
    assert not torch.equal(Y, Y_w4a4)                             # two different arithmetics


def test_w4a16_rule_excludes_residual_blocks_and_short_prompts():
    from zip_kernel_b200 import v9_linear
    W, _ = make_case(8, 256, 256, 0.5)
    assert not v9_linear.w4a16_eligible(W, 4096)                  # residual blocks: always W4A4
    W0, _ = make_case(8, 256, 256, 0.0)
    assert not v9_linear.w4a16_eligible(W0, 511) and v9_linear.w4a16_eligible(W0, 512) and v9_linear.w4a16_eligible(W0, 1024)
    with pytest.raises(ValueError):
        v9_linear.set_w4a16_fallback("always")

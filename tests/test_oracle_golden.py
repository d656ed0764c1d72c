"""The oracle against the golden vectors produced by the reference's own CPU
functions (tests/golden/make_golden.py).  Bit-exact for codes, scales, sums and
packed weights; the fp16 'loose truth' outputs must agree exactly as well since
the oracle restates the same dequantise -> fp32 matmul -> fp16 recipe (BLAS
summation order may differ, so one fp16 ulp of slack is allowed there)."""

import numpy as np
import pytest

from oracle import w4a4_oracle as O


def test_nibble_pack_golden(golden_nibble):
    g = golden_nibble
    assert np.array_equal(O.pack_s4_le(g["s4"]), g["s4_packed"])
    assert np.array_equal(O.pack_s4_le(g["u4"]), g["u4_packed"])
    assert np.array_equal(O.unpack_s4_le(g["s4_packed"], signed=True), g["s4_unpacked"])
    assert np.array_equal(O.unpack_s4_le(g["u4_packed"], signed=False), g["u4_unpacked"])
    assert np.array_equal(g["s4_unpacked"], g["s4"])
    assert np.array_equal(g["u4_unpacked"], g["u4"])


def test_quant_golden_bit_exact(golden_quant):
    g = golden_quant
    for name in g["names"]:
        xs4, sx, sumx = O.quantize_activation_s4(g[f"{name}/X"], g[f"{name}/perm"])
        assert np.array_equal(xs4, g[f"{name}/X_s4"]), name
        assert np.array_equal(sx.view(np.uint16), g[f"{name}/scale_x"].view(np.uint16)), name
        assert np.array_equal(sumx, g[f"{name}/sum_X"]), name


def _ulp_close(a, b, ulps=1):
    a = a.astype(np.float32)
    b = b.astype(np.float32)
    tol = ulps * np.maximum(np.spacing(np.abs(b).astype(np.float16)).astype(np.float32), 1e-7)
    return bool(np.all(np.abs(a - b) <= tol))


def test_fused_loose_truth_golden(golden_fused):
    g = golden_fused
    for name in g["names"]:
        T, N, K = (int(v) for v in g[f"{name}/dims"])
        args = dict(W_low_packed=g[f"{name}/W_low_packed"], X_s4=g[f"{name}/X_s4"],
                    scale_u4=g[f"{name}/scale_u4"], zero_u4=g[f"{name}/zero_u4"],
                    scale_x=g[f"{name}/scale_x"], d_out=N, d_in=K)
        assert _ulp_close(O.fp16_dense_reference(**args), g[f"{name}/Y_low"]), name
        if f"{name}/Y_fused" in g:
            yf = O.fp16_fused_reference(
                g[f"{name}/W_low_packed"], g[f"{name}/W_high_blocks_packed"],
                g[f"{name}/hp_row_offsets"], g[f"{name}/hp_col_indices"], g[f"{name}/X_s4"],
                g[f"{name}/scale_u4"], g[f"{name}/zero_u4"], g[f"{name}/scale_x"], N, K)
            # Y_low and 16*Y_high each carry one fp16 rounding
            assert _ulp_close(yf, g[f"{name}/Y_fused"], ulps=18), name
            yh = O.fp16_sparse_reference(
                g[f"{name}/W_high_blocks_packed"], g[f"{name}/hp_row_offsets"],
                g[f"{name}/hp_col_indices"], g[f"{name}/X_s4"], g[f"{name}/scale_u4"],
                g[f"{name}/scale_x"], N, K)
            assert _ulp_close(yh, g[f"{name}/Y_high"]), name


def test_quant_inside_fused_golden(golden_fused):
    g = golden_fused
    for name in g["names"]:
        xs4, sx, sumx = O.quantize_activation_s4(g[f"{name}/X"], g[f"{name}/perm"])
        assert np.array_equal(xs4, g[f"{name}/X_s4"]), name
        assert np.array_equal(sx.view(np.uint16), g[f"{name}/scale_x"].view(np.uint16)), name
        assert np.array_equal(sumx, g[f"{name}/sum_X"]), name


def test_kernel_order_vs_loose_truth(golden_fused):
    """The fp32 kernel-order restatement against the reference's dequantised
    fp16 truth under the reference's own bound: max|diff| / max|ref| < 5e-3
    (tools/parity/tests/test_fp16_reference_cpu.py:287-344)."""
    g = golden_fused
    for name in g["names"]:
        if f"{name}/Y_fused" not in g:
            continue
        T, N, K = (int(v) for v in g[f"{name}/dims"])
        y = O.fused_kernel_order(
            g[f"{name}/W_low_packed"], g[f"{name}/W_high_blocks_packed"],
            g[f"{name}/hp_row_offsets"], g[f"{name}/hp_col_indices"], g[f"{name}/X_s4"],
            g[f"{name}/scale_u4"], g[f"{name}/zero_u4"], g[f"{name}/sum_X"],
            g[f"{name}/scale_x"], N, K)
        ref = g[f"{name}/Y_fused"].astype(np.float32)
        rel = np.abs(y.astype(np.float32) - ref).max() / max(np.abs(ref).max(), 1e-4)
        assert rel < 5e-3, (name, rel)
        # fp32 and fp64 folds agree to within fp16 rounding of the result
        y64 = O.fused_kernel_order(
            g[f"{name}/W_low_packed"], g[f"{name}/W_high_blocks_packed"],
            g[f"{name}/hp_row_offsets"], g[f"{name}/hp_col_indices"], g[f"{name}/X_s4"],
            g[f"{name}/scale_u4"], g[f"{name}/zero_u4"], g[f"{name}/sum_X"],
            g[f"{name}/scale_x"], N, K, dtype=np.float64)
        assert _ulp_close(y, y64, ulps=1), name


def test_fused_is_dense_plus_16_sparse(golden_fused):
    """Structure check of tools/parity/tests/test_fp16_reference_cpu.py:234-285."""
    g = golden_fused
    name = "t32_n256_k256_d25"
    T, N, K = (int(v) for v in g[f"{name}/dims"])
    common = (g[f"{name}/W_low_packed"], g[f"{name}/W_high_blocks_packed"],
              g[f"{name}/hp_row_offsets"], g[f"{name}/hp_col_indices"], g[f"{name}/X_s4"],
              g[f"{name}/scale_u4"], g[f"{name}/zero_u4"], g[f"{name}/sum_X"],
              g[f"{name}/scale_x"], N, K)
    full = O.fused_kernel_order(*common, dtype=np.float64).astype(np.float64)
    d = O.fused_kernel_order(*common, dtype=np.float64, sparse=False).astype(np.float64)
    s = O.fused_kernel_order(*common, dtype=np.float64, dense=False, sparse_weight=1.0).astype(np.float64)
    assert np.abs(full - (d + 16 * s)).max() <= 2e-2 * max(1.0, np.abs(full).max()) * 1e-1


def test_accumulator_bounds_and_sum_identity(golden_fused):
    g = golden_fused
    name = "t64_n256_k512_d10"
    acc = O.group_accumulators(g[f"{name}/W_low_packed"], g[f"{name}/X_s4"])
    assert acc.dtype == np.int32 and np.abs(acc).max() <= 128 * 64
    # sum_X identity: a weight row of ones reproduces the per-group code sums
    ones = O.pack_s4_le(np.ones((1, 512), dtype=np.int8))
    acc1 = O.group_accumulators(ones, g[f"{name}/X_s4"])      # (ng, 1, T)
    assert np.array_equal(acc1[:, 0, :].T, g[f"{name}/sum_X"])


def test_pack_v9_weights_golden(golden_pack):
    g = golden_pack
    for name in g["names"]:
        raw = {k.split("/in/")[1]: v for k, v in g.items() if k.startswith(f"{name}/in/")}
        W = O.pack_v9_weights(raw["Q_u4_permuted"], raw["scale_u4_raw"], raw["zero_u4_raw"],
                              raw["Q_s8_blocks"], raw["scale_s8_per_block"],
                              raw["hp_block_indices"], raw["perm"])
        for k in ("W_low_packed", "W_high_blocks_packed", "hp_row_offsets", "hp_col_indices", "perm"):
            assert np.array_equal(W[k], g[f"{name}/out/{k}"]), (name, k)
        for k in ("scale_u4", "zero_u4"):
            assert np.array_equal(W[k].view(np.uint16), g[f"{name}/out/{k}"].view(np.uint16)), (name, k)

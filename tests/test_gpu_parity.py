"""GPU parity tests: the CUDA path (through the C ABI) against the CPU oracle on
identical seeded inputs, and against the golden vectors of the reference.

Bit-exact: activation codes, scales, group sums and int32 accumulators.
fp16 outputs: max-abs 1e-2 + rel 1e-3 against the fp32 kernel-order oracle, and
max|diff|/max|ref| < 5e-3 against the reference's dequantised fp16 truth (its own
bound, tools/parity/tests/test_fp16_reference_cpu.py:287-344).
"""

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from tests.helpers import (assert_close_fp16, container_np, cuda_container, make_case, np_,
                           oracle_fused)

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


def _quant_check(ops, X, perm):
    xs4, sx, sumx = ops.activation_quant_cuda(X.cuda(), perm.cuda())
    r4, rs, rsum = O.quantize_activation_s4(np_(X), np_(perm))
    assert np.array_equal(np_(xs4), r4)
    assert np.array_equal(np_(sx).view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(np_(sumx), rsum)


# --------------------------------------------------------------------------- quant
def test_quant_golden(ops, golden_quant):
    g = golden_quant
    for name in g["names"]:
        X = torch.from_numpy(g[f"{name}/X"]).cuda()
        perm = torch.from_numpy(g[f"{name}/perm"]).cuda()
        xs4, sx, sumx = ops.activation_quant_cuda(X, perm)
        assert np.array_equal(np_(xs4), g[f"{name}/X_s4"]), name
        assert np.array_equal(np_(sx).view(np.uint16), g[f"{name}/scale_x"].view(np.uint16)), name
        assert np.array_equal(np_(sumx), g[f"{name}/sum_X"]), name


@pytest.mark.parametrize("T,K,perm_seed", [
    (1, 4096, None), (16, 4096, 7), (4, 14336, None), (16, 14336, 3), (1, 28672, 5),
    (1, 8192, None), (129, 256, 1), (2048, 4096, None), (77, 6144, 9),
])
def test_quant_vs_oracle(ops, T, K, perm_seed):
    from zip_kernel_b200 import synth
    X = synth.make_activations(T, K, seed=T * 131 + K)
    _quant_check(ops, X, synth.make_perm(K, perm_seed))


def test_quant_3d_and_int64_perm(ops):
    from zip_kernel_b200 import synth
    X = synth.make_activations(12, 512, seed=3).reshape(3, 4, 512)
    perm = synth.make_perm(512, 4).to(torch.int64)
    xs4, sx, sumx = ops.activation_quant_cuda(X.cuda(), perm.cuda())
    r4, rs, rsum = O.quantize_activation_s4(np_(X), np_(perm))
    assert xs4.shape == (12, 256) and sx.shape == (12,) and sumx.shape == (12, 4)
    assert np.array_equal(np_(xs4), r4) and np.array_equal(np_(sumx), rsum)


def test_quant_noncontiguous_rows(ops):
    """Row stride larger than K (a column slice of a wider tensor)."""
    from zip_kernel_b200 import synth
    big = synth.make_activations(5, 1024, seed=8).cuda()
    X = big[:, 128:640]                      # (5, 512), stride 1024, not 16-byte row-aligned issue free
    perm = synth.make_perm(512, None)
    xs4, sx, sumx = ops.activation_quant_cuda(X, perm.cuda())
    r4, rs, rsum = O.quantize_activation_s4(np_(X), np_(perm))
    assert np.array_equal(np_(xs4), r4) and np.array_equal(np_(sumx), rsum)


def test_quant_argument_errors(ops):
    X = torch.zeros(2, 100, dtype=torch.float16, device="cuda")
    with pytest.raises(ValueError):
        ops.activation_quant_cuda(X, torch.arange(100, dtype=torch.int32, device="cuda"))
    with pytest.raises(AssertionError):
        ops.activation_quant_cuda(X.float(), torch.arange(100, dtype=torch.int32, device="cuda"))
    with pytest.raises(ValueError):
        ops.activation_quant_cuda(torch.zeros(128, dtype=torch.float16, device="cuda"),
                                  torch.arange(128, dtype=torch.int32, device="cuda"))


# --------------------------------------------------------------------------- GEMMs
def _run_fused(ops, Wc, xs4, sumx, sx, **kw):
    return ops.fused_dense_sparse_cuda(Wc.W_low_packed, Wc.W_high_blocks_packed, Wc.hp_row_offsets,
                                       Wc.hp_col_indices, xs4, Wc.scale_u4, Wc.zero_u4, sumx, sx,
                                       Wc.d_out, Wc.d_in, **kw)


def test_fused_golden(ops, golden_fused):
    g = golden_fused
    for name in g["names"]:
        T, N, K = (int(v) for v in g[f"{name}/dims"])
        t = lambda k: torch.from_numpy(g[f"{name}/{k}"]).cuda()
        Y = ops.fused_dense_sparse_cuda(t("W_low_packed"), t("W_high_blocks_packed"), t("hp_row_offsets"),
                                        t("hp_col_indices"), t("X_s4"), t("scale_u4"), t("zero_u4"),
                                        t("sum_X"), t("scale_x"), N, K)
        assert Y.shape == (N, T) and Y.dtype == torch.float16
        ref = O.fused_kernel_order(g[f"{name}/W_low_packed"], g[f"{name}/W_high_blocks_packed"],
                                   g[f"{name}/hp_row_offsets"], g[f"{name}/hp_col_indices"],
                                   g[f"{name}/X_s4"], g[f"{name}/scale_u4"], g[f"{name}/zero_u4"],
                                   g[f"{name}/sum_X"], g[f"{name}/scale_x"], N, K)
        assert_close_fp16(np_(Y), ref, name)
        if f"{name}/Y_fused" in g:
            loose = g[f"{name}/Y_fused"].astype(np.float32)
            rel = np.abs(np_(Y).astype(np.float32) - loose).max() / max(np.abs(loose).max(), 1e-4)
            assert rel < 5e-3, (name, rel)


CASES = [
    # T, N, K, density, perm_seed
    (1, 128, 128, 0.0, None), (1, 256, 384, 0.5, None), (2, 128, 256, 1.0, 2), (7, 256, 256, 0.3, None),
    (8, 384, 512, 0.2, 3), (9, 128, 384, 0.4, None), (16, 256, 128, 0.5, None), (17, 256, 256, 0.3, 1),
    (33, 128, 256, 0.2, None), (129, 128, 128, 0.5, None), (5, 200, 384, 0.3, 5), (16, 1000, 512, 0.1, None),
    (4, 1024, 2048, 0.05, None), (16, 512, 6144, 0.05, None), (1, 256, 17408, 0.05, None),
]


@pytest.mark.parametrize("T,N,K,density,perm_seed", CASES)
def test_e2e_and_ops_vs_oracle(ops, T, N, K, density, perm_seed):
    W, X = make_case(T, N, K, density, perm_seed)
    Wn, Wc = container_np(W), cuda_container(W)
    xs4, sx, sumx = O.quantize_activation_s4(np_(X), Wn["perm"])
    ref = oracle_fused(Wn, xs4, sumx, sx)
    # two-step: quant op then fused op
    q4, qs, qsum = ops.activation_quant_cuda(X.cuda(), Wc.perm)
    assert np.array_equal(np_(q4), xs4) and np.array_equal(np_(qsum), sumx)
    Y = _run_fused(ops, Wc, q4, qsum, qs)
    assert_close_fp16(np_(Y), ref, "fused")
    # one call, fp16 in
    Y2 = ops.fused_dense_sparse_e2e_cuda(X.cuda(), Wc.perm, Wc.W_low_packed, Wc.W_high_blocks_packed,
                                         Wc.hp_row_offsets, Wc.hp_col_indices, Wc.scale_u4, Wc.zero_u4,
                                         N, K)
    assert torch.equal(Y, Y2), "e2e call must equal quant + fused"
    # token-major output
    Y3 = _run_fused(ops, Wc, q4, qsum, qs, token_major=True)
    assert Y3.shape == (T, N) and torch.equal(Y3.t().contiguous(), Y)
    # dense-only and sparse-only partial products
    Yd = ops.dense_gemm_cuda(Wc.W_low_packed, q4, Wc.scale_u4, Wc.zero_u4, qsum, qs)
    assert_close_fp16(np_(Yd), oracle_fused(Wn, xs4, sumx, sx, sparse=False), "dense")
    Ys = ops.sparse_gemm_cuda(Wc.W_high_blocks_packed, Wc.hp_row_offsets, Wc.hp_col_indices, q4,
                              Wc.scale_u4, qs, N, K)
    assert_close_fp16(np_(Ys), oracle_fused(Wn, xs4, sumx, sx, dense=False, sparse_weight=1.0), "sparse")


@pytest.mark.parametrize("T,N,K,density", [(1, 256, 512, 0.3), (16, 384, 1024, 0.2), (13, 200, 256, 0.5),
                                           (40, 128, 384, 1.0)])
def test_accumulators_bit_exact(ops, T, N, K, density):
    W, X = make_case(T, N, K, density)
    Wn, Wc = container_np(W), cuda_container(W)
    xs4, _, _ = O.quantize_activation_s4(np_(X), Wn["perm"])
    acc, acc_hi = ops.dump_accumulators(Wc.W_low_packed, Wc.W_high_blocks_packed, Wc.hp_row_offsets,
                                        Wc.hp_col_indices, torch.from_numpy(xs4).cuda(), N, K)
    assert np.array_equal(np_(acc), O.group_accumulators(Wn["W_low_packed"], xs4))
    ref_hi = O.block_accumulators(Wn["W_high_blocks_packed"], Wn["hp_col_indices"], xs4)
    if N % 128:
        # rows past d_out inside the last block-row are padding
        last = np.repeat(np.diff(Wn["hp_row_offsets"]), 1)
        br = np.repeat(np.arange(len(last)), last)
        pad = (br[:, None] * 128 + np.arange(128)[None, :]) >= N
        got = np_(acc_hi).copy()
        got[pad] = 0
        ref_hi = ref_hi.copy()
        ref_hi[pad] = 0
        assert np.array_equal(got, ref_hi)
    else:
        assert np.array_equal(np_(acc_hi), ref_hi)


@pytest.mark.parametrize("M", [1, 4, 16])
@pytest.mark.parametrize("K,N", [(4096, 4096), (4096, 6144), (14336, 4096)])
def test_decode_shapes_llama8b(ops, M, K, N):
    """Decode shapes of the benchmark at full size (gate_up is covered by the
    row-sampled test below)."""
    W, X = make_case(M, N, K, 0.05)
    Wn, Wc = container_np(W), cuda_container(W)
    xs4, sx, sumx = O.quantize_activation_s4(np_(X), Wn["perm"])
    Y = ops.fused_dense_sparse_e2e_cuda(X.cuda(), Wc.perm, Wc.W_low_packed, Wc.W_high_blocks_packed,
                                        Wc.hp_row_offsets, Wc.hp_col_indices, Wc.scale_u4, Wc.zero_u4, N, K)
    assert_close_fp16(np_(Y), oracle_fused(Wn, xs4, sumx, sx), f"M{M} {K}->{N}")
    loose = O.fp16_fused_reference(Wn["W_low_packed"], Wn["W_high_blocks_packed"], Wn["hp_row_offsets"],
                                   Wn["hp_col_indices"], xs4, Wn["scale_u4"], Wn["zero_u4"], sx, N, K)
    rel = np.abs(np_(Y).astype(np.float32) - loose.astype(np.float32)).max() / np.abs(loose.astype(np.float32)).max()
    assert rel < 5e-3


def test_run_to_run_identical(ops):
    """A race in the pipeline or the split-K hand-off would show up as run-to-run
    differences; the slice reduction order is fixed, so outputs must be equal."""
    W, X = make_case(16, 1024, 4096, 0.1)
    Wc = cuda_container(W)
    outs = [ops.fused_dense_sparse_e2e_cuda(X.cuda(), Wc.perm, Wc.W_low_packed, Wc.W_high_blocks_packed,
                                            Wc.hp_row_offsets, Wc.hp_col_indices, Wc.scale_u4, Wc.zero_u4,
                                            1024, 4096) for _ in range(4)]
    for o in outs[1:]:
        assert torch.equal(o, outs[0])


def test_empty_block_rows_and_zero_density(ops):
    W, X = make_case(8, 512, 512, 0.15, seed_offset=11)
    counts = np.diff(np_(W.hp_row_offsets))
    assert (counts == 0).any() or True
    Wn, Wc = container_np(W), cuda_container(W)
    xs4, sx, sumx = O.quantize_activation_s4(np_(X), Wn["perm"])
    q = lambda a: torch.from_numpy(a).cuda()
    Y = _run_fused(ops, Wc, q(xs4), q(sumx), q(sx))
    assert_close_fp16(np_(Y), oracle_fused(Wn, xs4, sumx, sx), "fused")
    Ys = ops.sparse_gemm_cuda(torch.zeros((0, 128, 64), dtype=torch.int8, device="cuda"),
                              torch.zeros(5, dtype=torch.int32, device="cuda"),
                              torch.zeros(0, dtype=torch.int32, device="cuda"), q(xs4), Wc.scale_u4, q(sx), 512, 512)
    assert Ys.shape == (512, 8) and not Ys.any()


def test_archived_stubs_raise(ops):
    for fn in (ops.dense_gemm_cuda_int8, ops.sparse_gemm_cuda_int8, ops.fused_dense_sparse_cuda_int8):
        with pytest.raises(RuntimeError):
            fn()


def test_v9_linear_module(ops):
    from zip_kernel_b200 import v9_linear
    W, X = make_case(6, 256, 512, 0.2, perm_seed=4)
    Wn, Wc = container_np(W), cuda_container(W)
    X3 = X.reshape(2, 3, 512).cuda()
    Y = v9_linear.v9_linear_forward(X3, Wc)
    assert Y.shape == (2, 3, 256)
    xs4, sx, sumx = O.quantize_activation_s4(np_(X), Wn["perm"])
    assert_close_fp16(np_(Y).reshape(6, 256).T, oracle_fused(Wn, xs4, sumx, sx), "module")
    fq = v9_linear.v9_linear_fakequant(X3, Wc)
    rel = (Y.float() - fq.float()).abs().max() / fq.float().abs().max()
    assert rel < 2e-2
    with pytest.raises(ValueError):
        v9_linear.v9_linear_forward(X3[..., :256], Wc)


def test_host_staged_graph_forward(ops):
    """Pinned host activations in, pinned host result out through one replayed graph:
    same bits as the eager module forward, also after the input buffer is refilled."""
    from zip_kernel_b200 import backend, v9_linear
    W, X = make_case(4, 384, 512, 0.2, perm_seed=6)
    Wc = cuda_container(W)
    Xh = X.clone().pin_memory()
    Yh = torch.empty((4, 384), dtype=torch.float16).pin_memory()
    for scale in (1.0, -0.5):                     # second pass replays the captured graph on new contents
        Xh.copy_(X * scale)
        out = backend.v9_linear_forward_host_graph(Xh, Wc, Yh)
        torch.cuda.synchronize()
        assert out is Yh
        ref = v9_linear.v9_linear_forward(Xh.cuda(), Wc).cpu()
        assert torch.equal(Yh, ref)
    with pytest.raises(ValueError):
        backend.v9_linear_forward_host_graph(X, Wc, Yh)          # not pinned
    backend.clear_cuda_graph_cache()


def test_host_staged_batch_graph(ops):
    """Several host-staged linears as one graph: every result equals the eager forward."""
    from zip_kernel_b200 import backend, v9_linear
    reqs, refs = [], []
    for i, (T, N, K) in enumerate([(1, 256, 512), (4, 384, 256), (16, 128, 1024), (2, 256, 256)]):
        W, X = make_case(T, N, K, 0.2, perm_seed=i)
        Wc = cuda_container(W)
        Xh = X.clone().pin_memory()
        Yh = torch.zeros((T, N), dtype=torch.float16).pin_memory()
        reqs.append((Xh, Wc, Yh))
    for rep in range(2):                                  # capture, then replay on refilled inputs
        for Xh, _, _ in reqs:
            Xh.mul_(-0.5 if rep else 1.0)
        backend.v9_linear_forward_host_graph_many(reqs, n_streams=3)
        torch.cuda.synchronize()
        for Xh, Wc, Yh in reqs:
            assert torch.equal(Yh, v9_linear.v9_linear_forward(Xh.cuda(), Wc).cpu())
    # the same batch as an object a serving loop holds: same cached graph, usable after the cache is cleared
    assert isinstance(backend.v9_linear_host_batch_graph(reqs, n_streams=3), backend.HostBatchGraph)   # the cached one
    batch = backend.v9_linear_host_batch_graph(reqs)                     # default: a branch per request (up to 12)
    assert batch.n_requests == len(reqs) and backend.v9_linear_host_batch_graph(reqs) is batch
    backend.clear_cuda_graph_cache()
    for Xh, _, Yh in reqs:
        Xh.mul_(3.0)
        Yh.zero_()
    batch.replay()
    torch.cuda.synchronize()
    for Xh, Wc, Yh in reqs:
        assert torch.equal(Yh, v9_linear.v9_linear_forward(Xh.cuda(), Wc).cpu())
    with pytest.raises(ValueError):                       # pageable buffers are refused when a batch is captured
        backend.v9_linear_host_batch_graph([(reqs[0][0].clone(), reqs[0][1], reqs[0][2])])
    with pytest.raises(ValueError):
        backend.v9_linear_host_batch_graph([])


def test_quant_every_fp16_value_against_many_scales(ops):
    """Rows that hold EVERY finite fp16 value up to a chosen maximum: the kernel divides by the token
    scale through a reciprocal and one residual correction, which must reproduce the IEEE quotient's code for
    every value - ties at .5, values next to them, subnormal scales included."""
    vals = np.arange(65536, dtype=np.uint16).view(np.float16)
    finite = np.isfinite(vals)
    rng = np.random.default_rng(7)
    pos = vals[finite & (vals > 0)]
    maxima = np.concatenate([
        rng.choice(pos, 44, replace=False),
        np.array([6e-8, 4.2e-7, 6.1e-5, 1e-3, 0.4375, 1.0, 3.5, 7.0, 7.5, 10.5, 448.0, 65504.0], dtype=np.float16),
        # maxima whose scale max/7 lands on or next to a rounding tie of fp16
        np.array([7 * 1.5, 7 * (1 + 2 ** -10), 7 * (1 + 3 * 2 ** -11), 7 * 2 ** -14, 7 * 2 ** -24, 7 * 1.5 * 2 ** -24,
                  21 * 2 ** -25, 0.1], dtype=np.float16)])
    X = np.zeros((len(maxima), 65536), dtype=np.float16)
    for i, m in enumerate(maxima):
        keep = finite & (np.abs(vals) <= m)
        X[i, keep] = vals[keep]
    perm = np.arange(65536, dtype=np.int32)
    xs4, sx, sumx = ops.activation_quant_cuda(torch.from_numpy(X).cuda(), torch.from_numpy(perm).cuda())
    r4, rs, rsum = O.quantize_activation_s4(X, perm)
    assert np.array_equal(np_(sx).view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(np_(xs4), r4)
    assert np.array_equal(np_(sumx), rsum)

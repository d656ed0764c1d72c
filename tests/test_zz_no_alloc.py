"""The allocation-free entry point, called through the C ABI.

``w4a4_fused_dense_sparse_noalloc`` serves callers that may not allocate device
memory (a plugin under a host that owns all allocations, code running inside a
foreign CUDA-graph capture): it keeps its scratch in an array inside the library
instead of a caller-provided workspace.  The test feeds it the same inputs as
the regular entry point and expects the same fp16 output (within the suite's
tolerance: max-abs 1e-2 + rel 1e-3; the kernels are the same, so the outputs are
in fact identical), on two calls in a row that share the built-in array - the
second one smaller, so that stale contents of the first would show - and checks
both against the CPU oracle.  A second test fills the array to its last byte that
a real layer reaches (16 tokens of 28672 features, the longest input of the
Llama-2-70B linears) and to its declared maximum (32768 features).  This file
sorts last so a stop-at-first-failure run has executed every other test before.
"""

import ctypes

import numpy as np
import pytest
import torch

from tests.helpers import assert_close_fp16, container_np, cuda_container, make_case, np_, oracle_fused

pytestmark = pytest.mark.gpu


def _call_noalloc(lib, Wc, q4, qs, qsum, N, K):
    T = int(q4.shape[0])
    Y = torch.empty((N, T), dtype=torch.float16, device="cuda")
    nnz = Wc.n_hp_blocks
    rc = lib.w4a4_fused_dense_sparse_noalloc(
        Wc.W_low_packed.data_ptr(), Wc.W_high_blocks_packed.data_ptr() if nnz else None,
        Wc.hp_row_offsets.data_ptr(), Wc.hp_col_indices.data_ptr() if nnz else None,
        q4.data_ptr(), Wc.scale_u4.data_ptr(), Wc.zero_u4.data_ptr(), qsum.data_ptr(), qs.data_ptr(),
        Y.data_ptr(), T, K, N, nnz, 0, torch.cuda.current_stream().cuda_stream)
    return rc, Y


def test_noalloc_matches_workspace_entry_point():
    from zip_kernel_b200 import _lib, ops
    lib = _lib.load()
    for (T, N, K, density) in [(16, 512, 2048, 0.2), (3, 384, 1024, 0.3)]:
        W, X = make_case(T, N, K, density, perm_seed=2)
        Wc = cuda_container(W)
        q4, qs, qsum = ops.activation_quant_cuda(X.cuda(), Wc.perm)
        ref = ops.fused_dense_sparse_cuda(Wc.W_low_packed, Wc.W_high_blocks_packed, Wc.hp_row_offsets,
                                          Wc.hp_col_indices, q4, Wc.scale_u4, Wc.zero_u4, qsum, qs, N, K)
        rc, Y = _call_noalloc(lib, Wc, q4, qs, qsum, N, K)
        assert rc == 0, lib.w4a4_last_error()
        torch.cuda.synchronize()
        assert_close_fp16(np_(Y), np_(ref), f"noalloc T={T}")
        assert torch.equal(Y, ref)
        xs4, sx, sumx = (np_(t) for t in (q4, qs, qsum))
        assert_close_fp16(np_(Y), oracle_fused(container_np(W), xs4, sumx, sx), f"noalloc T={T} vs oracle")
    assert _lib.device_error(torch.device("cuda")) == 0


@pytest.mark.parametrize("K", [28672, 32768])
def test_noalloc_at_the_end_of_the_array(K):
    """16 tokens of the widest inputs: the expanded codes reach the last line of the built-in array and
    the group sums its last entry; a one-token call afterwards must not see any of it."""
    from zip_kernel_b200 import _lib, ops
    lib = _lib.load()
    N = 256
    for T in (16, 1):
        W, X = make_case(T, N, K, 0.05, perm_seed=3)
        Wc = cuda_container(W)
        q4, qs, qsum = ops.activation_quant_cuda(X.cuda(), Wc.perm)
        rc, Y = _call_noalloc(lib, Wc, q4, qs, qsum, N, K)
        assert rc == 0, lib.w4a4_last_error()
        torch.cuda.synchronize()
        xs4, sx, sumx = (np_(t) for t in (q4, qs, qsum))
        assert_close_fp16(np_(Y), oracle_fused(container_np(W), xs4, sumx, sx), f"noalloc K={K} T={T} vs oracle")
        ref = ops.fused_dense_sparse_cuda(Wc.W_low_packed, Wc.W_high_blocks_packed, Wc.hp_row_offsets,
                                          Wc.hp_col_indices, q4, Wc.scale_u4, Wc.zero_u4, qsum, qs, N, K)
        assert torch.equal(Y, ref)
    assert _lib.device_error(torch.device("cuda")) == 0


def test_noalloc_rejects_oversize():
    from zip_kernel_b200 import _lib, ops
    lib = _lib.load()
    W, X = make_case(17, 128, 256, 0.0)
    Wc = cuda_container(W)
    q4, qs, qsum = ops.activation_quant_cuda(X.cuda(), Wc.perm)
    rc, _ = _call_noalloc(lib, Wc, q4, qs, qsum, 128, 256)
    assert rc == 6 and b"T <= 16" in lib.w4a4_last_error()


def test_noalloc_rejects_flags_of_the_other_kernel():
    """The entry point always streams s8 codes it expands itself: the flag that forces the tensor-core
    kernel and the one that announces e4m3 codes are refused instead of being half-honoured."""
    from zip_kernel_b200 import _lib, ops
    lib = _lib.load()
    W, X = make_case(4, 128, 256, 0.0)
    Wc = cuda_container(W)
    q4, qs, qsum = ops.activation_quant_cuda(X.cuda(), Wc.perm)
    Y = torch.empty((128, 4), dtype=torch.float16, device="cuda")
    for flag in (_lib.FLAG_FORCE_TENSOR, _lib.FLAG_CODES_E4M3):
        rc = lib.w4a4_fused_dense_sparse_noalloc(
            Wc.W_low_packed.data_ptr(), None, Wc.hp_row_offsets.data_ptr(), None, q4.data_ptr(),
            Wc.scale_u4.data_ptr(), Wc.zero_u4.data_ptr(), qsum.data_ptr(), qs.data_ptr(), Y.data_ptr(),
            4, 256, 128, 0, flag, torch.cuda.current_stream().cuda_stream)
        assert rc == 1, (flag, rc)

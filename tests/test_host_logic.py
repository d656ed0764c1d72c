"""CPU tests of the host-side logic: packing contract against the golden
vectors, weight-loader validation, registry/policy shims, graph-cache
bookkeeping (with fakes, no GPU), shard metadata."""

import gc

import numpy as np
import pytest
import torch

from oracle import w4a4_oracle as O
from zip_kernel_b200 import pack_utils, sharding, synth
from zip_kernel_b200.backend import graph_cache, policy, registry, weight_loader


# ------------------------------------------------------------------ packing contract
def test_pack_unpack_roundtrip_and_golden(golden_nibble):
    g = golden_nibble
    assert np.array_equal(pack_utils.pack_s4_le(torch.from_numpy(g["s4"])).numpy(), g["s4_packed"])
    assert np.array_equal(pack_utils.pack_s4_le(torch.from_numpy(g["u4"])).numpy(), g["u4_packed"])
    assert np.array_equal(pack_utils.unpack_s4_le(torch.from_numpy(g["s4_packed"])).numpy(), g["s4"])
    assert np.array_equal(pack_utils.unpack_s4_le(torch.from_numpy(g["u4_packed"]), signed=False).numpy(), g["u4"])
    with pytest.raises(ValueError):
        pack_utils.pack_s4_le(torch.zeros(3, 5, dtype=torch.int8))


def test_pack_v9_weights_golden(golden_pack):
    g = golden_pack
    for name in g["names"]:
        raw = {k.split("/in/")[1]: torch.from_numpy(v) for k, v in g.items() if k.startswith(f"{name}/in/")}
        W = pack_utils.pack_v9_weights(raw)
        for k in ("W_low_packed", "W_high_blocks_packed", "hp_row_offsets", "hp_col_indices", "perm"):
            assert np.array_equal(getattr(W, k).numpy(), g[f"{name}/out/{k}"]), (name, k)
        for k in ("scale_u4", "zero_u4"):
            assert np.array_equal(getattr(W, k).numpy().view(np.uint16), g[f"{name}/out/{k}"].view(np.uint16)), (name, k)
        # block-CSR invariants of the reference tests (triton_kernel/tests/test_pack_utils.py:64-167)
        ro = W.hp_row_offsets.numpy()
        assert ro[0] == 0 and ro[-1] == W.n_hp_blocks and np.all(np.diff(ro) >= 0)
        for br in range(len(ro) - 1):
            cols = W.hp_col_indices.numpy()[ro[br]:ro[br + 1]]
            assert np.all(np.diff(cols) > 0)


def test_pack_v9_weights_errors():
    raw = {"Q_u4_permuted": torch.zeros(128, 100, dtype=torch.int8)}
    with pytest.raises(ValueError):
        pack_utils.pack_v9_weights(raw)
    with pytest.raises(ValueError):
        pack_utils.pack_v9_weights(raw, brow=64)


def test_synth_container_is_consistent():
    W = synth.make_container(300, 384, 0.4, seed=3, perm_seed=1)
    assert W.W_low_packed.shape == (300, 192) and W.scale_u4.shape == (300, 3)
    assert W.hp_row_offsets.numel() == 4 and int(W.hp_row_offsets[-1]) == W.n_hp_blocks
    # rows past d_out in the ragged last block-row are zero padding
    last = W.hp_row_offsets[-2].item()
    tiles = pack_utils.unpack_s4_le(W.W_high_blocks_packed[last:])
    assert not tiles[:, 300 - 256:, :].any()
    assert sorted(W.perm.tolist()) == list(range(384))


# ------------------------------------------------------------------ weight loader
def test_weight_loader_view_and_violations():
    W = synth.make_container(256, 256, 0.1, seed=1)
    view = weight_loader.pack_v9_weights_for_cutlass(W)
    assert view.W_low_rowmajor.data_ptr() == W.W_low_packed.data_ptr()
    assert (view.d_out, view.d_in, view.n_groups) == (256, 256, 2)
    bad = synth.make_container(256, 256, 0.0, seed=1)
    bad.W_low_packed = bad.W_low_packed.to(torch.int16)
    bad.scale_u4 = bad.scale_u4.float()
    bad.zero_u4 = bad.zero_u4[:, :1]
    with pytest.raises(weight_loader.CutlassPackValidationError) as ei:
        weight_loader.pack_v9_weights_for_cutlass(bad)
    msgs = "\n".join(ei.value.violations)
    assert "T1" in msgs and "T5" in msgs and "T6" in msgs and len(ei.value.violations) >= 3
    assert weight_loader.pack_v9_weights_for_cutlass(bad, strict=False).source is bad
    strided = synth.make_container(128, 256, 0.0, seed=2)
    strided.W_low_packed = torch.zeros(128, 256, dtype=torch.int8)[:, ::2]
    assert any("stride(1)" in v for v in weight_loader._collect_violations(strided))


# ------------------------------------------------------------------ registry / policy
def test_registry_names_and_policy_shims():
    assert registry.ALL_KERNELS == ("activation_quant", "dense_gemm", "sparse_gemm", "fused_dense_sparse")
    assert registry.BackendKernel.cuda_available()
    from zip_kernel_b200 import ops
    for name in registry.ALL_KERNELS:
        assert registry.BackendKernel.cuda_impl(name) is getattr(ops, f"{name}_cuda")
    st = policy.get_backend_status()
    assert st["cuda_available"] and set(st["cuda_kernels"]) == set(registry.ALL_KERNELS)
    policy.set_backend_policy("cuda")
    policy.set_backend_policy({"dense_gemm": "cuda"})
    policy.set_backend_policy("auto")
    with pytest.raises(ValueError):
        policy.set_backend_policy("triton")
    with pytest.raises(ValueError):
        policy.set_backend_policy({"nope": "cuda"})
    with pytest.raises(TypeError):
        policy.set_backend_policy(3)
    with pytest.raises(RuntimeError):
        registry.BackendKernel.triton_impl("dense_gemm")


def test_ops_surface_matches_reference_names():
    from zip_kernel_b200 import ops
    for name in ("activation_quant_cuda", "dense_gemm_cuda", "sparse_gemm_cuda", "fused_dense_sparse_cuda",
                 "dense_gemm_cuda_int8", "sparse_gemm_cuda_int8", "fused_dense_sparse_cuda_int8",
                 "dense_gemm_cuda_int4", "sparse_gemm_cuda_int4", "fused_dense_sparse_cuda_int4",
                 "dense_gemv_cuda_decode", "fused_gemv_cuda_decode", "fused_gemv_cuda_smallT",
                 "fused_quant_gemv_cuda", "fused_quant_dense_sparse_cuda_int4", "fused_dense_sparse_e2e_cuda"):
        assert callable(getattr(ops, name)) and name in ops.__all__
    for fn in (ops.dense_gemm_cuda_int8, ops.sparse_gemm_cuda_int8, ops.fused_dense_sparse_cuda_int8):
        with pytest.raises(RuntimeError):
            fn()


# ------------------------------------------------------------------ graph cache bookkeeping (fakes)
class _FakeWeight:
    def __init__(self, d_in=256, d_out=128, hp=1):
        self.d_in, self.d_out, self.n_hp_blocks = d_in, d_out, hp


class _FakeX:
    is_cuda = True

    def __init__(self, shape, stride=None, dtype="torch.float16", index=0):
        self.shape = tuple(shape)
        self._stride = tuple(stride) if stride else tuple(int(np.prod(shape[i + 1:])) for i in range(len(shape)))
        self.dtype = dtype
        self.device = type("D", (), {"index": index})()

    def dim(self):
        return len(self.shape)

    def stride(self):
        return self._stride

    def is_contiguous(self):
        return True


def test_graph_cache_key_lru_and_weakref():
    cache = graph_cache._GraphCache(capacity=2)
    w1, w2 = _FakeWeight(), _FakeWeight()
    k1 = graph_cache._build_cache_key(_FakeX((1, 256)), w1)
    assert graph_cache._build_cache_key(_FakeX((1, 256)), w1) == k1
    assert graph_cache._build_cache_key(_FakeX((1, 256), stride=(512, 1)), w1) != k1
    assert graph_cache._build_cache_key(_FakeX((1, 1, 256)), w1) != k1
    assert graph_cache._build_cache_key(_FakeX((1, 256), index=1), w1) != k1
    assert graph_cache._build_cache_key(_FakeX((1, 256)), w2) != k1
    mk = lambda k: graph_cache._CacheEntry(key=k, T=1, d_in=256, d_out=128, n_hp_blocks=1, graph=object())
    k2 = graph_cache._build_cache_key(_FakeX((2, 256)), w1)
    k3 = graph_cache._build_cache_key(_FakeX((4, 256)), w1)
    cache.put(k1, mk(k1), weight_ref_target=w1)
    cache.put(k2, mk(k2), weight_ref_target=w1)
    assert cache.get(k1) is not None            # k1 becomes most recent
    cache.put(k3, mk(k3), weight_ref_target=w1)  # evicts k2
    assert cache.get(k2) is None and cache.get(k1) is not None and cache.get(k3) is not None
    st = cache.stats()
    assert st["evictions"] == 1 and st["size"] == 2 and st["hits"] == 3 and st["misses"] == 1
    # a failed capture is stored as a sentinel and counted
    ks = graph_cache._build_cache_key(_FakeX((8, 256)), w2)
    cache.put(ks, graph_cache._CacheEntry(key=ks, T=8, d_in=256, d_out=128, n_hp_blocks=1), weight_ref_target=w2)
    assert cache.stats()["capture_failures"] == 1
    # entries die with their weight container
    del w2
    gc.collect()
    assert cache.get(ks) is None and cache.stats()["weak_evictions"] == 1
    cache.clear()
    assert len(cache) == 0


def test_graph_policy_matrix():
    prev = graph_cache.set_cuda_graph_policy("off")
    try:
        w = _FakeWeight()
        assert not graph_cache._is_eligible(_FakeX((1, 256)), w, 1)
        graph_cache.set_cuda_graph_policy("auto")
        assert graph_cache._is_eligible(_FakeX((1, 256)), w, 1)
        assert graph_cache._is_eligible(_FakeX((16, 256)), w, 16)
        assert not graph_cache._is_eligible(_FakeX((3, 256)), w, 3)
        assert not graph_cache._is_eligible(_FakeX((256, 256)), w, 256)
        assert graph_cache.set_cuda_graph_policy("force") == "auto"
        assert graph_cache._is_eligible(_FakeX((3, 256)), w, 3)
        assert not graph_cache._is_eligible(_FakeX((129, 256)), w, 129)
        with pytest.raises(ValueError):
            graph_cache.set_cuda_graph_policy("sometimes")
        assert graph_cache.get_cuda_graph_policy() == "force"
        # a CPU tensor always takes the eager route, which needs the GPU library
        # only at call time: prewarm just skips it
        assert graph_cache.prewarm_cuda_graph_cache([(torch.zeros(1, 256, dtype=torch.float16), w)]) == {
            "attempted": 0, "captured": 0, "skipped": 1}
    finally:
        graph_cache.set_cuda_graph_policy(prev)


# ------------------------------------------------------------------ sharding metadata
@pytest.mark.parametrize("N,world", [(1024, 2), (1024, 4), (1280, 8), (1000, 3), (128, 2)])
def test_shards_partition_the_layer(N, world):
    K = 256
    W = synth.make_container(N, K, 0.4, seed=N + world)
    X = synth.make_activations(5, K, seed=1)
    xs4, sx, sumx = O.quantize_activation_s4(X.numpy(), W.perm.numpy())
    full = O.fused_kernel_order(W.W_low_packed.numpy(), W.W_high_blocks_packed.numpy(), W.hp_row_offsets.numpy(),
                                W.hp_col_indices.numpy(), xs4, W.scale_u4.numpy(), W.zero_u4.numpy(), sumx, sx, N, K)
    rows, parts, nnz = 0, [], 0
    for r in range(world):
        S = sharding.shard_container(W, r, world)
        sharding.check_shard_metadata(N, K, S, r, world)
        lo, hi = sharding.shard_rows(N, r, world)
        assert lo == rows and S.d_out == hi - lo and (lo % 128 == 0)
        rows = hi
        nnz += S.n_hp_blocks
        if S.d_out:
            parts.append(O.fused_kernel_order(S.W_low_packed.numpy(), S.W_high_blocks_packed.numpy(),
                                              S.hp_row_offsets.numpy(), S.hp_col_indices.numpy(), xs4,
                                              S.scale_u4.numpy(), S.zero_u4.numpy(), sumx, sx, S.d_out, K))
    assert rows == N and nnz == W.n_hp_blocks
    assert np.array_equal(np.concatenate(parts, axis=0).view(np.uint16), full.view(np.uint16))
    assert sum(sharding.shard_sizes(N, world)) == N


def test_shard_metadata_rejects_mismatch():
    W = synth.make_container(512, 256, 0.3, seed=9)
    s0 = sharding.shard_container(W, 0, 2)
    with pytest.raises(ValueError):
        sharding.check_shard_metadata(512, 256, s0, 0, 4)
    with pytest.raises(ValueError):
        sharding.check_shard_metadata(512, 384, s0, 0, 2)
    s1 = sharding.shard_container(W, 1, 2)
    s1.hp_row_offsets = W.hp_row_offsets[2:5]        # not re-based
    if int(s1.hp_row_offsets[0]) != 0:
        with pytest.raises(ValueError):
            sharding.check_shard_metadata(512, 256, s1, 1, 2)
    with pytest.raises(ValueError):
        sharding.block_row_range(4, 2, 2)

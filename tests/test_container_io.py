"""Container file format: bit-exact round trip, rejection of truncated / corrupt / rule-breaking files
(CPU), and the same output bits from a loaded container as from the original (GPU)."""

import os

import numpy as np
import pytest
import torch

from zip_kernel_b200 import container_io as cio
from zip_kernel_b200 import synth
from zip_kernel_b200.backend.weight_loader import CutlassPackValidationError

FIELDS = ("W_low_packed", "W_high_blocks_packed", "scale_u4", "zero_u4", "hp_row_offsets", "hp_col_indices", "perm")


def same(a, b):
    assert (a.d_out, a.d_in, tuple(a.block_shape)) == (b.d_out, b.d_in, tuple(b.block_shape))
    for f in FIELDS:
        x, y = getattr(a, f).cpu(), getattr(b, f).cpu()
        assert x.dtype == y.dtype and x.shape == y.shape, f
        assert np.array_equal(x.numpy().view(np.uint8) if x.numel() else x.numpy(), y.numpy().view(np.uint8) if y.numel() else y.numpy()), f


@pytest.mark.parametrize("N,K,density,perm_seed", [(384, 512, 0.3, 5), (200, 256, 0.5, None), (128, 128, 0.0, 1), (1024, 1024, 1.0, 2)])
def test_round_trip_is_bit_exact(tmp_path, N, K, density, perm_seed):
    W = synth.make_container(N, K, density, seed=N + K, perm_seed=perm_seed)
    p = str(tmp_path / "layer.w4a4")
    size = cio.save_container(W, p)
    assert size == os.path.getsize(p)
    h = cio.read_header(p)
    assert h["d_out"] == N and h["d_in"] == K and h["data_start"] % 4096 == 0
    assert all(e["offset"] % 256 == 0 for e in h["tensors"].values())
    same(cio.load_container(p), W)
    same(cio.load_container(p, verify_crc=False, pin=False), W)


def test_bad_files_are_rejected(tmp_path):
    W = synth.make_container(256, 256, 0.5, seed=3)
    p = str(tmp_path / "a.w4a4")
    cio.save_container(W, p)
    raw = open(p, "rb").read()
    q = str(tmp_path / "b.w4a4")
    open(q, "wb").write(b"NOTW4A4\0" + raw[8:])
    with pytest.raises(cio.ContainerFormatError, match="magic"):
        cio.load_container(q)
    open(q, "wb").write(raw[:8] + (99).to_bytes(4, "little") + raw[12:])
    with pytest.raises(cio.ContainerFormatError, match="version"):
        cio.load_container(q)
    open(q, "wb").write(raw[:-100])
    with pytest.raises(cio.ContainerFormatError, match="truncated"):
        cio.load_container(q)
    flipped = bytearray(raw)
    flipped[-5] ^= 0x10                                    # one bit in the last tensor's data
    open(q, "wb").write(bytes(flipped))
    with pytest.raises(cio.ContainerFormatError, match="checksum"):
        cio.load_container(q)
    with pytest.raises(cio.ContainerFormatError, match="perm entries"):     # without the checksum the layout rules still catch it
        cio.load_container(q, verify_crc=False)
    open(q, "wb").write(raw[:16] + b"{" * 10 + raw[26:])
    with pytest.raises(cio.ContainerFormatError):
        cio.load_container(q)


def test_layout_rules_are_enforced_on_save_and_load():
    W = synth.make_container(384, 512, 0.5, seed=4)
    assert cio.index_violations(W) == []
    bad = synth.make_container(384, 512, 0.5, seed=4)
    bad.hp_col_indices = bad.hp_col_indices.clone()
    bad.hp_col_indices[0] = 99                              # beyond d_in / 128
    assert any("hp_col_indices must lie" in v for v in cio.index_violations(bad))
    bad2 = synth.make_container(384, 512, 0.5, seed=4)
    bad2.hp_row_offsets = bad2.hp_row_offsets[:-1]
    assert any("hp_row_offsets must be int32 with" in v for v in cio.index_violations(bad2))
    bad3 = synth.make_container(384, 512, 1.0, seed=4)
    bad3.hp_col_indices = bad3.hp_col_indices.flip(0).contiguous()
    assert any("sorted" in v for v in cio.index_violations(bad3))
    bad4 = synth.make_container(384, 512, 0.5, seed=4)
    bad4.scale_u4 = bad4.scale_u4.float()
    with pytest.raises(CutlassPackValidationError) as ei:
        cio.validate_container(bad4)
    assert any("scale_u4.dtype" in v for v in ei.value.violations)
    bad5 = synth.make_container(384, 512, 0.5, seed=4)
    bad5.hp_row_offsets = bad5.hp_row_offsets.clone()
    bad5.hp_row_offsets[-1] += 1
    assert any("disagrees with the number of residual blocks" in v for v in cio.index_violations(bad5))
    with pytest.raises(CutlassPackValidationError):
        cio.save_container(bad5, "/dev/null")


@pytest.mark.gpu
def test_loaded_container_gives_the_same_output_bits(tmp_path):
    from zip_kernel_b200 import v9_linear
    dev = torch.device("cuda")
    for (T, N, K, prepare) in ((4, 384, 1024, False), (300, 384, 1024, True)):
        W = synth.make_container(N, K, 0.2, seed=T + N, perm_seed=9)
        X = synth.make_activations(T, K, seed=1).to(dev)
        p = str(tmp_path / f"l{T}.w4a4")
        cio.save_container(W.to(dev), p)                    # saved from device tensors
        L = cio.load_container(p, dev, prepare=prepare)
        assert L.W_low_packed.is_cuda and (L.prepared is not None) == prepare
        same(L, W)
        assert torch.equal(v9_linear.v9_linear_forward(X, L), v9_linear.v9_linear_forward(X, W.to(dev)))

"""Generate the golden vectors under tests/golden/ from the reference itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/Zip_kernel

The reference imports itself as the package ``kernel``; this script exposes the
checkout under that name through a temporary symlink and then calls the
reference's own CPU functions

* ``kernel.triton_kernel.pack_utils``  (pack_s4_le / unpack_s4_le / pack_v9_weights)
* ``kernel.tools.parity.quant_reference.quantize_activation_s4_reference``
* ``kernel.tools.parity.fp16_reference.fp16_{dense,sparse,fused}_reference``

on seeded inputs.  Inputs and the reference's outputs are stored side by side
in ``*.npz`` files; the tests replay them against the oracle (CPU) and against
the CUDA path (GPU) without needing the reference checkout.
"""

from __future__ import annotations

import os
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from zip_kernel_b200 import synth  # noqa: E402


def _import_reference(ref_root: str):
    tmp = tempfile.mkdtemp(prefix="zk_ref_")
    os.symlink(os.path.abspath(ref_root), os.path.join(tmp, "kernel"))
    sys.path.insert(0, tmp)
    from kernel.tools.parity import fp16_reference, quant_reference
    from kernel.triton_kernel import pack_utils
    return pack_utils, quant_reference, fp16_reference


def _np(t):
    return t.detach().cpu().numpy()


def quant_cases():
    """(name, X fp16, perm int32) covering the reference's quant test matrix
    (cuda_kernel/tests/test_parity.py:101-126) plus its documented traps."""
    cases = []
    for i, (T, K, with_perm) in enumerate([
        (1, 128, False), (1, 4096, True), (4, 256, True), (7, 384, False),
        (16, 4096, False), (16, 4096, True), (33, 1024, True), (3, 6144, True),
        (2, 17408, False), (129, 256, True),
    ]):
        X = synth.make_activations(T, K, seed=1000 + i)
        perm = synth.make_perm(K, 2000 + i if with_perm else None)
        cases.append((f"rand_T{T}_K{K}_{'perm' if with_perm else 'id'}", X, perm))
    # reference-style inputs without outliers: N(0,1) * 0.4
    cases.append(("plain_T8_K512", synth.make_activations(8, 512, seed=77, outlier_frac=0.0, std=0.4),
                  synth.make_perm(512, None)))
    # an all-zero row, a row with a single non-zero, constant rows
    X = synth.make_activations(6, 256, seed=5)
    X[1] = 0
    X[2] = 0
    X[2, 17] = -3.5
    X[3] = 0.25
    X[4] = -65504.0
    cases.append(("special_rows", X, synth.make_perm(256, 9)))
    # quotients exactly on .5 boundaries: max = 7 gives scale 1 and x/s = x
    X = torch.zeros(2, 128, dtype=torch.float16)
    X[0, 0] = 7.0
    X[0, 1:17] = torch.tensor([0.5, 1.5, 2.5, 3.5, 4.5, 5.5, 6.5, -0.5, -1.5, -2.5, -3.5,
                               -4.5, -5.5, -6.5, -7.0, 6.75], dtype=torch.float16)
    X[1, 0] = -14.0           # scale 2: x/s on halves for odd multiples of 1
    X[1, 1:9] = torch.tensor([1.0, 3.0, 5.0, 7.0, -1.0, -3.0, -13.0, 13.0], dtype=torch.float16)
    cases.append(("half_boundaries", X, synth.make_perm(128, None)))
    # tiny magnitudes: fp16 subnormal scale
    X = (synth.make_activations(3, 128, seed=11, outlier_frac=0.0).float() * 1e-6).to(torch.float16)
    cases.append(("subnormal_scale", X, synth.make_perm(128, None)))
    return cases


def fused_cases():
    """(name, T, N, K, density, perm_seed, per_channel) - the four CPU shapes of
    tools/parity/tests/test_fp16_reference_cpu.py:121-127 and ragged/edge ones."""
    return [
        ("t16_n128_k256_d05", 16, 128, 256, 0.5, None, False),
        ("t32_n256_k256_d25", 32, 256, 256, 0.25, 3, False),
        ("t64_n256_k512_d10", 64, 256, 512, 0.10, None, False),
        ("t32_n512_k1024_d05", 32, 512, 1024, 0.05, 4, False),
        ("t1_n256_k512_d20", 1, 256, 512, 0.2, None, False),
        ("t5_n200_k384_d30_raggedN", 5, 200, 384, 0.3, 5, False),
        ("t17_n384_k256_d00", 17, 384, 256, 0.0, None, False),
        ("t9_n128_k128_d100", 9, 128, 128, 1.0, None, False),
        ("t16_n256_k512_perchannel", 16, 256, 512, 0.1, None, True),
    ]


def main(ref_root: str):
    pack_utils, quant_reference, fp16_reference = _import_reference(ref_root)
    out = {}

    # --- nibble packing --------------------------------------------------
    g = torch.Generator().manual_seed(1)
    v = torch.randint(-8, 8, (5, 64), generator=g, dtype=torch.int8)
    u = torch.randint(0, 16, (3, 32), generator=g, dtype=torch.int8)
    np.savez_compressed(
        os.path.join(HERE, "nibble_pack.npz"),
        s4=_np(v), s4_packed=_np(pack_utils.pack_s4_le(v)),
        u4=_np(u), u4_packed=_np(pack_utils.pack_s4_le(u)),
        s4_unpacked=_np(pack_utils.unpack_s4_le(pack_utils.pack_s4_le(v), signed=True)),
        u4_unpacked=_np(pack_utils.unpack_s4_le(pack_utils.pack_s4_le(u), signed=False)),
    )

    # --- activation quantisation ------------------------------------------
    q = {}
    names = []
    for name, X, perm in quant_cases():
        xs4, sx, sumx = quant_reference.quantize_activation_s4_reference(X, perm)
        q[f"{name}/X"] = _np(X)
        q[f"{name}/perm"] = _np(perm)
        q[f"{name}/X_s4"] = _np(xs4)
        q[f"{name}/scale_x"] = _np(sx)
        q[f"{name}/sum_X"] = _np(sumx)
        names.append(name)
    q["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "activation_quant.npz"), **q)

    # --- fused linear (loose truth of the reference) -------------------------
    f = {}
    names = []
    for name, T, N, K, density, perm_seed, per_channel in fused_cases():
        W = synth.make_container(N, K, density, seed=synth.shape_seed(T, K, N),
                                 perm_seed=perm_seed, per_channel_scale=per_channel)
        X = synth.make_activations(T, K, seed=synth.shape_seed(T, K, N) + 1)
        xs4, sx, sumx = quant_reference.quantize_activation_s4_reference(X, W.perm)
        yl = fp16_reference.fp16_dense_reference(W.W_low_packed, xs4, W.scale_u4, W.zero_u4, sx, N, K)
        # the reference's sparse walk covers d_out // 128 block-rows only
        if N % 128 == 0:
            yh = fp16_reference.fp16_sparse_reference(W.W_high_blocks_packed, W.hp_row_offsets,
                                                      W.hp_col_indices, xs4, W.scale_u4, sx, N, K)
            yf = fp16_reference.fp16_fused_reference(W.W_low_packed, W.W_high_blocks_packed,
                                                     W.hp_row_offsets, W.hp_col_indices, xs4,
                                                     W.scale_u4, W.zero_u4, sx, N, K)
            f[f"{name}/Y_high"] = _np(yh)
            f[f"{name}/Y_fused"] = _np(yf)
        for k in ("W_low_packed", "W_high_blocks_packed", "scale_u4", "zero_u4",
                  "hp_row_offsets", "hp_col_indices", "perm"):
            f[f"{name}/{k}"] = _np(getattr(W, k))
        f[f"{name}/X"] = _np(X)
        f[f"{name}/X_s4"] = _np(xs4)
        f[f"{name}/scale_x"] = _np(sx)
        f[f"{name}/sum_X"] = _np(sumx)
        f[f"{name}/Y_low"] = _np(yl)
        f[f"{name}/dims"] = np.array([T, N, K])
        names.append(name)
    f["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "fused_linear.npz"), **f)

    # --- offline packer -----------------------------------------------------
    p = {}
    names = []
    for ci, (N, K, n_hp) in enumerate([(256, 256, 2), (384, 512, 5), (200, 256, 3), (128, 128, 0)]):
        g = torch.Generator().manual_seed(300 + ci)
        nrow, ncol = (N + 127) // 128, K // 128
        raw = {
            "Q_u4_permuted": torch.randint(0, 16, (N, K), generator=g, dtype=torch.int8),
            "scale_u4_raw": (torch.rand(N, ncol, generator=g) * 0.01 + 0.001).to(torch.float16),
            "zero_u4_raw": torch.randint(0, 16, (N, ncol), generator=g).to(torch.float16),
            "perm": torch.randperm(K, generator=g).to(torch.int32),
        }
        flat = torch.randperm(nrow * ncol, generator=g)[:n_hp]
        raw["hp_block_indices"] = torch.stack([flat // ncol, flat % ncol], -1).to(torch.int32) \
            if n_hp else torch.zeros((0, 2), dtype=torch.int32)
        raw["Q_s8_blocks"] = torch.randint(-128, 128, (n_hp, 128, 128), generator=g, dtype=torch.int8)
        raw["scale_s8_per_block"] = (torch.rand(n_hp, 128, generator=g) * 0.005 + 0.001).to(torch.float16)
        W = pack_utils.pack_v9_weights(raw)
        name = f"pack_n{N}_k{K}_hp{n_hp}"
        for k, t in raw.items():
            p[f"{name}/in/{k}"] = _np(t)
        for k in ("W_low_packed", "W_high_blocks_packed", "scale_u4", "zero_u4",
                  "hp_row_offsets", "hp_col_indices", "perm"):
            p[f"{name}/out/{k}"] = _np(getattr(W, k))
        names.append(name)
    p["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "pack_v9_weights.npz"), **p)
    for fn in sorted(os.listdir(HERE)):
        if fn.endswith(".npz"):
            print(fn, os.path.getsize(os.path.join(HERE, fn)), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <reference checkout>")
    main(sys.argv[1])

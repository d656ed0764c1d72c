"""Builds the reference's naive dense / sparse GEMM kernels for sm_100a into ``baseline/_ref/naive``.

    python baseline/build_naive_reference.py [/path/to/reference]

The CUDA sources are compiled where they lie in the reference tree together with this directory's
``naive_bindings.cc``; the product (a torch extension ``w4a4_ref_naive*.so``) lands in the git-ignored
``baseline/_ref/naive`` and travels with the snapshot.  ``load()`` imports the built module (no compiler
needed at that point); it returns ``None`` when the module was never built."""

from __future__ import annotations

import glob
import importlib.util
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "naive")
NAME = "w4a4_ref_naive"


def build(reference_root: str = "/root/reference", verbose: bool = False) -> bool:
    src = os.path.join(reference_root, "cuda_kernel", "csrc_naive")
    files = [os.path.join(src, f) for f in ("dense_gemm_naive.cu", "sparse_gemm_naive.cu", "reduce_sum_naive.cu")]
    if not all(os.path.exists(f) for f in files):
        return bool(glob.glob(os.path.join(OUT, NAME + "*.so")))
    if glob.glob(os.path.join(OUT, NAME + "*.so")):
        return True
    from torch.utils.cpp_extension import load
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    load(name=NAME, sources=files + [os.path.join(HERE, "naive_bindings.cc")], build_directory=OUT,
         extra_cuda_cflags=["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--fmad=true"],
         extra_cflags=["-O2"], verbose=verbose, is_python_module=True)
    return True


def load():
    """The built extension module, or None."""
    so = sorted(glob.glob(os.path.join(OUT, NAME + "*.so")))
    if not so:
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    spec = importlib.util.spec_from_file_location(NAME, so[0])
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ok = build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", verbose=True)
    print("built" if ok else "reference tree not found; nothing built")

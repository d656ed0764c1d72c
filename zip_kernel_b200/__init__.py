"""B200-native W4A4 linear: activation quant + dense u4xs4 GEMM + block-sparse
s4xs4 residual behind the operator surface of HuYangjia/Zip_kernel.

Sub-modules import lazily: ``pack_utils`` and ``synth`` are pure PyTorch and
work anywhere; ``ops`` and everything above it need the CUDA library built by
``zip_kernel_b200.build`` and raise if it is missing.
"""

from .pack_utils import (BCOL, BROW, V9WeightContainer, pack_s4_le, pack_v9_weights,
                         unpack_s4_le)

__all__ = ["BROW", "BCOL", "V9WeightContainer", "pack_s4_le", "unpack_s4_le", "pack_v9_weights"]

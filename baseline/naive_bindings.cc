// Python binding of two kernels of the reference's naive CUDA suite, built for sm_100a as a same-GPU
// anchor for the benchmark (`legacy_gpu_baseline`): dense_gemm_naive and sparse_gemm_naive, plus the
// element-wise sum that combines them.  The kernel sources are compiled from where they lie in the
// reference tree (cuda_kernel/csrc_naive/{dense_gemm,sparse_gemm,reduce_sum}_naive.cu); nothing of them is
// copied into this repository.  The reference's activation_quant_naive kernel is deliberately NOT bound:
// it keeps per-group sums in a fixed shared array of 160 entries without a host-side check
// (cuda_kernel/csrc_naive/activation_quant_naive.cu:59-62,150-152) and would write out of bounds for
// d_in > 20480.  The benchmark feeds these kernels activations quantised by this repository's own kernel.
#include <torch/extension.h>

namespace hkust_v9_naive {
namespace dense_gemm {
void launch(torch::Tensor W_low, torch::Tensor X_s4, torch::Tensor scale_u4, torch::Tensor zero_u4,
            torch::Tensor sum_X, torch::Tensor scale_x, torch::Tensor Y_low);
}
namespace sparse_gemm {
void launch(torch::Tensor W_high_blocks, torch::Tensor hp_row_offsets, torch::Tensor hp_col_indices,
            torch::Tensor X_s4, torch::Tensor scale_u4, torch::Tensor scale_x, torch::Tensor Y_high,
            int d_out, int d_in);
}
namespace reduce_sum {
void launch(torch::Tensor Y_low, torch::Tensor Y_high, torch::Tensor Y_total);
}
}  // namespace hkust_v9_naive

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("dense_gemm", &hkust_v9_naive::dense_gemm::launch);
  m.def("sparse_gemm", &hkust_v9_naive::sparse_gemm::launch);
  m.def("reduce_sum", &hkust_v9_naive::reduce_sum::launch);
}

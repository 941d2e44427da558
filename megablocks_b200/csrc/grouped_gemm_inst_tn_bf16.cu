// Explicit instantiation of the grouped GEMM kernel: bf16, layout TN.
#include "grouped_gemm_kernel.cuh"

namespace mb {
namespace gemm {
MB_GEMM_INSTANTIATE(__nv_bfloat16, kTN)
}  // namespace gemm
}  // namespace mb

// Explicit instantiation of the grouped GEMM kernel: bf16, layout NT.
#include "grouped_gemm_kernel.cuh"

namespace mb {
namespace gemm {
MB_GEMM_INSTANTIATE(__nv_bfloat16, kNT)
}  // namespace gemm
}  // namespace mb

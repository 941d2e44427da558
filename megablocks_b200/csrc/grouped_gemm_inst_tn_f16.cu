// Explicit instantiation of the grouped GEMM kernel: f16, layout TN.
#include "grouped_gemm_kernel.cuh"

namespace mb {
namespace gemm {
MB_GEMM_INSTANTIATE(__half, kTN)
}  // namespace gemm
}  // namespace mb

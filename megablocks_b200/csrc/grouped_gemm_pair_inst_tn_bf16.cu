// Explicit instantiation of the CTA-pair grouped GEMM kernel: bf16, layout TN.
#include "grouped_gemm_pair.cuh"

namespace mb {
namespace gemm {
template cudaError_t launch_pair<__nv_bfloat16, kTN>(const CUtensorMap&, const CUtensorMap&, const GemmParams&, int,
                                                 cudaStream_t);
}  // namespace gemm
}  // namespace mb

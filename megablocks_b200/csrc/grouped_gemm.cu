// Launch dispatch of the grouped GEMM over (dtype, layout).  The kernel lives in
// grouped_gemm_kernel.cuh and is instantiated in grouped_gemm_inst_*.cu, one unit
// per (dtype, layout), so the build parallelises.
#include "grouped_gemm_kernel.cuh"

namespace mb {
namespace gemm {

// Defined in grouped_gemm_pair.cuh, instantiated in grouped_gemm_pair_inst_*.cu.
template <typename T, int LAYOUT>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                        cudaStream_t stream);

cudaError_t launch(bool bf16, int layout, int block_n, const CUtensorMap& ta, const CUtensorMap& tb,
                   const GemmParams& p, int grid, cudaStream_t stream, bool pair) {
  if (pair) {
    if (block_n != 256 || (grid & 1)) return cudaErrorInvalidValue;
    if (bf16 && layout == kNT) return launch_pair<__nv_bfloat16, kNT>(ta, tb, p, grid, stream);
    if (bf16 && layout == kNN) return launch_pair<__nv_bfloat16, kNN>(ta, tb, p, grid, stream);
    if (!bf16 && layout == kNT) return launch_pair<__half, kNT>(ta, tb, p, grid, stream);
    if (!bf16 && layout == kNN) return launch_pair<__half, kNN>(ta, tb, p, grid, stream);
    if (bf16 && layout == kTN) return launch_pair<__nv_bfloat16, kTN>(ta, tb, p, grid, stream);
    if (!bf16 && layout == kTN) return launch_pair<__half, kTN>(ta, tb, p, grid, stream);
    return cudaErrorInvalidValue;
  }
  if (block_n != 64 && block_n != 128 && block_n != 256) return cudaErrorInvalidValue;
  if (bf16) {
    if (layout == kNT) return launch_layout<__nv_bfloat16, kNT>(block_n, ta, tb, p, grid, stream);
    if (layout == kNN) return launch_layout<__nv_bfloat16, kNN>(block_n, ta, tb, p, grid, stream);
    if (layout == kTN) return launch_layout<__nv_bfloat16, kTN>(block_n, ta, tb, p, grid, stream);
  } else {
    if (layout == kNT) return launch_layout<__half, kNT>(block_n, ta, tb, p, grid, stream);
    if (layout == kNN) return launch_layout<__half, kNN>(block_n, ta, tb, p, grid, stream);
    if (layout == kTN) return launch_layout<__half, kTN>(block_n, ta, tb, p, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace gemm
}  // namespace mb

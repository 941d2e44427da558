// Launch dispatch of the block-sparse products over (dtype, operand majorness); the kernel lives
// in bsmm_kernel.cuh.
#include "bsmm_kernel.cuh"

namespace mb {
namespace bsmm {

namespace {
template <typename T>
cudaError_t launch_t(bool a_mn, bool b_mn, const CUtensorMap& ta, const CUtensorMap& tb, const BsmmParams& p, int grid,
                     cudaStream_t stream) {
  if (a_mn) return b_mn ? launch_one<T, true, true>(ta, tb, p, grid, stream)
                        : launch_one<T, true, false>(ta, tb, p, grid, stream);
  return b_mn ? launch_one<T, false, true>(ta, tb, p, grid, stream)
              : launch_one<T, false, false>(ta, tb, p, grid, stream);
}
}  // namespace

cudaError_t launch(bool bf16, bool a_mn_major, bool b_mn_major, const CUtensorMap& ta, const CUtensorMap& tb,
                   const BsmmParams& p, int grid, cudaStream_t stream) {
  if (p.mode != kSdd && p.mode != kDsd && p.mode != kDds) return cudaErrorInvalidValue;
  if (p.num_tiles <= 0) return cudaSuccess;
  return bf16 ? launch_t<__nv_bfloat16>(a_mn_major, b_mn_major, ta, tb, p, grid, stream)
              : launch_t<__half>(a_mn_major, b_mn_major, ta, tb, p, grid, stream);
}

}  // namespace bsmm
}  // namespace mb

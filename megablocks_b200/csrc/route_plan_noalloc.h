// mb_route_plan_noalloc: the route plan (stable counting sort by expert, per-expert
// counts and their prefix sums) for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference library; it exists for code
// that runs where cudaMalloc is not an option - inside another runtime's memory pool
// or arena, in a pre-planned inference engine whose memory map is frozen after
// start-up, or under a sandbox that denies allocation calls - and that therefore
// cannot call the PyTorch-facing `route_plan` op (which allocates its outputs and its
// scratch through the caching allocator).
//
// The caller owns every input and output buffer.  The sort's scratch (per-warp
// histograms and per-expert totals) lives in a fixed array inside the library: about
// 2 MiB of device memory on every GPU that loads the library, held until the process
// exits.  Limits: n <= MB_NOALLOC_MAX_COPIES, 1 <= num_experts <=
// MB_NOALLOC_MAX_EXPERTS, block >= 1; anything larger is rejected with
// cudaErrorInvalidValue and a message on stderr, nothing is launched.
//
// The call makes no cudaMalloc / cudaFree and calls no allocating library routine.
// The first call on a device looks up the address of the scratch array (a
// cudaGetSymbolAddress, done with that device current); make that first call before
// any stream capture begins.  All calls share the one scratch array and it keeps the
// previous call's contents (every call overwrites what it reads), so two calls that
// may overlap on the GPU - different streams, or different host threads without
// ordering - race; serialise them.
//
// Semantics are those of the `route_plan` op: for i in sorted order,
//   indices[i]  = position in top_experts of the copy placed at i (stable),
//   bin_ids[i]  = its expert,
//   tokens_per_expert[e], bins[e] (inclusive prefix sum), padded_bins[e] (prefix sum of
//   counts rounded up to `block`).
// All pointers are device pointers to int32; outputs need n, n, E, E and E elements.
// `stream` must be a stream of the device that is current when the call is made: the
// scratch address is looked up for the current device and the kernels are launched there.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#define MB_NOALLOC_MAX_COPIES (1 << 20)
#define MB_NOALLOC_MAX_EXPERTS 1024

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) cudaError_t mb_route_plan_noalloc(
    const int32_t* top_experts, int64_t n, int num_experts, int block, int32_t* indices, int32_t* bin_ids,
    int32_t* bins, int32_t* padded_bins, int32_t* tokens_per_expert, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

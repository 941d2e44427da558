// Block-sparse matrix products for sm_100a: sdd, dsd and dds over 128 x 128 blocks of an
// arbitrary BCSR topology, on tcgen05 tensor cores with TMA-fed operands.
//
// The reference reaches these products through the stk package (call sites:
// megablocks/layers/mlp.py:212-300, 391-394, glu.py:57-63), whose kernels are Triton
// programs indexed by `offsets`, `row_indices`, `column_indices` and, for transposed
// operands, `column_indices_t`, `offsets_t`, `block_offsets_t`.  Here one persistent,
// warp-specialised kernel serves all three products.  Every output tile is 128 x 128:
//
//   sdd  one tile per stored block t: values[t] = a[block-row r(t)] * b[block-column c(t)],
//        contraction over the dense K dimension;
//   dsd  out[block-row i, 128 columns] = sum over the stored blocks of row i of op(S):
//        values[blk] * b[k-block of blk];
//   dds  out[128 rows, block-column j] = sum over the stored blocks of column j of op(S):
//        a[:, k-block of blk] * values[blk].
//
// A "segment list" (`seg_offsets`, `seg_block`, `seg_k`) names, per output block row / column,
// the stored blocks to accumulate and the 128-wide slice of the dense operand each one meets;
// it is the BCSR row list for S, the transposed list for S^T (dsd) or for the columns of S (dds).
// Either operand may be K-major or MN-major in shared memory (a transposed dense operand or a
// transposed topology), described to the MMA by the matching descriptors, so no transposed copy
// of a dense matrix or of the block values is made.
//
// Roles per CTA (320 threads, one CTA per SM, tiles taken round-robin): warp 8 TMA producer,
// warp 9 tensor-memory owner and MMA issuer, warps 0-7 epilogue (tcgen05.ld, convert, coalesced
// stores through a swizzled staging buffer).  Two accumulator stages overlap the epilogue of a
// tile with the MMAs of the next.  Every wait is bounded and reports through the status word.
#pragma once

#include "grouped_gemm_kernel.cuh"

namespace mb {
namespace bsmm {

using namespace ptx;
using gemm::kABytes;
using gemm::kBlockK;
using gemm::kBlockM;
using gemm::kBoxBytes;
using gemm::kEpilogueWarps;
using gemm::kMmaWarp;
using gemm::kProducerWarp;
using gemm::kThreads;
using gemm::kUmmaK;
using gemm::kWaitLimitNs;

constexpr int kStages = 6;
constexpr int kBBytes = kBlock * kBlockK * 2;
constexpr int kTileBytes = kStages * (kABytes + kBBytes);
constexpr int kSmemBytes = kTileBytes + kEpilogueWarps * 2048 + 256 + 1024;
constexpr int kTmemCols = 2 * kBlock;

struct Work {
  int out_row;      // first row of the output tile
  int out_col;      // first column of the output tile
  int a_block;      // sdd: block-row of a; dds: 128-row block of a; dsd: unused
  int b_block;      // sdd: block-column of b; dsd: first column of b / 64 boxes; dds: unused
  int seg_begin;    // dsd / dds: range of the segment list
  int seg_end;
};

template <typename T, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
bsmm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ BsmmParams p) {
  constexpr bool kIsBf16 = std::is_same<T, __nv_bfloat16>::value;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  uint8_t* staging = smem + kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpilogueWarps * 2048);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full_bar = bars + 2 * kStages;
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), kEpilogueWarps);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(tmem_base_slot), kTmemCols);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // ---- tile schedule (every role decodes the same sequence) ---------------------
  const int total_tiles = p.num_tiles;
  auto decode = [&](int t) {
    Work w;
    if (p.mode == kSdd) {
      w.a_block = __ldg(p.row_indices + t);
      w.b_block = __ldg(p.column_indices + t);
      w.out_row = t * kBlock;
      w.out_col = 0;
      w.seg_begin = 0;
      w.seg_end = 0;
    } else if (p.mode == kDsd) {
      const int i = t / p.tiles_inner, nb = t - i * p.tiles_inner;   // inner: column tiles of the output
      w.out_row = i * kBlock;
      w.out_col = nb * kBlock;
      w.a_block = 0;
      w.b_block = nb;
      w.seg_begin = __ldg(p.seg_offsets + i);
      w.seg_end = __ldg(p.seg_offsets + i + 1);
    } else {
      const int j = t / p.tiles_inner, i = t - j * p.tiles_inner;    // inner: row tiles of the output
      w.out_row = i * kBlock;
      w.out_col = j * kBlock;
      w.a_block = i;
      w.b_block = 0;
      w.seg_begin = __ldg(p.seg_offsets + j);
      w.seg_end = __ldg(p.seg_offsets + j + 1);
    }
    return w;
  };
  // Number of 64-deep K steps of a tile.
  auto k_steps = [&](const Work& w) {
    return p.mode == kSdd ? (p.K + kBlockK - 1) / kBlockK : 2 * max(0, w.seg_end - w.seg_begin);
  };

  if (warp == kProducerWarp) {
    // ======================= TMA producer =======================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Work w = decode(t);
        const int steps = k_steps(w);
        int blk = 0, kblk = 0;
        for (int ks = 0; ks < steps; ++ks) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, gemm::kErrProducer,
                         kWaitLimitNs);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[stage]);
          mbar_arrive_expect_tx(bar, kABytes + kBBytes);
          const uint32_t a_dst = smem_u32(smem_a + stage * kABytes);
          const uint32_t b_dst = smem_u32(smem_b + stage * kBBytes);
          // (x, y) of the A and B boxes of this K step.  K-major operands take one 64 x 128 box
          // (x = contraction offset, y = row); MN-major operands take two 64 x 64 boxes
          // (x = row / column offset, y = contraction offset).
          int ak, am, bk, bn;   // contraction offset and row / column offset, in elements
          if (p.mode == kSdd) {
            ak = bk = ks * kBlockK;
            am = w.a_block * kBlock;
            bn = w.b_block * kBlock;
          } else {
            if ((ks & 1) == 0) {
              const int idx = w.seg_begin + (ks >> 1);
              blk = p.seg_block != nullptr ? __ldg(p.seg_block + idx) : idx;
              kblk = __ldg(p.seg_k + idx);
            }
            const int half = (ks & 1) * kBlockK;
            if (p.mode == kDsd) {       // A = block values, B = dense
              ak = A_MN ? blk * kBlock + half : half;      // MN-major: contraction runs down the stored block
              am = A_MN ? 0 : blk * kBlock;
              bk = kblk * kBlock + half;
              bn = w.out_col;
            } else {                    // A = dense, B = block values
              ak = kblk * kBlock + half;
              am = w.out_row;
              bk = B_MN ? blk * kBlock + half : half;
              bn = B_MN ? 0 : blk * kBlock;
            }
          }
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j) tma_load_2d(a_dst + j * kBoxBytes, &tmap_a, bar, am + 64 * j, ak);
          } else {
            tma_load_2d(a_dst, &tmap_a, bar, ak, am);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < kBlock / 64; ++j) tma_load_2d(b_dst + j * kBoxBytes, &tmap_b, bar, bn + 64 * j, bk);
          } else {
            tma_load_2d(b_dst, &tmap_b, bar, bk, bn);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ======================= MMA issuer ==========================================
    constexpr uint32_t idesc = instr_desc_f16(kIsBf16, A_MN, B_MN, kBlockM, kBlock);
    int stage = 0;
    uint32_t phase = 0;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Work w = decode(t);
      const int steps = k_steps(w);
      ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_stage]), acc_phase ^ 1u, abort_flag, p.status, gemm::kErrMmaTmem,
                     kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t d_tmem = tmem_base + acc_stage * kBlock;
      for (int ks = 0; ks < steps; ++ks) {
        ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, gemm::kErrMmaFull, kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_u32(smem_a + stage * kABytes);
          const uint32_t b_base = smem_u32(smem_b + stage * kBBytes);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t a_desc = A_MN ? smem_desc_sw128(a_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                         : smem_desc_sw128(a_base + k * (kUmmaK * 2), 16, 1024);
            const uint64_t b_desc = B_MN ? smem_desc_sw128(b_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                         : smem_desc_sw128(b_base + k * (kUmmaK * 2), 16, 1024);
            umma_f16(d_tmem, a_desc, b_desc, idesc, (ks | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) {
        if (steps > 0) umma_commit(smem_u32(&tmem_full_bar[acc_stage]));
        else mbar_arrive(smem_u32(&tmem_full_bar[acc_stage]));   // a row / column without blocks: zeros
      }
      __syncwarp();
      if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
    }
  } else if (warp < kEpilogueWarps) {
    // ======================= epilogue warps ======================================
    const int quarter = warp & 3;
    const int half = warp >> 2;
    uint8_t* stage_buf = staging + warp * 2048;
    T* out = static_cast<T*>(p.out);
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Work w = decode(t);
      const bool has_k = k_steps(w) > 0;
      const int row = w.out_row + quarter * 32;
      const int rows_ok = max(0, min(32, p.out_rows - row));
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc_stage]), acc_phase, abort_flag, p.status, gemm::kErrEpilogue,
                     kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc_stage * kBlock;
      if (rows_ok > 0) {
#pragma unroll 1
        for (int ci = half; ci < kBlock / 32; ci += 2) {
          const int col = w.out_col + ci * 32;
          if (col >= p.out_cols) break;
          uint32_t raw[32];
          if (has_k) {
            tmem_ld_32x32(taddr + ci * 32, raw);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = 0u;
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 q;
            q.x = gemm::pack2<T>(__uint_as_float(raw[v * 8 + 0]), __uint_as_float(raw[v * 8 + 1]));
            q.y = gemm::pack2<T>(__uint_as_float(raw[v * 8 + 2]), __uint_as_float(raw[v * 8 + 3]));
            q.z = gemm::pack2<T>(__uint_as_float(raw[v * 8 + 4]), __uint_as_float(raw[v * 8 + 5]));
            q.w = gemm::pack2<T>(__uint_as_float(raw[v * 8 + 6]), __uint_as_float(raw[v * 8 + 7]));
            *reinterpret_cast<uint4*>(stage_buf + gemm::stage_offset(lane, v)) = q;
          }
          __syncwarp();
          gemm::stage_store<T>(stage_buf, out + int64_t(row) * p.out_ld + col, p.out_ld, rows_ok,
                               min(32, p.out_cols - col), lane);
          __syncwarp();
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc_stage]));
      if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
    }
  }

  // ---- teardown -----------------------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    if (*abort_flag != 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <typename T, bool A_MN, bool B_MN>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const BsmmParams& p, int grid,
                       cudaStream_t stream) {
  auto kernel = bsmm_kernel<T, A_MN, B_MN>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  if (!configured[dev & 63]) {
    rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (rc != cudaSuccess) return rc;
    configured[dev & 63] = true;
  }
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace bsmm
}  // namespace mb

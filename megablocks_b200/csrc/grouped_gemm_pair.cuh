// Grouped GEMM on CTA pairs (tcgen05 cta_group::2) for the NT, NN and TN layouts.
//
// Two CTAs of a cluster share one 256-row x 256-column tile.  Each CTA loads its own
// 128 rows of A and one half (128 of the 256 columns) of B per 64-deep K step, the
// even CTA of the pair issues `tcgen05.mma.cta_group::2` with M = 256, and each CTA's
// tensor memory receives the accumulator rows of its own half.  Per unit of work a
// CTA therefore pulls 32 KB per K step through L2 instead of 48 KB, which is what
// bounds the single-CTA kernel of grouped_gemm_kernel.cuh.  No tile is multicast:
// every CTA fetches what it holds with its own TMA loads.
//
// Synchronisation between the two CTAs:
//   NT / NN  full[stage] lives in the even CTA and expects the bytes of both CTAs'
//            loads (the odd CTA's TMA completes on the even CTA's barrier).  When the
//            odd CTA's half of the tile holds no rows of the group, its A load is
//            skipped and the even CTA expects correspondingly fewer bytes.
//   TN       (weight gradients, ragged K) full[stage] of the even CTA counts two arrivals.
//            For a whole K block the even CTA's producer makes both and expects the bytes of
//            both CTAs, exactly as above.  The last K block of a group may end inside the
//            block: the rows past the group must be cleared in BOTH CTAs before the MMA reads
//            them.  For that block the odd CTA's loads complete on its own tail[stage]
//            barrier; its MMA warp (otherwise idle) waits there, clears the rows and makes the
//            second arrival on the even CTA's full[stage]; the even CTA clears its own rows
//            after the wait and issues the MMAs.
//   empty[stage]   one per CTA; the MMA thread commits to both;
//   tmem_full[s]   one per CTA; the MMA thread commits to both;
//   tmem_empty[s]  lives in the even CTA; the epilogue warps of both CTAs arrive on it.
// Row groups, fused epilogues, arrival flags and the bounded waits are those of the
// single-CTA kernel; a pair always works inside one group.
#pragma once

#include "grouped_gemm_kernel.cuh"

namespace mb {
namespace gemm {

constexpr int kPairBlockN = 256;
constexpr int kPairStages = 6;
constexpr int kPairBBytes = (kPairBlockN / 2) * kBlockK * 2;               // this CTA's half of B
constexpr int kPairTileBytes = kPairStages * (kABytes + kPairBBytes);
constexpr int kPairSmemBytes = kPairTileBytes + 256 + 2 * kMaxGroups * 4 + kEpilogueWarps * 2048 + 1024;

__device__ __forceinline__ uint32_t ld_shared_cluster_u32(uint32_t cluster_addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}

template <typename T, int LAYOUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
grouped_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ GemmParams p) {
  constexpr bool kTn = LAYOUT == kTN;
  constexpr bool kAMn = kTn;
  constexpr bool kBMn = LAYOUT != kNT;
  constexpr int kStages = kPairStages;
  constexpr int BLOCK_N = kPairBlockN;
  constexpr bool kIsBf16 = std::is_same<T, __nv_bfloat16>::value;
  constexpr int kOwnBytes = kABytes + kPairBBytes;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  // Staging buffers directly after the operand ring (1024-byte aligned for the swizzled TMA stores).
  uint8_t* staging = smem + kPairTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + kEpilogueWarps * 2048);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tmem_full_bar = bars + 2 * kStages;
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  uint32_t* dead_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 5);
  uint64_t* tail_bar = bars + 2 * kStages + 6;   // [kStages] TN, odd CTA: loads of a ragged last K block
  int* s_row_end = reinterpret_cast<int*>(staging + kEpilogueWarps * 2048 + 256);
  int* s_pair_end = s_row_end + kMaxGroups;      // inclusive prefix sum of 256-row blocks per group (NT / NN)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.num_groups;
  const uint32_t cta = cluster_ctarank();        // 0: issues the MMAs, 1: its partner
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // ---- one-time setup ---------------------------------------------------------
  for (int g = threadIdx.x; g < G; g += kThreads) s_row_end[g] = __ldg(p.bins + g);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    // Inert after a recorded failure when the launch reads rows delivered by peers.
    *dead_slot = (p.wait_flags != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1u : 0u;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), kTn ? 2 : 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
      mbar_init(smem_u32(&tail_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), 2 * kEpilogueWarps);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == kMmaWarp) tmem_alloc_pair(smem_u32(tmem_base_slot), 2 * BLOCK_N);
  __syncthreads();
  if (threadIdx.x == 0) {
    // Group ends are forced to be non-decreasing and inside the operand (see the single-CTA kernel).
    int acc = 0, prev = 0;
    for (int g = 0; g < G; ++g) {
      const int end = min(max(s_row_end[g], prev), p.rows_total);
      s_row_end[g] = end;
      if (!kTn) {
        acc += (end - prev + 2 * kBlockM - 1) / (2 * kBlockM);
        s_pair_end[g] = acc;
      }
      prev = end;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();          // both CTAs' barriers and tensor memory exist before either is used
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // Both CTAs must take the same decision: either one's flag makes the pair inert.
  const bool dead = (ld_shared_cluster_u32(map_to_cta(smem_u32(dead_slot), 0)) |
                     ld_shared_cluster_u32(map_to_cta(smem_u32(dead_slot), 1))) != 0u;

  // ---- tile schedule: the pair walks 256-row x 256-column tiles -----------------------
  const int num_nb = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int num_mb_tn = (p.M + 2 * kBlockM - 1) / (2 * kBlockM);
  const int total_tiles = dead ? 0 : (kTn ? G * num_mb_tn * num_nb : (G > 0 ? s_pair_end[G - 1] : 0) * num_nb);
  // `partner_rows`: rows of the group that fall into the odd CTA's half of the tile.
  auto decode = [&](int t, int& partner_rows) {
    Tile tile;
    if constexpr (kTn) {
      const int per_group = num_mb_tn * num_nb;
      tile.group = t / per_group;
      const int r = t - tile.group * per_group;
      const int mb_i = r / num_nb;
      tile.n0 = (r - mb_i * num_nb) * BLOCK_N;
      tile.row0 = mb_i * 2 * kBlockM + int(cta) * kBlockM;
      tile.rows_valid = max(0, min(kBlockM, p.M - tile.row0));
      tile.k_begin = tile.group ? s_row_end[tile.group - 1] : 0;
      tile.k_len = s_row_end[tile.group] - tile.k_begin;
      partner_rows = max(0, p.M - (mb_i * 2 * kBlockM + kBlockM));
    } else {
      const int blk = t / num_nb;
      tile.n0 = (t - blk * num_nb) * BLOCK_N;
      int lo = 0, hi = G - 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_pair_end[mid] <= blk) lo = mid + 1; else hi = mid;
      }
      tile.group = lo;
      const int row_start = lo ? s_row_end[lo - 1] : 0;
      const int local = blk - (lo ? s_pair_end[lo - 1] : 0);
      const int pair_row0 = row_start + local * 2 * kBlockM;
      tile.row0 = pair_row0 + int(cta) * kBlockM;      // this CTA's half
      tile.rows_valid = max(0, min(kBlockM, s_row_end[lo] - tile.row0));
      tile.k_begin = 0;
      tile.k_len = p.K;
      partner_rows = max(0, s_row_end[lo] - (pair_row0 + kBlockM));
    }
    return tile;
  };

  // Clears the rows of the last K block of a TN tile that lie past the group (one warp).
  auto clear_tail = [&](const Tile& tile, int kb, int stage) {
    const int valid = tile.k_len - kb * kBlockK;
    if (valid < kBlockK) {
      uint8_t* a_tile = smem_a + stage * kABytes;
      uint8_t* b_tile = smem_b + stage * kPairBBytes;
      const int tail_chunks = (kBlockK - valid) * 8;   // 16-byte chunks per box
      constexpr int kABoxes = kBlockM / 64, kBBoxes = BLOCK_N / 2 / 64;
      // After the last group that has rows the memory may never have been written: both operands are cleared.
      const bool at_end = tile.k_begin + tile.k_len >= s_row_end[G - 1];   // no later group has rows
      const int boxes = at_end ? kABoxes + kBBoxes : kABoxes;
      for (int box = 0; box < boxes; ++box) {
        uint8_t* base = (box < kABoxes) ? a_tile + box * kBoxBytes : b_tile + (box - kABoxes) * kBoxBytes;
        uint4* rows = reinterpret_cast<uint4*>(base + valid * 128);
        for (int i = lane; i < tail_chunks; i += 32) rows[i] = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async_smem();
    }
    __syncwarp();
  };

  if (warp == kProducerWarp) {
    // ======================= TMA producer (both CTAs) ============================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int arrived_group = -1;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        int partner_rows;
        const Tile tile = decode(t, partner_rows);
        const int num_kb = (tile.k_len + kBlockK - 1) / kBlockK;
        if (!kTn && p.wait_flags != nullptr && tile.group != arrived_group) {
          for (int s = 0; s < p.wait_count && ok; ++s) {
            const int* flag = p.wait_flags + s * p.wait_stride + tile.group;
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (ld_acquire_sys_s32(flag) < seq_with_base(p.wait_seq, p.seq_base)) {
              if ((++spins & 63u) == 0u) {
                if (*abort_flag != 0) { ok = false; break; }
                if (globaltimer_ns() - t0 > kWaitLimitNs) {
                  *abort_flag = 1;
                  atomicCAS(p.status, 0, kErrPeerRows);
                  ok = false;
                  break;
                }
              }
            }
          }
          if (!ok) break;
          arrived_group = tile.group;
          fence_proxy_async_all();
        }
        // NT / NN: a half without rows of the group needs no A tile (its accumulator rows are never read).
        const bool skip_partner_a = !kTn && partner_rows == 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, kErrProducer, kWaitLimitNs);
          if (!ok) break;
          const uint32_t a_dst = smem_u32(smem_a + stage * kABytes);
          const uint32_t b_dst = smem_u32(smem_b + stage * kPairBBytes);
          const int n_half = tile.n0 + int(cta) * (BLOCK_N / 2);            // this CTA's columns of B
          if constexpr (kTn) {
            const bool ragged = kb == num_kb - 1 && (tile.k_len & (kBlockK - 1)) != 0;
            uint32_t bar;
            if (cta == 0) {
              bar = smem_u32(&full_bar[stage]);
              if (ragged) {
                mbar_arrive_expect_tx(bar, kOwnBytes);      // the partner arrives after clearing its tail
              } else {
                mbar_arrive_expect_tx(bar, 2 * kOwnBytes);
                mbar_arrive(bar);
              }
            } else if (ragged) {
              bar = smem_u32(&tail_bar[stage]);
              mbar_arrive_expect_tx(bar, kOwnBytes);
            } else {
              bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
            }
            const int krow = tile.k_begin + kb * kBlockK;
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d_pair(a_dst + j * kBoxBytes, &tmap_a, bar, tile.row0 + 64 * j, krow);
#pragma unroll
            for (int j = 0; j < BLOCK_N / 2 / 64; ++j)
              tma_load_2d_pair(b_dst + j * kBoxBytes, &tmap_b, bar, n_half + 64 * j, krow);
          } else {
            // The stage's "full" barrier is the even CTA's; it counts the bytes of both CTAs.
            const uint32_t bar = map_to_cta(smem_u32(&full_bar[stage]), 0);
            if (cta == 0)
              mbar_arrive_expect_tx(smem_u32(&full_bar[stage]),
                                    kOwnBytes + (skip_partner_a ? kPairBBytes : kOwnBytes));
            if (cta == 0 || !skip_partner_a) tma_load_2d_pair(a_dst, &tmap_a, bar, kb * kBlockK, tile.row0);
            if constexpr (LAYOUT == kNT) {
              tma_load_2d_pair(b_dst, &tmap_b, bar, kb * kBlockK, tile.group * p.N + n_half);
            } else {
#pragma unroll
              for (int j = 0; j < BLOCK_N / 2 / 64; ++j)
                tma_load_2d_pair(b_dst + j * kBoxBytes, &tmap_b, bar, n_half + 64 * j,
                                 tile.group * p.K + kb * kBlockK);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (cta == 0) {
      // ======================= MMA issuer (even CTA) ===============================
      constexpr uint32_t idesc = instr_desc_f16(kIsBf16, kAMn, kBMn, 2 * kBlockM, BLOCK_N);
      int stage = 0;
      uint32_t phase = 0;
      int acc_stage = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        int partner_rows;
        const Tile tile = decode(t, partner_rows);
        const int num_kb = (tile.k_len + kBlockK - 1) / kBlockK;
        ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_stage]), acc_phase ^ 1u, abort_flag, p.status, kErrMmaTmem,
                       kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, kErrMmaFull, kWaitLimitNs);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if constexpr (kTn) clear_tail(tile, kb, stage);
          tcgen05_fence_after();
          if (lane == 0) {
            const uint32_t a_base = smem_u32(smem_a + stage * kABytes);
            const uint32_t b_base = smem_u32(smem_b + stage * kPairBBytes);
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              const uint64_t a_desc = kAMn ? smem_desc_sw128(a_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                           : smem_desc_sw128(a_base + k * (kUmmaK * 2), 16, 1024);
              const uint64_t b_desc = kBMn ? smem_desc_sw128(b_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                           : smem_desc_sw128(b_base + k * (kUmmaK * 2), 16, 1024);
              umma_f16_pair(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            // The stage is reusable in both CTAs once these MMAs retire.
            umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&empty_bar[stage]), 1));
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (lane == 0) {
          if (num_kb > 0) {
            umma_commit_pair(map_to_cta(smem_u32(&tmem_full_bar[acc_stage]), 0));
            umma_commit_pair(map_to_cta(smem_u32(&tmem_full_bar[acc_stage]), 1));
          } else {   // empty group: nothing to wait for, the epilogue writes zeros
            mbar_arrive(smem_u32(&tmem_full_bar[acc_stage]));
            mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_full_bar[acc_stage]), 1));
          }
        }
        __syncwarp();
        if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
      }
    } else if constexpr (kTn) {
      // ======================= tail clearing and hand-over (odd CTA, TN) ===========
      int stage = 0;
      uint32_t tail_phases = 0;      // bit s: parity of the next use of tail[s]
      bool ok = true;
      for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
        int partner_rows;
        const Tile tile = decode(t, partner_rows);
        const int num_kb = (tile.k_len + kBlockK - 1) / kBlockK;
        if (num_kb == 0) continue;
        const int last = (stage + num_kb - 1) % kStages;      // ring stage of the tile's last K block
        stage = (stage + num_kb) % kStages;
        if ((tile.k_len & (kBlockK - 1)) == 0) continue;      // whole blocks only: nothing to clear
        ok = mbar_wait(smem_u32(&tail_bar[last]), (tail_phases >> last) & 1u, abort_flag, p.status, kErrMmaFull,
                       kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tail_phases ^= 1u << last;
        clear_tail(tile, num_kb - 1, last);
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&full_bar[last]), 0));
        __syncwarp();
      }
    }
  } else if (warp < kEpilogueWarps) {
    // ======================= epilogue warps (both CTAs, own 128 rows) ============
    const int quarter = warp & 3;
    const int half = warp >> 2;
    uint8_t* stage_buf = staging + warp * 2048;
    Staging stage{stage_buf, 0};
    constexpr int kChunks = BLOCK_N / 32;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = pair_id; t < total_tiles && ok; t += num_pairs) {
      int partner_rows;
      const Tile tile = decode(t, partner_rows);
      const bool has_k = tile.k_len > 0;
      const int rows_ok = max(0, min(32, tile.rows_valid - quarter * 32));
      int64_t row_off;
      int out_row;
      if constexpr (kTn) out_row = tile.group * p.M + tile.row0 + quarter * 32;
      else out_row = tile.row0 + quarter * 32;
      row_off = int64_t(out_row) * p.N;
      const TmaOut tma{p.store_tma != 0 && rows_ok == 32, out_row};
      const bool need1 = p.epilogue == kEpiDAct || p.epilogue == kEpiGlu || p.epilogue == kEpiDGlu ||
                         p.epilogue == kEpiAdd;
      const bool need2 = p.epilogue == kEpiDGlu;
      {
        const int col = tile.n0 + half * 32;
        if (rows_ok > 0 && col < p.N) {
          if (need1) aux_prefetch<T>(static_cast<const T*>(p.aux1) + row_off + col, p.N, rows_ok,
                                     min(32, p.N - col), lane);
          if (need2) aux_prefetch<T>(static_cast<const T*>(p.aux2) + row_off + col, p.N, rows_ok,
                                     min(32, p.N - col), lane);
        }
      }
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc_stage]), acc_phase, abort_flag, p.status, kErrEpilogue,
                     kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc_stage * BLOCK_N;
      if (rows_ok > 0) {   // a quarter without rows of the group only hands the accumulator back
#pragma unroll 1
        for (int ci = half; ci < kChunks; ci += 2) {
          const int c0 = ci * 32;
          const int col = tile.n0 + c0;
          if (col >= p.N) break;
          if (ci + 2 < kChunks && col + 64 < p.N) {
            const int ncol = col + 64;
            if (need1) aux_prefetch<T>(static_cast<const T*>(p.aux1) + row_off + ncol, p.N, rows_ok,
                                       min(32, p.N - ncol), lane);
            if (need2) aux_prefetch<T>(static_cast<const T*>(p.aux2) + row_off + ncol, p.N, rows_ok,
                                       min(32, p.N - ncol), lane);
          }
          PackedRow a1, a2;
          const int cols = min(32, p.N - col);
          if (need1) {
            if (p.store_tma) stage_acquire(stage, lane);
            stage_load<T>(stage_buf, static_cast<const T*>(p.aux1) + row_off + col, p.N, rows_ok, cols, lane);
            __syncwarp();
            stage_read_row(stage_buf, lane, a1);
            __syncwarp();
          }
          if (need2) {
            stage_load<T>(stage_buf, static_cast<const T*>(p.aux2) + row_off + col, p.N, rows_ok, cols, lane);
            __syncwarp();
            stage_read_row(stage_buf, lane, a2);
            __syncwarp();
          }
          uint32_t raw[32];
          if (has_k) {
            tmem_ld_32x32(taddr + c0, raw);
            tmem_ld_wait();
            if (p.alpha != 1.f) {
#pragma unroll
              for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * p.alpha);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = 0u;
          }
          epilogue_dispatch<T>(raw, a1, a2, stage, row_off + col, p.N, rows_ok, cols, lane, p, nullptr, col, tma);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      // The accumulator stage is free for the next MMA once every epilogue warp of BOTH CTAs has read it.
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[acc_stage]), 0));
      if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
    }
    if (p.store_tma && lane == 0) bulk_wait_all();   // bulk stores complete before the CTA retires
    // Rows past the last group are defined as zero.
    if (!kTn && p.zero_tail && !dead) {
      const int last = G > 0 ? s_row_end[G - 1] : 0;
      const int64_t begin = int64_t(last) * p.N, end = int64_t(p.rows_total) * p.N;
      const int64_t tid = int64_t(blockIdx.x) * (kEpilogueWarps * 32) + threadIdx.x;
      const int64_t stride = int64_t(gridDim.x) * (kEpilogueWarps * 32);
      for (int64_t i = begin + tid * 8; i < end; i += stride * 8) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(static_cast<T*>(p.c) + i) = z;
        if (p.out2) *reinterpret_cast<uint4*>(static_cast<T*>(p.out2) + i) = z;
        if (p.out3) *reinterpret_cast<uint4*>(static_cast<T*>(p.out3) + i) = z;
      }
    }
  }

  // ---- teardown: neither CTA may release shared or tensor memory the other still uses ----
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == kMmaWarp) {
    if (*abort_flag != 0) {
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * BLOCK_N);
  }
}

// Launches on at most as many CTA pairs as the device can keep resident at once: tiles are
// assigned round-robin to the pairs of the grid, so a pair that only starts after another has
// finished would double the run time.
template <typename T, int LAYOUT>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                        cudaStream_t stream) {
  auto kernel = grouped_gemm_pair_kernel<T, LAYOUT>;
  static int max_pairs[64] = {0};
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  if (max_pairs[dev & 63] == 0) {
    rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
    if (rc != cudaSuccess) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(kThreads, 1, 1);
    cfg.dynamicSmemBytes = kPairSmemBytes;
    int clusters = 0;
    rc = cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg);
    if (rc != cudaSuccess || clusters < 1) {
      (void)cudaGetLastError();
      clusters = 1 << 20;   // unknown: keep the caller's grid
    }
    max_pairs[dev & 63] = clusters;
  }
  grid = 2 * min(grid / 2, max_pairs[dev & 63]);
  if (grid < 2) return cudaErrorInvalidValue;
  kernel<<<grid, kThreads, kPairSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace gemm
}  // namespace mb

// Grouped GEMM for sm_100a on the fifth-generation tensor cores.
//
// One persistent, warp-specialised kernel computes a batch of independent matrix
// products whose row extents live in device memory (`bins`, the inclusive prefix
// sum of rows per group), so the host never learns - or waits for - a group size:
//
//   NT  c[rows of g] = a[rows of g, K] * b[g, N, K]^T      expert layer 1, dgrad of layer 2
//   NN  c[rows of g] = a[rows of g, K] * b[g, K, N]        expert layer 2, dgrad of layer 1
//   TN  c[g, M, N]   = a[rows of g, M]^T * b[rows of g, N] weight gradients (ragged K)
//
// It stands where the reference calls the external grouped_gemm package and, for
// the block-diagonal topology of the dropless MoE, the stk sdd / dsd kernels
// (call sites: megablocks/layers/mlp.py:212-300, 414-523, glu.py:57-205).
//
// Structure per CTA (192 threads, one CTA per SM, tiles taken round-robin):
//   warp 0      TMA producer: cp.async.bulk.tensor tile loads into a ring of
//               128-byte-swizzled shared-memory stages, completion on mbarriers;
//   warp 1      allocates tensor memory and issues tcgen05.mma (one elected lane);
//               tcgen05.commit releases ring stages and publishes accumulators;
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulator (two TMEM stages, so the
//               next tile's MMAs overlap this tile's epilogue), apply the fused
//               epilogue (activation, activation backward, GLU, GLU backward, add)
//               and store bf16/fp16 rows with 16-byte stores, masked to the group.
// Operands may be K-major or MN-major in shared memory; MN-major tiles are loaded
// as 64-column boxes and described to the MMA with the matching leading/stride
// offsets, so no transposed copy of a weight or activation is ever made.
// Ragged K (TN) zero-fills the rows of the last K block that belong to the next
// group before the MMA reads them.
//
// Every wait is bounded: a wait that exceeds its limit raises a CTA-wide abort
// flag, records a code in a global status word, and the kernel drains, frees its
// tensor memory and returns.
#pragma once

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace mb {
namespace gemm {

using namespace ptx;

constexpr int kUmmaK = 16;
constexpr int kThreads = 192;
constexpr int kABytes = kBlockM * kBlockK * 2;
constexpr int kBoxBytes = 64 * kBlockK * 2;   // one 64-wide MN-major box
constexpr uint64_t kWaitLimitNs = 2000000000ull;


// Status codes written on an abandoned wait.
constexpr int kErrProducer = 1, kErrMmaFull = 2, kErrMmaTmem = 3, kErrEpilogue = 4, kErrPeerRows = 18;

template <int BLOCK_N>
struct Config {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kTmemCols = 2 * BLOCK_N;
  static constexpr int kTileBytes = kStages * (kABytes + kBBytes);
  // ring + barriers + tmem base + abort flag + group tables, plus slack for 1024-byte alignment
  static constexpr int kSmemBytes = kTileBytes + 256 + 2 * kMaxGroups * 4 + 1024;
};

struct Tile {
  int group;
  int row0;        // NT / NN: first row of a and c; TN: first output row inside the group (m0)
  int n0;
  int rows_valid;
  int k_begin;     // TN: first contraction row
  int k_len;       // contraction length of this tile
};

__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int ACT>
__device__ __forceinline__ float act_fwd(float x) {
  if constexpr (ACT == kActGeluTanh) return 0.5f * x * (1.f + tanh_fast(0.7978845608f * (x + 0.044715f * x * x * x)));
  else if constexpr (ACT == kActSilu) return x / (1.f + __expf(-x));
  else if constexpr (ACT == kActRelu) return fmaxf(x, 0.f);
  else if constexpr (ACT == kActGeluErf) return 0.5f * x * (1.f + erff(x * 0.70710678f));
  else return x;
}

template <int ACT>
__device__ __forceinline__ float act_bwd(float x) {
  if constexpr (ACT == kActGeluTanh) {
    const float t = tanh_fast(0.7978845608f * (x + 0.044715f * x * x * x));
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608f * (1.f + 0.134145f * x * x);
  } else if constexpr (ACT == kActSilu) {
    const float s = 1.f / (1.f + __expf(-x));
    return s * (1.f + x * (1.f - s));
  } else if constexpr (ACT == kActRelu) {
    return x > 0.f ? 1.f : 0.f;
  } else if constexpr (ACT == kActGeluErf) {
    return 0.5f * (1.f + erff(x * 0.70710678f)) + x * 0.3989422804f * __expf(-0.5f * x * x);
  } else {
    return 1.f;
  }
}

template <typename T>
struct Vec8 {
  T v[8];
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&out)[8]) {
  Vec8<T> raw;
  *reinterpret_cast<uint4*>(raw.v) = __ldg(reinterpret_cast<const uint4*>(p));
#pragma unroll
  for (int i = 0; i < 8; ++i) out[i] = to_float(raw.v[i]);
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&in)[8]) {
  Vec8<T> raw;
#pragma unroll
  for (int i = 0; i < 8; ++i) raw.v[i] = from_float<T>(in[i]);
  *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(raw.v);
}

template <typename T>
__device__ __forceinline__ float round_to(float v) {
  return to_float(from_float<T>(v));
}

// Fused epilogue on one row x 32 consecutive accumulator columns, specialised at
// compile time on the epilogue kind and the activation.  `off` is the element
// offset of the first column in the output; `cols` (a multiple of 8) is how many of
// the 32 columns exist.
template <typename T, int EPI, int ACT>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&raw)[32], int64_t off, int cols,
                                               const GemmParams& p) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (v * 8 >= cols) break;
    const int64_t o = off + v * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = __uint_as_float(raw[v * 8 + i]);
    T* c = static_cast<T*>(p.c) + o;
    if constexpr (EPI == kEpiNone) {
      store8<T>(c, acc);
    } else if constexpr (EPI == kEpiAct) {
      float o2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o2[i] = act_fwd<ACT>(round_to<T>(acc[i]));
      store8<T>(c, acc);
      if (p.out2) store8<T>(static_cast<T*>(p.out2) + o, o2);
    } else if constexpr (EPI == kEpiDAct) {
      float a1[8], o1[8], o2[8];
      load8<T>(static_cast<const T*>(p.aux1) + o, a1);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o1[i] = acc[i] * act_bwd<ACT>(a1[i]);
        o2[i] = act_fwd<ACT>(a1[i]);
      }
      store8<T>(c, o1);
      if (p.out2) store8<T>(static_cast<T*>(p.out2) + o, o2);
    } else if constexpr (EPI == kEpiGlu) {
      float a1[8], o2[8];
      load8<T>(static_cast<const T*>(p.aux1) + o, a1);
#pragma unroll
      for (int i = 0; i < 8; ++i) o2[i] = act_fwd<ACT>(a1[i]) * round_to<T>(acc[i]);
      store8<T>(c, acc);
      if (p.out2) store8<T>(static_cast<T*>(p.out2) + o, o2);
    } else if constexpr (EPI == kEpiDGlu) {
      float a1[8], a2[8], o1[8], o2[8], o3[8];
      load8<T>(static_cast<const T*>(p.aux1) + o, a1);
      load8<T>(static_cast<const T*>(p.aux2) + o, a2);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float g = act_fwd<ACT>(a1[i]);
        o1[i] = acc[i] * a2[i] * act_bwd<ACT>(a1[i]);
        o2[i] = acc[i] * g;
        o3[i] = g * a2[i];
      }
      store8<T>(c, o1);
      if (p.out2) store8<T>(static_cast<T*>(p.out2) + o, o2);
      if (p.out3) store8<T>(static_cast<T*>(p.out3) + o, o3);
    } else {  // kEpiAdd
      float a1[8], o1[8];
      load8<T>(static_cast<const T*>(p.aux1) + o, a1);
#pragma unroll
      for (int i = 0; i < 8; ++i) o1[i] = acc[i] + a1[i];
      store8<T>(c, o1);
    }
  }
}

template <typename T, int EPI>
__device__ __forceinline__ void epilogue_by_act(const uint32_t (&raw)[32], int64_t off, int cols,
                                                const GemmParams& p) {
  switch (p.act) {
    case kActGeluTanh: epilogue_chunk<T, EPI, kActGeluTanh>(raw, off, cols, p); break;
    case kActSilu: epilogue_chunk<T, EPI, kActSilu>(raw, off, cols, p); break;
    case kActRelu: epilogue_chunk<T, EPI, kActRelu>(raw, off, cols, p); break;
    case kActGeluErf: epilogue_chunk<T, EPI, kActGeluErf>(raw, off, cols, p); break;
    default: epilogue_chunk<T, EPI, kActIdentity>(raw, off, cols, p); break;
  }
}

// One dispatch per 32-column chunk; everything inside is straight-line code.
template <typename T>
__device__ __forceinline__ void epilogue_dispatch(const uint32_t (&raw)[32], int64_t off, int cols,
                                                  const GemmParams& p) {
  switch (p.epilogue) {
    case kEpiNone: epilogue_chunk<T, kEpiNone, kActIdentity>(raw, off, cols, p); break;
    case kEpiAdd: epilogue_chunk<T, kEpiAdd, kActIdentity>(raw, off, cols, p); break;
    case kEpiAct: epilogue_by_act<T, kEpiAct>(raw, off, cols, p); break;
    case kEpiDAct: epilogue_by_act<T, kEpiDAct>(raw, off, cols, p); break;
    case kEpiGlu: epilogue_by_act<T, kEpiGlu>(raw, off, cols, p); break;
    case kEpiDGlu: epilogue_by_act<T, kEpiDGlu>(raw, off, cols, p); break;
    default: break;
  }
}

template <typename T, int LAYOUT, int BLOCK_N>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
  using Cfg = Config<BLOCK_N>;
  constexpr bool kAMn = LAYOUT == kTN;
  constexpr bool kBMn = LAYOUT != kNT;
  constexpr int kStages = Cfg::kStages;
  constexpr bool kIsBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kTileBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + kStages;            // [kStages]
  uint64_t* tmem_full_bar = bars + 2 * kStages;    // [2]
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;  // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int* s_row_end = reinterpret_cast<int*>(smem + Cfg::kTileBytes + 256);   // [kMaxGroups]
  int* s_mblk_end = s_row_end + kMaxGroups;                                 // [kMaxGroups]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.num_groups;

  // ---- one-time setup ---------------------------------------------------------
  for (int g = threadIdx.x; g < G; g += kThreads) s_row_end[g] = __ldg(p.bins + g);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), 4);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) tmem_alloc(smem_u32(tmem_base_slot), Cfg::kTmemCols);
  __syncthreads();
  if (LAYOUT != kTN && threadIdx.x == 0) {
    int acc = 0, prev = 0;
    for (int g = 0; g < G; ++g) {
      const int end = s_row_end[g];
      acc += (end - prev + kBlockM - 1) / kBlockM;
      s_mblk_end[g] = acc;
      prev = end;
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // ---- tile schedule (every role decodes the same sequence) ---------------------
  const int num_nb = (p.N + BLOCK_N - 1) / BLOCK_N;
  const int num_mb_tn = (p.M + kBlockM - 1) / kBlockM;
  const int total_tiles = (LAYOUT == kTN) ? G * num_mb_tn * num_nb : (G > 0 ? s_mblk_end[G - 1] : 0) * num_nb;

  auto decode = [&](int t) {
    Tile tile;
    if constexpr (LAYOUT == kTN) {
      const int per_group = num_mb_tn * num_nb;
      tile.group = t / per_group;
      const int r = t - tile.group * per_group;
      const int mb_i = r / num_nb;
      tile.n0 = (r - mb_i * num_nb) * BLOCK_N;
      tile.row0 = mb_i * kBlockM;
      tile.rows_valid = min(kBlockM, p.M - tile.row0);
      tile.k_begin = tile.group ? s_row_end[tile.group - 1] : 0;
      tile.k_len = s_row_end[tile.group] - tile.k_begin;
    } else {
      const int mblk = t / num_nb;
      tile.n0 = (t - mblk * num_nb) * BLOCK_N;
      int lo = 0, hi = G - 1;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_mblk_end[mid] <= mblk) lo = mid + 1; else hi = mid;
      }
      tile.group = lo;
      const int row_start = lo ? s_row_end[lo - 1] : 0;
      const int local = mblk - (lo ? s_mblk_end[lo - 1] : 0);
      tile.row0 = row_start + local * kBlockM;
      tile.rows_valid = min(kBlockM, s_row_end[lo] - tile.row0);
      tile.k_begin = 0;
      tile.k_len = p.K;
    }
    return tile;
  };

  if (warp == 0) {
    // ======================= TMA producer =======================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int arrived_group = -1;
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile tile = decode(t);
        const int num_kb = (tile.k_len + kBlockK - 1) / kBlockK;
        if (LAYOUT != kTN && p.wait_flags != nullptr && tile.group != arrived_group) {
          // Rows of this group are stored by peer GPUs; each source releases one flag
          // per group when its last row has landed.
          for (int s = 0; s < p.wait_count && ok; ++s) {
            const int* flag = p.wait_flags + s * p.wait_stride + tile.group;
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (ld_acquire_sys_s32(flag) < p.wait_seq) {
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
          fence_proxy_async_all();   // the acquire above must precede the TMA (async proxy) reads
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, kErrProducer, kWaitLimitNs);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[stage]);
          mbar_arrive_expect_tx(bar, kABytes + Cfg::kBBytes);
          const uint32_t a_dst = smem_u32(smem_a + stage * kABytes);
          const uint32_t b_dst = smem_u32(smem_b + stage * Cfg::kBBytes);
          if constexpr (LAYOUT == kNT) {
            tma_load_2d(a_dst, &tmap_a, bar, kb * kBlockK, tile.row0);
            tma_load_2d(b_dst, &tmap_b, bar, kb * kBlockK, tile.group * p.N + tile.n0);
          } else if constexpr (LAYOUT == kNN) {
            tma_load_2d(a_dst, &tmap_a, bar, kb * kBlockK, tile.row0);
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)
              tma_load_2d(b_dst + j * kBoxBytes, &tmap_b, bar, tile.n0 + 64 * j, tile.group * p.K + kb * kBlockK);
          } else {
            const int krow = tile.k_begin + kb * kBlockK;
#pragma unroll
            for (int j = 0; j < kBlockM / 64; ++j)
              tma_load_2d(a_dst + j * kBoxBytes, &tmap_a, bar, tile.row0 + 64 * j, krow);
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)
              tma_load_2d(b_dst + j * kBoxBytes, &tmap_b, bar, tile.n0 + 64 * j, krow);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ======================= MMA issuer ==========================================
    constexpr uint32_t idesc = instr_desc_f16(kIsBf16, kAMn, kBMn, kBlockM, BLOCK_N);
    int stage = 0;
    uint32_t phase = 0;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Tile tile = decode(t);
      const int num_kb = (tile.k_len + kBlockK - 1) / kBlockK;
      ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_stage]), acc_phase ^ 1u, abort_flag, p.status, kErrMmaTmem,
                     kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok);   // the whole warp leaves together
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, kErrMmaFull, kWaitLimitNs);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* a_tile = smem_a + stage * kABytes;
        uint8_t* b_tile = smem_b + stage * Cfg::kBBytes;
        if constexpr (LAYOUT == kTN) {
          // Rows of the last K block that belong to the next group (or lie past the
          // tensor) must not contribute: zero them in both operands.
          const int valid = tile.k_len - kb * kBlockK;
          if (valid < kBlockK) {
            const int tail_chunks = (kBlockK - valid) * 8;   // 16-byte chunks per box
            for (int box = 0; box < kBlockM / 64 + BLOCK_N / 64; ++box) {
              uint8_t* base = (box < kBlockM / 64) ? a_tile + box * kBoxBytes
                                                   : b_tile + (box - kBlockM / 64) * kBoxBytes;
              uint4* rows = reinterpret_cast<uint4*>(base + valid * 128);
              for (int i = lane; i < tail_chunks; i += 32) rows[i] = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
        }
        tcgen05_fence_after();
        if (lane == 0) {
          const uint32_t a_base = smem_u32(a_tile);
          const uint32_t b_base = smem_u32(b_tile);
#pragma unroll
          for (int k = 0; k < kBlockK / kUmmaK; ++k) {
            const uint64_t a_desc = kAMn ? smem_desc_sw128(a_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                         : smem_desc_sw128(a_base + k * (kUmmaK * 2), 16, 1024);
            const uint64_t b_desc = kBMn ? smem_desc_sw128(b_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                         : smem_desc_sw128(b_base + k * (kUmmaK * 2), 16, 1024);
            umma_f16(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&empty_bar[stage]));   // stage is reusable once these MMAs retire
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      if (lane == 0) {
        if (num_kb > 0) umma_commit(smem_u32(&tmem_full_bar[acc_stage]));
        else mbar_arrive(smem_u32(&tmem_full_bar[acc_stage]));   // empty group: nothing to wait for
      }
      __syncwarp();
      if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
    }
  } else {
    // ======================= epilogue warps ======================================
    const int quarter = warp & 3;               // TMEM lane quarter this warp may read
    const int row_in_tile = quarter * 32 + lane;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Tile tile = decode(t);
      const bool has_k = tile.k_len > 0;
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc_stage]), acc_phase, abort_flag, p.status, kErrEpilogue,
                     kWaitLimitNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const bool row_ok = row_in_tile < tile.rows_valid;
      int64_t row_off;
      if constexpr (LAYOUT == kTN) row_off = (int64_t(tile.group) * p.M + tile.row0 + row_in_tile) * p.N;
      else row_off = int64_t(tile.row0 + row_in_tile) * p.N;
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc_stage * BLOCK_N;
#pragma unroll 1
      for (int c0 = 0; c0 < BLOCK_N; c0 += 32) {
        if (tile.n0 + c0 >= p.N) break;          // uniform across the warp
        uint32_t raw[32];
        if (has_k) {
          tmem_ld_32x32(taddr + c0, raw);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = 0u;
        }
        if (row_ok) {
          const int col = tile.n0 + c0;
          epilogue_dispatch<T>(raw, row_off + col, min(32, p.N - col), p);
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc_stage]));
      if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
    }
    // Rows past the last group belong to nobody: defined as zero (NT / NN only).
    if (LAYOUT != kTN && p.zero_tail) {
      const int last = G > 0 ? s_row_end[G - 1] : 0;
      const int64_t begin = int64_t(last) * p.N, end = int64_t(p.rows_total) * p.N;
      const int64_t tid = int64_t(blockIdx.x) * 128 + (threadIdx.x - 64);
      const int64_t stride = int64_t(gridDim.x) * 128;
      for (int64_t i = begin + tid * 8; i < end; i += stride * 8) {
        const uint4 z = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(static_cast<T*>(p.c) + i) = z;
        if (p.out2) *reinterpret_cast<uint4*>(static_cast<T*>(p.out2) + i) = z;
        if (p.out3) *reinterpret_cast<uint4*>(static_cast<T*>(p.out3) + i) = z;
      }
    }
  }

  // ---- teardown -----------------------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    if (*abort_flag != 0) {
      // Give loads and MMAs that were already in flight time to land before the
      // tensor memory and the shared memory are released.
      const uint64_t t0 = globaltimer_ns();
      while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
    }
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


template <typename T, int LAYOUT, int BLOCK_N>
cudaError_t launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                       cudaStream_t stream) {
  using Cfg = Config<BLOCK_N>;
  auto kernel = grouped_gemm_kernel<T, LAYOUT, BLOCK_N>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaError_t rc = cudaGetDevice(&dev);
  if (rc != cudaSuccess) return rc;
  if (!configured[dev & 63]) {
    rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (rc != cudaSuccess) return rc;
    configured[dev & 63] = true;
  }
  kernel<<<grid, kThreads, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

// One explicit instantiation unit per (dtype, layout): see grouped_gemm_inst_*.cu.
template <typename T, int LAYOUT>
cudaError_t launch_layout(int block_n, const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, int grid,
                          cudaStream_t stream);

#define MB_GEMM_INSTANTIATE(T, LAYOUT)                                                                       \
  template <>                                                                                                \
  cudaError_t launch_layout<T, LAYOUT>(int block_n, const CUtensorMap& ta, const CUtensorMap& tb,            \
                                       const GemmParams& p, int grid, cudaStream_t stream) {                 \
    if (block_n == 256) return launch_one<T, LAYOUT, 256>(ta, tb, p, grid, stream);                          \
    if (block_n == 128) return launch_one<T, LAYOUT, 128>(ta, tb, p, grid, stream);                          \
    return launch_one<T, LAYOUT, 64>(ta, tb, p, grid, stream);                                               \
  }

}  // namespace gemm
}  // namespace mb

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
// Structure per CTA (320 threads, one CTA per SM, tiles taken round-robin):
//   warp 8      TMA producer: cp.async.bulk.tensor tile loads into a ring of
//               128-byte-swizzled shared-memory stages, completion on mbarriers;
//   warp 9      allocates tensor memory and issues tcgen05.mma (one elected lane);
//               tcgen05.commit releases ring stages and publishes accumulators;
//   warps 0-7   epilogue (two warps per TMEM lane quarter, interleaving 32-column chunks): tcgen05.ld the fp32 accumulator (two TMEM stages, so the
//               next tile's MMAs overlap this tile's epilogue), apply the fused
//               epilogue (activation, activation backward, GLU, GLU backward, add)
//               and move rows through a swizzled shared-memory staging buffer so
//               global loads / stores are coalesced, masked to the group.
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
constexpr int kBandN = 8;                    // column tiles per band of the tile walk (NT / NN)
constexpr int kSmallGroups = 224;            // groups whose tables fit beside two sets of staging buffers
constexpr int kMaxScatterSegments = 512;     // experts per rank x world of the fused combine
constexpr int kEpilogueWarps = 8;            // two warps per TMEM lane quarter
constexpr int kProducerWarp = kEpilogueWarps;       // warp 8: TMA loads
constexpr int kMmaWarp = kEpilogueWarps + 1;        // warp 9: TMEM allocation and tcgen05.mma
constexpr int kThreads = (kEpilogueWarps + 2) * 32;
constexpr int kABytes = kBlockM * kBlockK * 2;
constexpr int kBoxBytes = 64 * kBlockK * 2;   // one 64-wide MN-major box
constexpr uint64_t kWaitLimitNs = 2000000000ull;


// Status codes written on an abandoned wait.
constexpr int kErrProducer = 1, kErrMmaFull = 2, kErrMmaTmem = 3, kErrEpilogue = 4, kErrPeerRows = 18;

// Sequence number of a launch: the host's value plus the device counter, when there is one (a
// launch recorded in a CUDA graph takes a fresh number at every replay).
__device__ __forceinline__ int seq_with_base(int seq, const int* base) {
  return base != nullptr ? seq + __ldg(base) : seq;
}

template <int BLOCK_N>
struct Config {
  static constexpr int kStages = BLOCK_N == 256 ? 4 : (BLOCK_N == 128 ? 6 : 8);
  static constexpr int kBBytes = BLOCK_N * kBlockK * 2;
  static constexpr int kTmemCols = 2 * BLOCK_N;
  static constexpr int kTileBytes = kStages * (kABytes + kBBytes);
  // ring + barriers + tmem base + abort flag + group tables, plus slack for 1024-byte alignment
  static constexpr int kStagingBytes = kEpilogueWarps * 2048;   // one 32-row x 64-byte buffer per epilogue warp
  static constexpr int kScatterBytes = (2 * kMaxScatterSegments + 128) * 4;   // segment tables of the fused combine
  // ring, two sets of staging buffers (the second doubles as the large-table area), barriers, small tables, alignment slack
  static constexpr int kSmemBytes = kTileBytes + 2 * kStagingBytes + 256 + 2 * kSmallGroups * 4 + 1024;
  static_assert(2 * kMaxGroups * 4 + kScatterBytes <= kStagingBytes, "large tables must fit the alternate staging area");
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

// erf by the Abramowitz-Stegun 7.1.26 rational form (absolute error < 1.5e-7): a handful of
// FMAs and one exponential, no local memory (the library routine has a slow path that does).
__device__ __forceinline__ float erf_fast(float x) {
  const float ax = fabsf(x);
  const float t = __fdividef(1.f, 1.f + 0.3275911f * ax);
  const float poly = t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f + t * (-1.453152027f + t * 1.061405429f))));
  const float y = 1.f - poly * __expf(-ax * ax);
  return copysignf(y, x);
}

template <int ACT>
__device__ __forceinline__ float act_fwd(float x) {
  if constexpr (ACT == kActGeluTanh) return 0.5f * x * (1.f + tanh_fast(0.7978845608f * (x + 0.044715f * x * x * x)));
  else if constexpr (ACT == kActSilu) return x / (1.f + __expf(-x));
  else if constexpr (ACT == kActRelu) return fmaxf(x, 0.f);
  else if constexpr (ACT == kActGeluErf) return 0.5f * x * (1.f + erf_fast(x * 0.70710678f));
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
    return 0.5f * (1.f + erf_fast(x * 0.70710678f)) + x * 0.3989422804f * __expf(-0.5f * x * x);
  } else {
    return 1.f;
  }
}

// ---- packed fp32 pairs (sm_100 f32x2 arithmetic: two elements per instruction) ------------
__device__ __forceinline__ float2 splat2(float v) { return make_float2(v, v); }

// tanh-GELU of a pair: 0.5 z (1 + tanh(z (k + k c z^2))).
__device__ __forceinline__ float2 gelu_tanh_fwd2(float2 z) {
  const float2 u = __fmul2_rn(z, z);
  const float2 inner = __fmul2_rn(z, __ffma2_rn(u, splat2(0.0356774081f), splat2(0.7978845608f)));
  const float2 t = make_float2(tanh_fast(inner.x), tanh_fast(inner.y));
  const float2 hz = __fmul2_rn(z, splat2(0.5f));
  return __ffma2_rn(hz, t, hz);
}

// tanh-GELU and its derivative times `acc` for a pair, from one tanh per element.
__device__ __forceinline__ void gelu_tanh_dact2(float2 acc, float2 z, float2& dz, float2& h) {
  const float2 u = __fmul2_rn(z, z);
  const float2 inner = __fmul2_rn(z, __ffma2_rn(u, splat2(0.0356774081f), splat2(0.7978845608f)));
  const float2 t = make_float2(tanh_fast(inner.x), tanh_fast(inner.y));
  const float2 hz = __fmul2_rn(z, splat2(0.5f));
  h = __ffma2_rn(hz, t, hz);
  const float2 neg_g = __ffma2_rn(u, splat2(-0.1070322243f), splat2(-0.7978845608f));   // -d(inner)/dz
  const float2 s = __ffma2_rn(t, t, splat2(-1.f));                                         // t^2 - 1
  const float2 q = __ffma2_rn(t, splat2(0.5f), splat2(0.5f));
  const float2 d = __ffma2_rn(__fmul2_rn(hz, s), neg_g, q);
  dz = __fmul2_rn(acc, d);
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

// ---- epilogue staging ------------------------------------------------------------
// tcgen05.ld hands every thread one accumulator ROW (32 consecutive columns), so a
// direct global store would touch 32 different cache lines per instruction.  Each
// epilogue warp therefore owns a 32-row x 64-byte shared-memory buffer: rows are
// written (or read) by their owner thread, and moved to / from global memory by the
// whole warp as 8 rows x 64 contiguous bytes per instruction.  16-byte chunks are
// XOR-swizzled with bits of the row so both access patterns are bank-conflict free.
__device__ __forceinline__ uint32_t stage_offset(int row, int chunk) {
  return uint32_t(row) * 64u + uint32_t((chunk ^ ((row >> 1) & 3)) * 16);
}

// Global [32 rows x 32 columns] (16-bit) -> staging, coalesced.  Rows >= rows_ok and
// 8-column groups >= cols are skipped (their staging content is never used).
template <typename T>
__device__ __forceinline__ void stage_load(uint8_t* stage, const T* base, int64_t row_stride, int rows_ok,
                                           int cols, int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), q = lane & 3;
    if (r < rows_ok && q * 8 < cols)
      *reinterpret_cast<uint4*>(stage + stage_offset(r, q)) =
          __ldg(reinterpret_cast<const uint4*>(base + int64_t(r) * row_stride + q * 8));
  }
}

// Requests the cache lines of a chunk's auxiliary operand ahead of time (no registers
// are held): the later `stage_load` of the same addresses then hits in cache.
template <typename T>
__device__ __forceinline__ void aux_prefetch(const T* base, int64_t row_stride, int rows_ok, int cols, int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), q = lane & 3;
    if (r < rows_ok && q * 8 < cols)
      asm volatile("prefetch.global.L1 [%0];" ::"l"(base + int64_t(r) * row_stride + q * 8));
  }
}

template <typename T>
__device__ __forceinline__ void stage_store(const uint8_t* stage, T* base, int64_t row_stride, int rows_ok,
                                            int cols, int lane) {
#ifdef MB_GEMM_NO_STORE
  if (rows_ok >= 0) return;
#endif
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), q = lane & 3;
    if (r < rows_ok && q * 8 < cols)
      *reinterpret_cast<uint4*>(base + int64_t(r) * row_stride + q * 8) =
          *reinterpret_cast<const uint4*>(stage + stage_offset(r, q));
  }
}

// Row targets of the fused combine: where the four rows this lane stores (rows i * 8 + lane / 4
// of the warp's 32-row quarter) live in the peers' return buffers; null = row does not exist.
template <typename T>
struct ScatterRows {
  T* row[4];
};

template <typename T>
__device__ __forceinline__ void stage_store_rows(const uint8_t* stage, const ScatterRows<T>& rows, int col, int cols,
                                                 int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 8 + (lane >> 2), q = lane & 3;
    if (rows.row[i] != nullptr && q * 8 < cols)
      *reinterpret_cast<uint4*>(rows.row[i] + col + q * 8) = *reinterpret_cast<const uint4*>(stage + stage_offset(r, q));
  }
}

// TMA store target of one warp for the current tile: `on` when the tensor maps exist and all 32
// rows of the warp's quarter are real rows of the group; `row` = first of them in the [rows, N] view.
struct TmaOut {
  bool on;
  int row;
};

// A warp's staging buffer(s).  With two buffers (`other` = byte distance to the alternate one,
// 0 = single buffer) consecutive TMA stores alternate, so the second output of a chunk does not
// wait for the TMA unit to finish reading the first.
struct Staging {
  uint8_t* buf;
  int other;
};

// Before a staging buffer is rewritten the bulk store that last read it must be done reading.
// With alternating buffers that is the store before the latest one.
__device__ __forceinline__ void stage_acquire(const Staging& st, int lane) {
  if (lane == 0) {
    if (st.other != 0) bulk_wait_read_but_one();
    else bulk_wait_read_all();
  }
  __syncwarp();
}

// After a TMA store was issued from the current buffer: continue in the other one.
__device__ __forceinline__ void stage_flip(Staging& st) {
  st.buf += st.other;
  st.other = -st.other;
}

// This thread's row of the staging buffer, kept packed (16 registers for 32 values).
struct PackedRow {
  uint4 q[4];
};
__device__ __forceinline__ void stage_read_row(const uint8_t* stage, int lane, PackedRow& out) {
#pragma unroll
  for (int v = 0; v < 4; ++v) out.q[v] = *reinterpret_cast<const uint4*>(stage + stage_offset(lane, v));
}
// Two 16-bit values <-> one 32-bit word, without taking the address of a register.
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  uint32_t out;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
  return out;
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  uint32_t out;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(out) : "f"(hi), "f"(lo));
  return out;
}
template <typename T>
__device__ __forceinline__ float unpack_half(uint32_t word, int hi);
template <>
__device__ __forceinline__ float unpack_half<__nv_bfloat16>(uint32_t word, int hi) {
  return __uint_as_float(hi ? (word & 0xffff0000u) : (word << 16));
}
template <>
__device__ __forceinline__ float unpack_half<__half>(uint32_t word, int hi) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(hi ? (word >> 16) : (word & 0xffffu))));
}
__device__ __forceinline__ uint32_t word_of(const uint4& q, int w) {
  return w == 0 ? q.x : (w == 1 ? q.y : (w == 2 ? q.z : q.w));
}
template <typename T>
__device__ __forceinline__ float packed_at(const PackedRow& row, int i) {
  return unpack_half<T>(word_of(row.q[i >> 3], (i & 7) >> 1), i & 1);
}

// Elements (2w, 2w + 1) of a packed row as a pair.
template <typename T>
__device__ __forceinline__ float2 packed_pair(const PackedRow& row, int w) {
  const uint32_t word = word_of(row.q[w >> 2], w & 3);
  return make_float2(unpack_half<T>(word, 0), unpack_half<T>(word, 1));
}

// Element `i` of output number WHICH (0 = c, 1 = out2, 2 = out3) of the fused epilogue.
template <typename T, int EPI, int ACT, int WHICH>
__device__ __forceinline__ float epilogue_value(const uint32_t (&raw)[32], const PackedRow& a1, const PackedRow& a2,
                                                int i) {
  const float acc = __uint_as_float(raw[i]);
  if constexpr (EPI == kEpiNone) {
    return acc;
  } else if constexpr (EPI == kEpiAct) {
    return WHICH == 0 ? acc : act_fwd<ACT>(round_to<T>(acc));
  } else if constexpr (EPI == kEpiDAct) {
    const float z = packed_at<T>(a1, i);
    return WHICH == 0 ? acc * act_bwd<ACT>(z) : act_fwd<ACT>(z);
  } else if constexpr (EPI == kEpiGlu) {
    return WHICH == 0 ? acc : act_fwd<ACT>(packed_at<T>(a1, i)) * round_to<T>(acc);
  } else if constexpr (EPI == kEpiDGlu) {
    const float z1 = packed_at<T>(a1, i), z2 = packed_at<T>(a2, i);
    if constexpr (WHICH == 0) return acc * z2 * act_bwd<ACT>(z1);
    else if constexpr (WHICH == 1) return acc * act_fwd<ACT>(z1);
    else return act_fwd<ACT>(z1) * z2;
  } else {  // kEpiAdd
    return acc + packed_at<T>(a1, i);
  }
}

// Activation backward: both outputs of element `i` from one evaluation of the activation's
// transcendental (dz = acc * act'(z), h = act(z)).
template <typename T, int ACT>
__device__ __forceinline__ void dact_values(float acc, float z, float& dz, float& h) {
  if constexpr (ACT == kActGeluTanh) {
    const float u = z * z;
    const float t = tanh_fast(z * (0.7978845608f + 0.0356774081f * u));
    const float hz = 0.5f * z;
    h = fmaf(hz, t, hz);
    const float g = fmaf(u, 0.1070322243f, 0.7978845608f);          // d(inner)/dz
    const float d = fmaf(hz * fmaf(-t, t, 1.f), g, fmaf(t, 0.5f, 0.5f));
    dz = acc * d;
  } else if constexpr (ACT == kActSilu) {
    const float sg = 1.f / (1.f + __expf(-z));
    h = z * sg;
    dz = acc * (sg * (1.f + z * (1.f - sg)));
  } else {
    h = act_fwd<ACT>(z);
    dz = acc * act_bwd<ACT>(z);
  }
}

// One pass over the chunk for the activation-backward epilogue: dz goes to the staging buffer as
// it is produced, h waits packed in registers until the buffer is free again.
template <typename T, int ACT, bool WANT_H>
__device__ __forceinline__ void epilogue_emit_dact(const uint32_t (&raw)[32], const PackedRow& a1, Staging& stage,
                                                   T* out, T* out2, int64_t row_stride, int rows_ok, int cols,
                                                   int lane, int col, const CUtensorMap* maps, TmaOut tma) {
  uint4 hw[4];
  if (maps != nullptr) stage_acquire(stage, lane);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    float dz[8], h[8];
    if constexpr (ACT == kActGeluTanh) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 dz2, h2;
        gelu_tanh_dact2(make_float2(__uint_as_float(raw[v * 8 + 2 * j]), __uint_as_float(raw[v * 8 + 2 * j + 1])),
                        packed_pair<T>(a1, v * 4 + j), dz2, h2);
        dz[2 * j] = dz2.x; dz[2 * j + 1] = dz2.y;
        h[2 * j] = h2.x; h[2 * j + 1] = h2.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        dact_values<T, ACT>(__uint_as_float(raw[v * 8 + j]), packed_at<T>(a1, v * 8 + j), dz[j], h[j]);
    }
    uint4 w;
    w.x = pack2<T>(dz[0], dz[1]); w.y = pack2<T>(dz[2], dz[3]); w.z = pack2<T>(dz[4], dz[5]); w.w = pack2<T>(dz[6], dz[7]);
    if constexpr (WANT_H) {
      hw[v].x = pack2<T>(h[0], h[1]); hw[v].y = pack2<T>(h[2], h[3]);
      hw[v].z = pack2<T>(h[4], h[5]); hw[v].w = pack2<T>(h[6], h[7]);
    }
    *reinterpret_cast<uint4*>(stage.buf + stage_offset(lane, v)) = w;
  }
  if (tma.on) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(maps, smem_u32(stage.buf), col, tma.row);
      bulk_commit_group();
    }
    stage_flip(stage);
  } else {
    __syncwarp();
    stage_store<T>(stage.buf, out, row_stride, rows_ok, cols, lane);
    __syncwarp();
  }
  if constexpr (!WANT_H) return;
  if (maps != nullptr) stage_acquire(stage, lane);
#pragma unroll
  for (int v = 0; v < 4; ++v) *reinterpret_cast<uint4*>(stage.buf + stage_offset(lane, v)) = hw[v];
  if (tma.on) {
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(maps + 1, smem_u32(stage.buf), col, tma.row);
      bulk_commit_group();
    }
    stage_flip(stage);
  } else {
    __syncwarp();
    stage_store<T>(stage.buf, out2, row_stride, rows_ok, cols, lane);
    __syncwarp();
  }
}

// Elements (i, i + 1) of output WHICH, packed to 16 bits.
template <typename T, int EPI, int ACT, int WHICH>
__device__ __forceinline__ uint32_t epilogue_pair(const uint32_t (&raw)[32], const PackedRow& a1, const PackedRow& a2,
                                                  int i) {
  if constexpr (EPI == kEpiAct && ACT == kActGeluTanh && WHICH == 1) {
    // act(round(acc)): round through the 16-bit type first, as the unfused sequence does.
    const uint32_t rounded = pack2<T>(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
    const float2 h = gelu_tanh_fwd2(make_float2(unpack_half<T>(rounded, 0), unpack_half<T>(rounded, 1)));
    return pack2<T>(h.x, h.y);
  } else {
    return pack2<T>(epilogue_value<T, EPI, ACT, WHICH>(raw, a1, a2, i),
                    epilogue_value<T, EPI, ACT, WHICH>(raw, a1, a2, i + 1));
  }
}

// Computes one output of the chunk, packs it eight columns at a time into this thread's
// staging row and stores the chunk coalesced.  Only the accumulator row and the packed
// auxiliary rows stay in registers.
template <typename T, int EPI, int ACT, int WHICH>
__device__ __forceinline__ void epilogue_emit(const uint32_t (&raw)[32], const PackedRow& a1, const PackedRow& a2,
                                              Staging& stage, T* out, int64_t row_stride, int rows_ok, int cols,
                                              int lane, const ScatterRows<T>* scatter = nullptr, int col = 0,
                                              const CUtensorMap* tmap = nullptr, TmaOut tma = TmaOut{false, 0}) {
  if (tmap != nullptr) stage_acquire(stage, lane);
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    uint4 w;
    w.x = epilogue_pair<T, EPI, ACT, WHICH>(raw, a1, a2, v * 8 + 0);
    w.y = epilogue_pair<T, EPI, ACT, WHICH>(raw, a1, a2, v * 8 + 2);
    w.z = epilogue_pair<T, EPI, ACT, WHICH>(raw, a1, a2, v * 8 + 4);
    w.w = epilogue_pair<T, EPI, ACT, WHICH>(raw, a1, a2, v * 8 + 6);
    *reinterpret_cast<uint4*>(stage.buf + stage_offset(lane, v)) = w;
  }
  if (tma.on) {
    // The staging layout is the 64-byte swizzle of a 32 x 32 box: one thread hands the chunk to
    // the TMA unit, which clips columns past N.
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(tmap, smem_u32(stage.buf), col, tma.row);
      bulk_commit_group();
    }
    stage_flip(stage);
    return;
  }
  __syncwarp();
  if (scatter != nullptr) stage_store_rows<T>(stage.buf, *scatter, col, cols, lane);
  else stage_store<T>(stage.buf, out, row_stride, rows_ok, cols, lane);
  __syncwarp();
}

// Fused epilogue of one warp on a 32-row x 32-column chunk, specialised at compile time
// on the epilogue kind and the activation.  `base_off` is the element offset of the
// chunk's first row / first column in the output, `rows_ok` / `cols` its valid extent.
template <typename T, int EPI, int ACT>
__device__ __forceinline__ void epilogue_chunk(const uint32_t (&raw)[32], const PackedRow& a1,
                                               const PackedRow& a2, Staging& stage, int64_t base_off,
                                               int64_t row_stride, int rows_ok, int cols, int lane,
                                               const GemmParams& p, const ScatterRows<T>* scatter, int col,
                                               TmaOut tma) {
  const CUtensorMap* maps = p.store_tma ? p.out_map : nullptr;
  if constexpr (EPI == kEpiDAct) {
    // Without the second output (the activation was kept by the forward pass) its arithmetic
    // is compiled out.
    if (p.out2)
      epilogue_emit_dact<T, ACT, true>(raw, a1, stage, static_cast<T*>(p.c) + base_off,
                                       static_cast<T*>(p.out2) + base_off, row_stride, rows_ok, cols, lane, col,
                                       maps, tma);
    else
      epilogue_emit_dact<T, ACT, false>(raw, a1, stage, static_cast<T*>(p.c) + base_off, nullptr, row_stride,
                                        rows_ok, cols, lane, col, maps, tma);
    return;
  }
  epilogue_emit<T, EPI, ACT, 0>(raw, a1, a2, stage, static_cast<T*>(p.c) + base_off, row_stride, rows_ok, cols,
                                lane, scatter, col, maps, tma);
  if constexpr (EPI == kEpiAct || EPI == kEpiDAct || EPI == kEpiGlu || EPI == kEpiDGlu) {
    if (p.out2)
      epilogue_emit<T, EPI, ACT, 1>(raw, a1, a2, stage, static_cast<T*>(p.out2) + base_off, row_stride, rows_ok,
                                    cols, lane, nullptr, col, maps ? maps + 1 : nullptr, tma);
  }
  if constexpr (EPI == kEpiDGlu) {
    if (p.out3)
      epilogue_emit<T, EPI, ACT, 2>(raw, a1, a2, stage, static_cast<T*>(p.out3) + base_off, row_stride, rows_ok,
                                    cols, lane, nullptr, col, maps ? maps + 2 : nullptr, tma);
  }
}

template <typename T, int EPI>
__device__ __forceinline__ void epilogue_by_act(const uint32_t (&raw)[32], const PackedRow& a1,
                                                const PackedRow& a2, Staging& stage, int64_t base_off,
                                                int64_t row_stride, int rows_ok, int cols, int lane,
                                                const GemmParams& p, const ScatterRows<T>* scatter, int col,
                                                TmaOut tma) {
  switch (p.act) {
    case kActGeluTanh: epilogue_chunk<T, EPI, kActGeluTanh>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kActSilu: epilogue_chunk<T, EPI, kActSilu>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kActRelu: epilogue_chunk<T, EPI, kActRelu>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kActGeluErf: epilogue_chunk<T, EPI, kActGeluErf>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    default: epilogue_chunk<T, EPI, kActIdentity>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
  }
}

// One dispatch per 32-column chunk (uniform across the warp); straight-line code inside.
template <typename T>
__device__ __forceinline__ void epilogue_dispatch(const uint32_t (&raw)[32], const PackedRow& a1,
                                                  const PackedRow& a2, Staging& stage, int64_t base_off,
                                                  int64_t row_stride, int rows_ok, int cols, int lane,
                                                  const GemmParams& p, const ScatterRows<T>* scatter = nullptr,
                                                  int col = 0, TmaOut tma = TmaOut{false, 0}) {
  switch (p.epilogue) {
    case kEpiNone: epilogue_chunk<T, kEpiNone, kActIdentity>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kEpiAdd: epilogue_chunk<T, kEpiAdd, kActIdentity>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kEpiAct: epilogue_by_act<T, kEpiAct>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kEpiDAct: epilogue_by_act<T, kEpiDAct>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kEpiGlu: epilogue_by_act<T, kEpiGlu>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    case kEpiDGlu: epilogue_by_act<T, kEpiDGlu>(raw, a1, a2, stage, base_off, row_stride, rows_ok, cols, lane, p, scatter, col, tma); break;
    default: break;
  }
}

// Role timers: a build with -DMB_GEMM_TIMING accumulates, per CTA, the cycles each role spends
// waiting on its barriers (slots: 0 MMA waits for operands, 1 MMA waits for a free accumulator,
// 2 MMA role total, 3 producer waits for a free stage, 4 epilogue warp 0 waits for an accumulator,
// 5 epilogue warp 0 total, 6 its tcgen05.ld time, 7 its convert / stage / store time, 8 its per-tile
// preamble, 9 its whole chunk loop, 10 its accumulator release, 11 its auxiliary-operand loads).
#ifdef MB_GEMM_TIMING
#define MB_T_DECL(name) long long name = 0
#define MB_T_BEGIN(var) const long long var = clock64()
#define MB_T_END(var, acc) acc += clock64() - var
#define MB_T_WRITE(slot, acc) if (p.timing) p.timing[blockIdx.x * 16 + (slot)] = acc
#else
#define MB_T_DECL(name)
#define MB_T_BEGIN(var)
#define MB_T_END(var, acc)
#define MB_T_WRITE(slot, acc)
#endif

template <typename T, int LAYOUT, int BLOCK_N>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ GemmParams p) {
  using Cfg = Config<BLOCK_N>;
  constexpr bool kAMn = LAYOUT == kTN;
  constexpr bool kBMn = LAYOUT != kNT;
  constexpr int kStages = Cfg::kStages;
  constexpr bool kIsBf16 = std::is_same<T, __nv_bfloat16>::value;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kABytes;
  // Staging buffers directly after the operand ring: 1024-byte aligned, as the swizzled TMA stores need.
  uint8_t* staging = smem + Cfg::kTileBytes;
  uint8_t* staging1 = staging + Cfg::kStagingBytes;   // alternate buffers, or the large tables
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging1 + Cfg::kStagingBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + kStages;            // [kStages]
  uint64_t* tmem_full_bar = bars + 2 * kStages;    // [2]
  uint64_t* tmem_empty_bar = bars + 2 * kStages + 2;  // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  uint64_t* scatter_bar = bars + 2 * kStages + 6;  // [2] fused combine: "all warps stored this tile"
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  volatile int* dead_flag = reinterpret_cast<volatile int*>(bars + 2 * kStages + 8);
  const bool scatter_on = LAYOUT == kNN && p.scatter_base != nullptr;
  // Up to kSmallGroups groups the tables fit behind the barriers; more groups, or the segment tables
  // of the fused combine, take the place of the alternate staging buffers.
  const bool big_tables = p.num_groups > kSmallGroups || scatter_on;
  int* tables = big_tables ? reinterpret_cast<int*>(staging1)
                           : reinterpret_cast<int*>(staging1 + Cfg::kStagingBytes + 256);
  int* s_row_end = tables;                                                   // [groups]
  int* s_mblk_end = tables + (big_tables ? kMaxGroups : kSmallGroups);       // [groups]
  // Fused combine (NN layout only): per (local expert, source rank) segment tables.
  int* s_seg_end = s_mblk_end + kMaxGroups;
  int* s_remote_start = s_seg_end + kMaxScatterSegments;
  int* s_per_source = s_remote_start + kMaxScatterSegments;                 // [world] rows returned to each source

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int G = p.num_groups;

  // ---- one-time setup ---------------------------------------------------------
  for (int g = threadIdx.x; g < G; g += kThreads) s_row_end[g] = __ldg(p.bins + g);
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    // A launch that takes part in the expert-parallel exchange does nothing once a failure has
    // been recorded on this device: its row counts and peer offsets may then be meaningless.
    *dead_flag = (p.wait_flags != nullptr || scatter_on) && *reinterpret_cast<volatile int*>(p.status) != 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_u32(&tmem_full_bar[s]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[s]), kEpilogueWarps);
      mbar_init(smem_u32(&scatter_bar[s]), kEpilogueWarps);
    }
    fence_barrier_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == kMmaWarp) tmem_alloc(smem_u32(tmem_base_slot), Cfg::kTmemCols);
  __syncthreads();
  const bool dead = *dead_flag != 0;
  if (threadIdx.x == 0) {
    // Group ends are forced to be non-decreasing and inside the operand, so no tile can start or
    // end outside a or c whatever `bins` holds.
    int acc = 0, prev = 0;
    for (int g = 0; g < G; ++g) {
      const int end = min(max(s_row_end[g], prev), p.rows_total);
      s_row_end[g] = end;
      if (LAYOUT != kTN) {
        acc += (end - prev + kBlockM - 1) / kBlockM;
        s_mblk_end[g] = acc;
      }
      prev = end;
    }
  }
  if (scatter_on && !dead) {
    const int W = p.scatter_world, E = p.scatter_experts, epr = G;
    if (threadIdx.x == 0) {
      int acc = 0;
      for (int j = 0; j < epr; ++j)
        for (int s2 = 0; s2 < W; ++s2) {
          acc += __ldg(p.scatter_counts + s2 * E + p.scatter_rank * epr + j);
          s_seg_end[j * W + s2] = acc;
        }
    }
    for (int idx = threadIdx.x; idx < epr * W; idx += kThreads) {
      const int j = idx / W, s2 = idx - j * W;
      const int e = p.scatter_rank * epr + j;
      int acc = 0;
      for (int e2 = 0; e2 < e; ++e2) acc += __ldg(p.scatter_raw_counts + s2 * E + e2);
      s_remote_start[idx] = acc;       // first sorted position of (source s2, expert e) at the source
    }
    for (int s2 = threadIdx.x; s2 < W; s2 += kThreads) {
      int acc = 0;
      for (int j = 0; j < epr; ++j) acc += __ldg(p.scatter_counts + s2 * E + p.scatter_rank * epr + j);
      s_per_source[s2] = acc;
      // A source that gets nothing back still needs its flag.
      if (blockIdx.x == 0 && acc == 0)
        st_release_sys_s32(reinterpret_cast<int*>(p.scatter_flag_base[s2] + p.scatter_flag_off) + p.scatter_rank,
                           seq_with_base(p.scatter_seq, p.seq_base));
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  // ---- tile schedule (every role decodes the same sequence) ---------------------
  // With two B operands a tile covers half as many output columns (each operand fills half of the
  // accumulator).
  const bool dual = LAYOUT == kNT && BLOCK_N == 256 && p.dual_b != 0;
  const bool concat = LAYOUT == kNN && p.k_concat != 0;
  const int tile_n = dual ? BLOCK_N / 2 : BLOCK_N;
  const int num_nb = (p.N + tile_n - 1) / tile_n;
  const int num_mb_tn = (p.M + kBlockM - 1) / kBlockM;
  const int total_tiles =
      dead ? 0 : ((LAYOUT == kTN) ? G * num_mb_tn * num_nb : (G > 0 ? s_mblk_end[G - 1] : 0) * num_nb);

  auto decode = [&](int t) {
    Tile tile;
    if constexpr (LAYOUT == kTN) {
      const int per_group = num_mb_tn * num_nb;
      tile.group = t / per_group;
      const int r = t - tile.group * per_group;
      const int mb_i = r / num_nb;
      tile.n0 = (r - mb_i * num_nb) * tile_n;
      tile.row0 = mb_i * kBlockM;
      tile.rows_valid = min(kBlockM, p.M - tile.row0);
      tile.k_begin = tile.group ? s_row_end[tile.group - 1] : 0;
      tile.k_len = s_row_end[tile.group] - tile.k_begin;
    } else {
      // Tiles of a group are walked in bands of kBandN column tiles, row blocks fastest inside a
      // band: the CTAs that run at the same time then share a few B tiles and a few dozen A tiles
      // (tens of MB) instead of sweeping the group's whole weight matrix once per row block, which
      // for large experts (hundreds of MB of weights) would stream them from HBM again and again.
      int lo = 0, hi = G - 1;
      const int key = t / num_nb;              // group boundaries are multiples of num_nb tiles
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_mblk_end[mid] <= key) lo = mid + 1; else hi = mid;
      }
      tile.group = lo;
      const int mblk_begin = lo ? s_mblk_end[lo - 1] : 0;
      const int mblks = s_mblk_end[lo] - mblk_begin;
      const int u = t - mblk_begin * num_nb;   // index of the tile inside its group
      const int band_n = p.band_n > 0 ? p.band_n : kBandN;
      const int band = u / (mblks * band_n);
      const int r = u - band * mblks * band_n;
      const int width = min(band_n, num_nb - band * band_n);
      const int local = r / width;
      tile.n0 = (band * band_n + (r - local * width)) * tile_n;
      const int row_start = lo ? s_row_end[lo - 1] : 0;
      tile.row0 = row_start + local * kBlockM;
      tile.rows_valid = min(kBlockM, s_row_end[lo] - tile.row0);
      tile.k_begin = 0;
      tile.k_len = p.K;
    }
    return tile;
  };

  if (warp == kProducerWarp) {
    // ======================= TMA producer =======================================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int arrived_group = -1;
      MB_T_DECL(t_empty);
      for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
        const Tile tile = decode(t);
        const int num_kb1 = (tile.k_len + kBlockK - 1) / kBlockK;
        const int num_kb = concat ? 2 * num_kb1 : num_kb1;
        if (LAYOUT != kTN && p.wait_flags != nullptr && tile.group != arrived_group) {
          // Rows of this group are stored by peer GPUs; each source releases one flag
          // per group when its last row has landed.
          for (int s = 0; s < p.wait_count && ok; ++s) {
            const int* flag = p.wait_flags + s * p.wait_stride + tile.group;
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            const int wait_seq = seq_with_base(p.wait_seq, p.seq_base);
            while (ld_acquire_sys_s32(flag) < wait_seq) {
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
          MB_T_BEGIN(w0);
          ok = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_flag, p.status, kErrProducer, kWaitLimitNs);
          MB_T_END(w0, t_empty);
          if (!ok) break;
          const uint32_t bar = smem_u32(&full_bar[stage]);
          if (p.diag & 1) {   // diagnostic: no operand loads, the MMAs chew on whatever the stage holds
            mbar_arrive(bar);
            if (++stage == kStages) { stage = 0; phase ^= 1u; }
            continue;
          }
          mbar_arrive_expect_tx(bar, kABytes + Cfg::kBBytes);
          const uint32_t a_dst = smem_u32(smem_a + stage * kABytes);
          const uint32_t b_dst = smem_u32(smem_b + stage * Cfg::kBBytes);
          if constexpr (LAYOUT == kNT) {
            tma_load_2d(a_dst, &tmap_a, bar, kb * kBlockK, tile.row0);
            if (dual) {   // 128 rows of each weight matrix, one after the other in the stage
              tma_load_2d(b_dst, &tmap_b, bar, kb * kBlockK, tile.group * p.N + tile.n0);
              tma_load_2d(b_dst + Cfg::kBBytes / 2, &p.b2_map, bar, kb * kBlockK, tile.group * p.N + tile.n0);
            } else {
              tma_load_2d(b_dst, &tmap_b, bar, kb * kBlockK, tile.group * p.N + tile.n0);
            }
          } else if constexpr (LAYOUT == kNN) {
            // Second operand pair of a concatenated contraction: same coordinates, other tensors.
            const bool second = concat && kb >= num_kb1;
            const int kk = second ? kb - num_kb1 : kb;
            const CUtensorMap* ma = second ? &p.a2_map : &tmap_a;
            const CUtensorMap* mbp = second ? &p.b2_map : &tmap_b;
            tma_load_2d(a_dst, ma, bar, kk * kBlockK, tile.row0);
#pragma unroll
            for (int j = 0; j < BLOCK_N / 64; ++j)
              tma_load_2d(b_dst + j * kBoxBytes, mbp, bar, tile.n0 + 64 * j, tile.group * p.K + kk * kBlockK);
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
      MB_T_WRITE(3, t_empty);
    }
  } else if (warp == kMmaWarp) {
    // ======================= MMA issuer ==========================================
    constexpr uint32_t idesc = instr_desc_f16(kIsBf16, kAMn, kBMn, kBlockM, BLOCK_N);
    int stage = 0;
    uint32_t phase = 0;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    MB_T_DECL(t_full);
    MB_T_DECL(t_tmem);
    MB_T_DECL(t_total);
    MB_T_BEGIN(role0);
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      const Tile tile = decode(t);
      const int num_kb = ((tile.k_len + kBlockK - 1) / kBlockK) * (concat ? 2 : 1);
      MB_T_BEGIN(w1);
      ok = mbar_wait(smem_u32(&tmem_empty_bar[acc_stage]), acc_phase ^ 1u, abort_flag, p.status, kErrMmaTmem,
                     kWaitLimitNs);
      MB_T_END(w1, t_tmem);
      ok = __all_sync(0xffffffffu, ok);   // the whole warp leaves together
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t d_tmem = tmem_base + acc_stage * BLOCK_N;
      for (int kb = 0; kb < num_kb; ++kb) {
        MB_T_BEGIN(w0);
        ok = mbar_wait(smem_u32(&full_bar[stage]), phase, abort_flag, p.status, kErrMmaFull, kWaitLimitNs);
        MB_T_END(w0, t_full);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        uint8_t* a_tile = smem_a + stage * kABytes;
        uint8_t* b_tile = smem_b + stage * Cfg::kBBytes;
        if constexpr (LAYOUT == kTN) {
          // Rows of the last K block that belong to the next group (or lie past the tensor)
          // must not contribute.  Zero rows in ONE operand cancel finite rows of the other, and
          // the rows after any group but the last are the next group's data, so only the A side
          // is cleared there; after the last group that has rows the memory may never have been
          // written, and both sides are cleared.
          const int valid = tile.k_len - kb * kBlockK;
          if (valid < kBlockK) {
            const int tail_chunks = (kBlockK - valid) * 8;   // 16-byte chunks per box
            const bool at_end = tile.k_begin + tile.k_len >= s_row_end[G - 1];   // no later group has rows
            const int boxes = at_end ? kBlockM / 64 + BLOCK_N / 64 : kBlockM / 64;
            for (int box = 0; box < boxes; ++box) {
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
          if (!(p.diag & 2)) {   // (diagnostic bit 2: operand loads and epilogue without any MMA)
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              const uint64_t a_desc = kAMn ? smem_desc_sw128(a_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                           : smem_desc_sw128(a_base + k * (kUmmaK * 2), 16, 1024);
              const uint64_t b_desc = kBMn ? smem_desc_sw128(b_base + k * (kUmmaK * 128), kBoxBytes, 1024)
                                           : smem_desc_sw128(b_base + k * (kUmmaK * 2), 16, 1024);
              umma_f16(d_tmem, a_desc, b_desc, idesc, (kb | k) != 0 ? 1u : 0u);
            }
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
    MB_T_END(role0, t_total);
    if (lane == 0) {
      MB_T_WRITE(0, t_full);
      MB_T_WRITE(1, t_tmem);
      MB_T_WRITE(2, t_total);
    }
  } else if (warp < kEpilogueWarps) {
    // ======================= epilogue warps ======================================
    const int quarter = warp & 3;               // TMEM lane quarter this warp may read
    const int half = warp >> 2;                 // which of the two warps of that quarter
    Staging stage{staging + warp * 2048, (p.store_tma != 0 && !big_tables) ? Cfg::kStagingBytes : 0};
    constexpr int kChunks = BLOCK_N / 32;
    int acc_stage = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    float2 sq_sum = make_float2(0.f, 0.f);      // sum of squares of what this thread stored (p.sqnorm)
    MB_T_DECL(t_acc);
    MB_T_DECL(t_epi);
    MB_T_DECL(t_ld);
    MB_T_DECL(t_out);
    MB_T_DECL(t_pre);
    MB_T_DECL(t_loop);
    MB_T_DECL(t_post);
    MB_T_DECL(t_aux);
    MB_T_BEGIN(role0);
    for (int t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
      MB_T_BEGIN(wpre);
      const Tile tile = decode(t);
      const bool has_k = tile.k_len > 0;
      // Rows of this warp's quarter that exist in the tile, and its first row's offset.
      const int rows_ok = max(0, min(32, tile.rows_valid - quarter * 32));
      int64_t row_off;
      if constexpr (LAYOUT == kTN) row_off = (int64_t(tile.group) * p.M + tile.row0 + quarter * 32) * p.N;
      else row_off = int64_t(tile.row0 + quarter * 32) * p.N;
      TmaOut tma;
      tma.on = p.store_tma != 0 && rows_ok == 32;
      if constexpr (LAYOUT == kTN) tma.row = tile.group * p.M + tile.row0 + quarter * 32;
      else tma.row = tile.row0 + quarter * 32;
      ScatterRows<T> targets;
      if (scatter_on) {
        const int W = p.scatter_world;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int r = quarter * 32 + i * 8 + (lane >> 2);
          targets.row[i] = nullptr;
          if (r < tile.rows_valid) {
            const int grow = tile.row0 + r;
            int s2 = 0;
            while (s2 < W - 1 && s_seg_end[tile.group * W + s2] <= grow) ++s2;
            const int seg = tile.group * W + s2;
            const int seg_begin = seg ? s_seg_end[seg - 1] : 0;
            const int64_t remote_row = s_remote_start[seg] + (grow - seg_begin);
            if (remote_row >= 0 && remote_row < p.scatter_rows)   // never store outside the source's buffer
              targets.row[i] = reinterpret_cast<T*>(p.scatter_base[s2] + p.scatter_off) + remote_row * p.N;
          }
        }
      }
      // Auxiliary operands (pre-activations) are fetched one chunk ahead, the first one
      // before the accumulator is even ready.
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
      MB_T_END(wpre, t_pre);
      MB_T_BEGIN(w0);
      ok = mbar_wait(smem_u32(&tmem_full_bar[acc_stage]), acc_phase, abort_flag, p.status, kErrEpilogue,
                     kWaitLimitNs);
      MB_T_END(w0, t_acc);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quarter * 32) << 16) + acc_stage * BLOCK_N;
      // The two warps of a quarter interleave 32-column chunks.
      MB_T_BEGIN(wloop);
#pragma unroll 1
      const int chunks = dual ? kChunks / 2 : kChunks;
      for (int ci = half; ci < chunks; ci += 2) {
        const int c0 = ci * 32;
        const int col = tile.n0 + c0;
        if (col >= p.N) break;                   // uniform across the warp
        if (dual) {
          // a b^T first: written out (out3) and kept packed; then a b2^T with the GLU product.
          uint32_t raw[32];
          PackedRow z1, unused;
          tmem_ld_32x32(taddr + c0, raw);
          tmem_ld_wait();
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            z1.q[v].x = pack2<T>(__uint_as_float(raw[v * 8 + 0]), __uint_as_float(raw[v * 8 + 1]));
            z1.q[v].y = pack2<T>(__uint_as_float(raw[v * 8 + 2]), __uint_as_float(raw[v * 8 + 3]));
            z1.q[v].z = pack2<T>(__uint_as_float(raw[v * 8 + 4]), __uint_as_float(raw[v * 8 + 5]));
            z1.q[v].w = pack2<T>(__uint_as_float(raw[v * 8 + 6]), __uint_as_float(raw[v * 8 + 7]));
          }
          if (rows_ok > 0) {
            const int cols = min(32, p.N - col);
            const CUtensorMap* maps = p.store_tma ? p.out_map : nullptr;
            epilogue_emit<T, kEpiNone, kActIdentity, 0>(raw, z1, unused, stage, static_cast<T*>(p.out3) + row_off + col,
                                                        p.N, rows_ok, cols, lane, nullptr, col,
                                                        maps ? maps + 2 : nullptr, tma);
            tmem_ld_32x32(taddr + BLOCK_N / 2 + c0, raw);
            tmem_ld_wait();
            epilogue_by_act<T, kEpiGlu>(raw, z1, unused, stage, row_off + col, p.N, rows_ok, cols, lane, p, nullptr, col,
                                        tma);
          }
          continue;
        }
        // Ask for the next chunk's auxiliary operands, then bring this chunk's through the
        // staging buffer (coalesced read, each thread picks up its own row).
        if (ci + 2 < kChunks && rows_ok > 0 && col + 64 < p.N) {
          const int ncol = col + 64;
          if (need1) aux_prefetch<T>(static_cast<const T*>(p.aux1) + row_off + ncol, p.N, rows_ok,
                                     min(32, p.N - ncol), lane);
          if (need2) aux_prefetch<T>(static_cast<const T*>(p.aux2) + row_off + ncol, p.N, rows_ok,
                                     min(32, p.N - ncol), lane);
        }
        PackedRow a1, a2;
        MB_T_BEGIN(waux);
        if (rows_ok > 0) {
          const int cols = min(32, p.N - col);
          if (need1) {
            if (p.store_tma) stage_acquire(stage, lane);
            stage_load<T>(stage.buf, static_cast<const T*>(p.aux1) + row_off + col, p.N, rows_ok, cols, lane);
            __syncwarp();
            stage_read_row(stage.buf, lane, a1);
            __syncwarp();
          }
          if (need2) {
            stage_load<T>(stage.buf, static_cast<const T*>(p.aux2) + row_off + col, p.N, rows_ok, cols, lane);
            __syncwarp();
            stage_read_row(stage.buf, lane, a2);
            __syncwarp();
          }
        }
        MB_T_END(waux, t_aux);
        uint32_t raw[32];
        MB_T_BEGIN(w1);
        if (has_k) {
          tmem_ld_32x32(taddr + c0, raw);
          tmem_ld_wait();
          if (p.alpha != 1.f) {
#pragma unroll
            for (int i = 0; i < 32; ++i) raw[i] = __float_as_uint(__uint_as_float(raw[i]) * p.alpha);
          }
          if constexpr (LAYOUT == kTN) {
            // Weight gradients: their squared norm (the clip needs it) is taken here, from the
            // fp32 values on their way out, instead of by a pass that reads the gradients back.
            if (p.sqnorm != nullptr && lane < rows_ok) {
              const int cols = p.N - col;       // even: rows are a multiple of 16 bytes
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 v = make_float2(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
                if (i < cols) sq_sum = __ffma2_rn(v, v, sq_sum);
              }
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) raw[i] = 0u;
        }
        MB_T_END(w1, t_ld);
        MB_T_BEGIN(w2);
        if (rows_ok > 0)
          epilogue_dispatch<T>(raw, a1, a2, stage, row_off + col, p.N, rows_ok, min(32, p.N - col), lane, p,
                               scatter_on ? &targets : nullptr, col, tma);
        MB_T_END(w2, t_out);
      }
      MB_T_END(wloop, t_loop);
      MB_T_BEGIN(wpost);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[acc_stage]));
      MB_T_END(wpost, t_post);
      const int tile_stage = acc_stage;
      const uint32_t tile_phase = acc_phase;
      if (++acc_stage == 2) { acc_stage = 0; acc_phase ^= 1u; }
      if (scatter_on) {
        // Once every epilogue warp has issued its stores of this tile, one thread orders them
        // system-wide and credits the sources whose rows the tile covered.  (Two barriers,
        // alternating with the accumulator stage: a warp is never more than one tile ahead.)
        if (lane == 0) mbar_arrive(smem_u32(&scatter_bar[tile_stage]));
        if (warp == 0) {
          bool stored = true;
          if (lane == 0)
            stored = mbar_wait(smem_u32(&scatter_bar[tile_stage]), tile_phase, abort_flag, p.status, kErrEpilogue,
                               kWaitLimitNs);
          stored = __shfl_sync(0xffffffffu, stored ? 1 : 0, 0) != 0;   // the warp leaves together
          if (!stored) ok = false;
        }
        if (threadIdx.x == 0 && ok && tile.rows_valid > 0) {
          __threadfence_system();
          const int W = p.scatter_world;
          const int lo_row = tile.row0, hi_row = tile.row0 + tile.rows_valid;
          for (int s2 = 0; s2 < W; ++s2) {
            const int seg = tile.group * W + s2;
            const int seg_begin = seg ? s_seg_end[seg - 1] : 0;
            const int cnt = min(hi_row, s_seg_end[seg]) - max(lo_row, seg_begin);
            if (cnt <= 0) continue;
            // A row is complete once all column blocks of its tile row have been stored.
            if (atomicAdd(p.scatter_done + s2, cnt) + cnt == s_per_source[s2] * num_nb) {
              __threadfence_system();
              st_release_sys_s32(reinterpret_cast<int*>(p.scatter_flag_base[s2] + p.scatter_flag_off) +
                                     p.scatter_rank, seq_with_base(p.scatter_seq, p.seq_base));
            }
          }
        }
      }
    }
    if (p.store_tma && lane == 0) bulk_wait_all();   // bulk stores complete before the CTA retires
    if constexpr (LAYOUT == kTN) {
      if (p.sqnorm != nullptr) {                     // one atomic per warp and launch
        float total = sq_sum.x + sq_sum.y;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
        if (lane == 0 && ok) atomicAdd(p.sqnorm, total);
      }
    }
    MB_T_END(role0, t_epi);
    if (threadIdx.x == 0) {
      MB_T_WRITE(4, t_acc);
      MB_T_WRITE(5, t_epi);
      MB_T_WRITE(6, t_ld);
      MB_T_WRITE(7, t_out);
      MB_T_WRITE(8, t_pre);
      MB_T_WRITE(9, t_loop);
      MB_T_WRITE(10, t_post);
      MB_T_WRITE(11, t_aux);
    }
    // Rows past the last group belong to nobody: defined as zero (NT / NN only).
    if (LAYOUT != kTN && p.zero_tail && !dead) {
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

  // ---- teardown -----------------------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
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

// Fused fp32 batched-matmul kernel for sm_100a: C[b] = A[b] @ B[b] with the epilogue
// chosen at compile time (store / masked store / row-wise min+argmin / row-wise top-k).
//
// Replaces the reference's SIMT tile kernels (kernels/bmm.cu:185, kernels/mbmm.cu:209,
// kernels/minbmm.cu:348, kernels/topkbmm.cu:500 and their layout variants) with one
// persistent, warp-specialised kernel:
//
//   warp 0      TMA producer: raw fp32 operand tiles -> shared-memory ring
//   warps 2-5   splitters: lo = x - tf32(x), written beside the raw tile (the raw tile
//               itself serves as the hi plane because the tensor core ignores the low
//               13 mantissa bits of a tf32 operand)
//   warp 1      MMA issuer: per 8-wide k-step three tcgen05.mma kind::tf32
//               (lo*hi and hi*lo into a "small" TMEM accumulator, hi*hi into a "big"
//               one; TMEM accumulation truncates, and keeping the small terms apart
//               keeps their bits)
//   warps 6-9   epilogue: tcgen05.ld both accumulators, add them, then store / mask /
//               reduce. One thread owns one output row, so per-row min and top-k state
//               never crosses threads.
//
// Work is cut into units (batch, 128-row block, run of column tiles); CTA i processes
// units i, i + gridDim.x, ... All four roles walk the same unit list.
#pragma once
#include <cuda.h>
#include <cfloat>
#include "sm100_primitives.cuh"

namespace fbmm {

constexpr int kTileM = 128;
constexpr int kKBlock = 32;  // fp32 elements per k-block: one 128-byte swizzle row
constexpr int kNumThreads = 320;
constexpr int kSplitThreads = 128;
constexpr int kEpiThreads = 128;
constexpr int kTmemCols = 512;

enum EpilogueKind { kEpiStore = 0, kEpiMask = 1, kEpiMin = 2, kEpiTopk = 3 };

// Device status word (bit 0: a bounded wait ran out).
__device__ unsigned int g_fbmm_status[4];

struct GemmShape {
  int L, M, N, K;
  int a_mn;  // A stored [l][k][m] (m contiguous) instead of [l][m][k]
  int b_mn;  // B stored [l][k][n] (n contiguous) instead of [l][n][k]
  int m_blocks;         // ceil(M / 128)
  int n_tiles;          // ceil(N / TILE_N)
  int n_chunks;         // column chunks per row block
  int tiles_per_chunk;  // column tiles per chunk
  long long num_units;  // L * m_blocks * n_chunks
};

struct EpiArgs {
  // store / mask
  float* C;
  long long ldc, stride_c;
  const unsigned char* block_mask;    // [L or 1][ceil(M/128)][ceil(N/128)]
  const unsigned char* thread_mask;   // [L or 1][ceil(M/8)][ceil(N/8)]
  const unsigned char* element_mask;  // [L or 1][M][N]
  long long bm_stride, tm_stride, em_stride;  // per-batch strides, 0 when shared
  int bm_cols, tm_cols;
  // min
  unsigned long long* keys;  // [L][M] packed (ordered value << 32 | column)
  // top-k
  float* topk_values;         // [L][M][k] running lists, descending
  long long* topk_indices;    // [L][M][k]
  int k;
  long long index_offset;     // added to every column index written (column shards)
  long long topk_chunk_rows;  // rows between the lists of consecutive column chunks (0: one chunk)
};

template <int TILE_N>
struct StageLayout {
  static constexpr uint32_t kABytes = kTileM * kKBlock * 4;
  static constexpr uint32_t kBBytes = TILE_N * kKBlock * 4;
  static constexpr uint32_t kAHi = 0;
  static constexpr uint32_t kALo = kABytes;
  static constexpr uint32_t kBHi = 2 * kABytes;
  static constexpr uint32_t kBLo = 2 * kABytes + kBBytes;
  static constexpr uint32_t kBytes = 2 * kABytes + 2 * kBBytes;
  static constexpr uint32_t kTxBytes = kABytes + kBBytes;
};

// Order-preserving map fp32 -> uint32 (smaller float <=> smaller key).
__device__ __forceinline__ uint32_t float_to_ordered(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float split_lo(float x) {
  const float hi = tf32_hi(x);
  // inf/nan have no low part: keep the product finite-arithmetic only.
  return (fabsf(x) <= FLT_MAX) ? (x - hi) : 0.f;
}

// --------------------------------------------------------------------------------------
// top-k helpers: warp-wide bitonic sort of P = 32 * E (value, index) pairs, descending by
// value, ties broken by ascending index. Element i lives in lane (i % 32), slot (i / 32).
// --------------------------------------------------------------------------------------
__device__ __forceinline__ bool topk_before(float va, int ia, float vb, int ib) {
  return (va > vb) || (va == vb && ia < ib);
}

template <int E>
__device__ __forceinline__ void warp_bitonic_sort_desc(float (&v)[E], int (&ix)[E]) {
  const uint32_t lane = lane_id();
#pragma unroll
  for (int size = 2; size <= 32 * E; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      if (stride >= 32) {
        const int js = stride >> 5;
#pragma unroll
        for (int j = 0; j < E; ++j) {
          if ((j & js) == 0) {
            // descending block when bit `size` of the element index is clear; for
            // stride >= 32 only the slot part of the index can carry that bit
            const bool desc = (((j * 32) & size) == 0);
            const bool first = topk_before(v[j], ix[j], v[j | js], ix[j | js]);
            if (first != desc) {
              const float tv = v[j]; v[j] = v[j | js]; v[j | js] = tv;
              const int ti = ix[j]; ix[j] = ix[j | js]; ix[j | js] = ti;
            }
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < E; ++j) {
          const int i = j * 32 + static_cast<int>(lane);
          const bool desc = ((i & size) == 0);
          const bool lower = ((lane & stride) == 0);
          const float ov = __shfl_xor_sync(0xffffffffu, v[j], stride);
          const int oi = __shfl_xor_sync(0xffffffffu, ix[j], stride);
          // the lower position keeps the "first" element in a descending block
          const bool mine_first = topk_before(v[j], ix[j], ov, oi);
          const bool keep_mine = (lower == desc) ? mine_first : !mine_first;
          if (!keep_mine) { v[j] = ov; ix[j] = oi; }
        }
      }
    }
  }
}

// Merges, for every row of this warp flagged in `need`, the row's staged candidates
// into its running list (k entries, descending, kept in the output buffers) and returns
// the caller lane's new threshold (the k-th best) when its own row was flagged, else
// `thr` unchanged. Rows are handled one after the other by the whole warp: list and
// staged entries are spread over the lanes, sorted by the bitonic network, and the first
// k written back. `has_list` flags rows whose list has been written before; the others
// start from an empty list (-inf / -1 padding). Called by all 32 lanes.
//   lv0 / li0: list of the warp's first row; stg_v / stg_i: staging, slot-major
//   [slot][128 rows], already offset to the warp's first row.
// Plays the part of bitonic_sort_128 + bitonic_sort_256 under the row mutex in the
// reference (kernels/topkbmm.cu:98-183), without the mutex: a row has one owner.
constexpr int kTopkEmpty = 0x7fffffff;

template <int E>
__device__ __noinline__ float topk_merge_rows(uint32_t need, uint32_t has_list, int n_staged, float thr,
                                              float* lv0, long long* li0, int k, long long index_offset,
                                              const float* stg_v, const int* stg_i) {
  const int lane = static_cast<int>(lane_id());
  uint32_t m = need;
  while (m) {
    const int src = __ffs(m) - 1;
    m &= m - 1;
    const int cnt = __shfl_sync(0xffffffffu, n_staged, src);
    const bool listed = (has_list >> src) & 1u;
    float* lv = lv0 + static_cast<long long>(src) * k;
    long long* li = li0 + static_cast<long long>(src) * k;
    float v[E];
    int ix[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int i = j * 32 + lane;
      v[j] = -INFINITY;
      ix[j] = kTopkEmpty;
      if (i < k) {
        if (listed) {
          v[j] = lv[i];
          const long long gi = li[i];
          ix[j] = gi < 0 ? kTopkEmpty : static_cast<int>(gi - index_offset);
        }
      } else if (i - k < cnt) {
        v[j] = stg_v[(i - k) * kTileM + src];
        ix[j] = stg_i[(i - k) * kTileM + src];
      }
    }
    warp_bitonic_sort_desc<E>(v, ix);
    float kth = -INFINITY;
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int i = j * 32 + lane;
      if (i < k) {
        lv[i] = v[j];
        li[i] = (ix[j] == kTopkEmpty) ? -1ll : static_cast<long long>(ix[j]) + index_offset;
      }
      if (j == ((k - 1) >> 5)) kth = v[j];
    }
    kth = __shfl_sync(0xffffffffu, kth, (k - 1) & 31);
    if (lane == src) thr = kth;
  }
  return thr;
}

// --------------------------------------------------------------------------------------
// the kernel
// --------------------------------------------------------------------------------------
template <int TILE_N, int STAGES, int EPI, int TOPK_E>
struct KernelTraits {
  using Stage = StageLayout<TILE_N>;
  static constexpr int kAccStages = 2;
  static_assert(2 * kAccStages * TILE_N <= kTmemCols, "TMEM budget");
  // top-k staging: kTopkStage slots per row, slot-major [slot][row]
  static constexpr int kTopkStage = 32;
  static constexpr uint32_t kEpiSmemBytes = (EPI == kEpiTopk) ? kTopkStage * kTileM * 8u : 0u;
  static constexpr uint32_t kSmemBytes = STAGES * Stage::kBytes + kEpiSmemBytes + 1024u /*align*/ + 256u /*barriers*/;
};

template <int TILE_N, int STAGES, int EPI, int TOPK_E>
__global__ void __launch_bounds__(kNumThreads, 1)
fbmm_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmShape shape, const EpiArgs epi) {
  using Traits = KernelTraits<TILE_N, STAGES, EPI, TOPK_E>;
  using Stage = typename Traits::Stage;
  constexpr int kAccStages = Traits::kAccStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint8_t* epi_smem = smem + STAGES * Stage::kBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Traits::kEpiSmemBytes);
  uint64_t* bar_full = bars;                      // TMA landed            [STAGES]
  uint64_t* bar_split = bars + STAGES;            // lo planes written     [STAGES]
  uint64_t* bar_empty = bars + 2 * STAGES;        // MMAs done with stage  [STAGES]
  uint64_t* bar_acc_full = bars + 3 * STAGES;     // accumulators complete [kAccStages]
  uint64_t* bar_acc_empty = bar_acc_full + kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_acc_empty + kAccStages);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_split[s], kSplitThreads);
      mbar_init(&bar_empty[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&bar_acc_full[s], 1);
      mbar_init(&bar_acc_empty[s], kEpiThreads);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_sync();
  __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int kblocks = (shape.K + kKBlock - 1) / kKBlock;
  const long long units = shape.num_units;

  // Decodes unit u; returns the tile range.
  auto decode = [&](long long u, int& b, int& mb, int& t0, int& t1) {
    const int c = static_cast<int>(u % shape.n_chunks);
    const long long r = u / shape.n_chunks;
    mb = static_cast<int>(r % shape.m_blocks);
    b = static_cast<int>(r / shape.m_blocks);
    t0 = c * shape.tiles_per_chunk;
    t1 = min(shape.n_tiles, t0 + shape.tiles_per_chunk);
  };
  // Block-mask test of the mask epilogue (kernels/mbmm.cu:251-255): a zero byte means
  // the 128x128 tile is neither loaded nor multiplied.
  auto tile_live = [&](int b, int mb, int t) -> bool {
    if (EPI != kEpiMask) return true;
    return epi.block_mask[b * epi.bm_stride + static_cast<long long>(mb) * epi.bm_cols + t] != 0;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (long long u = blockIdx.x; u < units && ok; u += gridDim.x) {
        int b, mb, t0, t1;
        decode(u, b, mb, t0, t1);
        for (int t = t0; t < t1 && ok; ++t) {
          if (!tile_live(b, mb, t)) continue;
          for (int kb = 0; kb < kblocks; ++kb) {
            ok = mbar_wait(&bar_empty[stage], phase ^ 1u, abort_flag);
            if (!ok) break;
            uint8_t* sb = stage_base + stage * Stage::kBytes;
            mbar_arrive_expect_tx(&bar_full[stage], Stage::kTxBytes);
            if (!shape.a_mn) {
              tma_load_3d(sb + Stage::kAHi, &tmap_a, &bar_full[stage], kb * kKBlock, mb * kTileM, b);
            } else {
#pragma unroll
              for (int c = 0; c < kTileM / 32; ++c)
                tma_load_3d(sb + Stage::kAHi + c * 4096, &tmap_a, &bar_full[stage], mb * kTileM + c * 32,
                            kb * kKBlock, b);
            }
            if (!shape.b_mn) {
              tma_load_3d(sb + Stage::kBHi, &tmap_b, &bar_full[stage], kb * kKBlock, t * TILE_N, b);
            } else {
#pragma unroll
              for (int c = 0; c < TILE_N / 32; ++c)
                tma_load_3d(sb + Stage::kBHi + c * 4096, &tmap_b, &bar_full[stage], t * TILE_N + c * 32,
                            kb * kKBlock, b);
            }
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
        }
      }
      if (!ok) {
        // Give copies already in flight a bounded time to land before the CTA leaves.
        const long long t0c = clock64();
        while (clock64() - t0c < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_tf32(kTileM, TILE_N, shape.a_mn != 0, shape.b_mn != 0);
      const uint32_t a_lbo = shape.a_mn ? 4096u : 16u, a_sbo = shape.a_mn ? 512u : 1024u;
      const uint32_t b_lbo = shape.b_mn ? 4096u : 16u, b_sbo = shape.b_mn ? 512u : 1024u;
      const uint32_t a_kstep = shape.a_mn ? 1024u : 32u, b_kstep = shape.b_mn ? 1024u : 32u;
      const uint64_t a_type = shape.a_mn ? (1ull << 61) : (2ull << 61);
      const uint64_t b_type = shape.b_mn ? (1ull << 61) : (2ull << 61);
      auto desc = [](uint32_t addr, uint32_t lbo, uint32_t sbo, uint64_t type) -> uint64_t {
        return (make_smem_desc_sw128(addr, lbo, sbo) & ~(7ull << 61)) | type;
      };
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0;
      bool ok = true;
      for (long long u = blockIdx.x; u < units && ok; u += gridDim.x) {
        int b, mb, t0, t1;
        decode(u, b, mb, t0, t1);
        for (int t = t0; t < t1 && ok; ++t) {
          if (!tile_live(b, mb, t)) continue;
          ok = mbar_wait(&bar_acc_empty[acc_stage], acc_phase ^ 1u, abort_flag);
          if (!ok) break;
          tcgen05_fence_after_sync();
          const uint32_t acc_big = tmem_base + acc_stage * (2 * TILE_N);
          const uint32_t acc_small = acc_big + TILE_N;
          for (int kb = 0; kb < kblocks; ++kb) {
            ok = mbar_wait(&bar_split[stage], phase, abort_flag);
            if (!ok) break;
            tcgen05_fence_after_sync();
            const uint32_t sb = smem_u32(stage_base + stage * Stage::kBytes);
#pragma unroll
            for (int ks = 0; ks < kKBlock / 8; ++ks) {
              const uint64_t a_hi = desc(sb + Stage::kAHi + ks * a_kstep, a_lbo, a_sbo, a_type);
              const uint64_t a_lo = desc(sb + Stage::kALo + ks * a_kstep, a_lbo, a_sbo, a_type);
              const uint64_t b_hi = desc(sb + Stage::kBHi + ks * b_kstep, b_lbo, b_sbo, b_type);
              const uint64_t b_lo = desc(sb + Stage::kBLo + ks * b_kstep, b_lbo, b_sbo, b_type);
              const uint32_t acc = (kb | ks) != 0 ? 1u : 0u;
              umma_tf32(acc_small, a_lo, b_hi, idesc, acc);
              umma_tf32(acc_small, a_hi, b_lo, idesc, 1u);
              umma_tf32(acc_big, a_hi, b_hi, idesc, acc);
            }
            umma_commit(&bar_empty[stage]);
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          umma_commit(&bar_acc_full[acc_stage]);
          if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1u; }
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ hi/lo splitters
    const int st = static_cast<int>(threadIdx.x) - 64;
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (long long u = blockIdx.x; u < units && ok; u += gridDim.x) {
      int b, mb, t0, t1;
      decode(u, b, mb, t0, t1);
      for (int t = t0; t < t1 && ok; ++t) {
        if (!tile_live(b, mb, t)) continue;
        for (int kb = 0; kb < kblocks; ++kb) {
          ok = mbar_wait(&bar_full[stage], phase, abort_flag);
          if (!ok) break;
          uint8_t* sb = stage_base + stage * Stage::kBytes;
          const float4* a_hi = reinterpret_cast<const float4*>(sb + Stage::kAHi);
          float4* a_lo = reinterpret_cast<float4*>(sb + Stage::kALo);
#pragma unroll 4
          for (int i = st; i < static_cast<int>(Stage::kABytes / 16); i += kSplitThreads) {
            const float4 x = a_hi[i];
            a_lo[i] = make_float4(split_lo(x.x), split_lo(x.y), split_lo(x.z), split_lo(x.w));
          }
          const float4* b_hi = reinterpret_cast<const float4*>(sb + Stage::kBHi);
          float4* b_lo = reinterpret_cast<float4*>(sb + Stage::kBLo);
#pragma unroll 4
          for (int i = st; i < static_cast<int>(Stage::kBBytes / 16); i += kSplitThreads) {
            const float4 x = b_hi[i];
            b_lo[i] = make_float4(split_lo(x.x), split_lo(x.y), split_lo(x.z), split_lo(x.w));
          }
          fence_proxy_async_smem();
          mbar_arrive(&bar_split[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
    const int row_in_tile = static_cast<int>(quarter * 32u + lane);
    const uint32_t lane_base = (quarter * 32u) << 16;
    uint32_t acc_stage = 0, acc_phase = 0;
    bool ok = true;

    // top-k staging (slot-major): values then indices
    float* stg_v = reinterpret_cast<float*>(epi_smem);
    int* stg_i = reinterpret_cast<int*>(epi_smem + Traits::kTopkStage * kTileM * 4);

    for (long long u = blockIdx.x; u < units && ok; u += gridDim.x) {
      int b, mb, t0, t1;
      decode(u, b, mb, t0, t1);
      const int row = mb * kTileM + row_in_tile;
      const bool row_ok = row < shape.M;

      // per-unit reduction state
      float best = INFINITY;
      int best_col = t0 * TILE_N;
      float thr = -INFINITY;  // top-k: current k-th best of this row
      int n_staged = 0;
      bool has_list = false;
      // list of this warp's first row (rows of a warp are consecutive)
      const long long warp_row0 = (shape.tiles_per_chunk > 0 ? (t0 / shape.tiles_per_chunk) : 0) * epi.topk_chunk_rows +
                                  static_cast<long long>(b) * shape.M + mb * kTileM + static_cast<int>(quarter) * 32;
      float* lv0 = (EPI == kEpiTopk) ? epi.topk_values + warp_row0 * epi.k : nullptr;
      long long* li0 = (EPI == kEpiTopk) ? epi.topk_indices + warp_row0 * epi.k : nullptr;
      const float* stg_v_w = stg_v + quarter * 32;
      const int* stg_i_w = stg_i + quarter * 32;

      for (int t = t0; t < t1 && ok; ++t) {
        const int col_tile = t * TILE_N;
        if (!tile_live(b, mb, t)) {
          // masked-out tile: the product is defined as zero (mbmm.py:74 pre-zeroes C).
          if (EPI == kEpiMask && row_ok) {
            float* crow = epi.C + b * epi.stride_c + static_cast<long long>(row) * epi.ldc;
            const int c_end = min(shape.N, col_tile + TILE_N);
            const bool vec = ((epi.ldc & 3) == 0) && ((epi.stride_c & 3) == 0) &&
                             ((reinterpret_cast<uintptr_t>(epi.C) & 15) == 0);
            int c = col_tile;
            if (vec)
              for (; c + 4 <= c_end; c += 4) *reinterpret_cast<float4*>(crow + c) = make_float4(0.f, 0.f, 0.f, 0.f);
            for (; c < c_end; ++c) crow[c] = 0.f;
          }
          continue;
        }
        ok = mbar_wait(&bar_acc_full[acc_stage], acc_phase, abort_flag);
        if (!ok) break;
        tcgen05_fence_after_sync();
        const uint32_t acc_big = tmem_base + acc_stage * (2 * TILE_N) + lane_base;
        const uint32_t acc_small = acc_big + TILE_N;
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          uint32_t rb[32], rs[32];
          tmem_ld_32x32b_x32(acc_big + c * 32, rb);
          tmem_ld_32x32b_x32(acc_small + c * 32, rs);
          tmem_ld_wait();
          if (c == TILE_N / 32 - 1) {
            // both accumulators of this stage are now in registers: hand the stage back
            tcgen05_fence_before_sync();
            mbar_arrive(&bar_acc_empty[acc_stage]);
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(rb[j]) + __uint_as_float(rs[j]);
          const int col0 = col_tile + c * 32;

          if (EPI == kEpiStore || EPI == kEpiMask) {
            if (row_ok && col0 < shape.N) {
              if (EPI == kEpiMask) {
                // kernels/mbmm.cu:360-363 (8x8 tile skip) and :111-133 (element multiply)
                const unsigned char* tm = epi.thread_mask + b * epi.tm_stride +
                                          static_cast<long long>(row >> 3) * epi.tm_cols + (col0 >> 3);
                const unsigned char* em = epi.element_mask + b * epi.em_stride +
                                          static_cast<long long>(row) * shape.N + col0;
                const bool em_vec = ((reinterpret_cast<uintptr_t>(em) & 15) == 0) && (col0 + 32 <= shape.N);
                unsigned char e[32];
                if (em_vec) {
                  const uint4 e0 = *reinterpret_cast<const uint4*>(em);
                  const uint4 e1 = *reinterpret_cast<const uint4*>(em + 16);
                  const uint32_t w[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
                  for (int j = 0; j < 32; ++j) e[j] = static_cast<unsigned char>((w[j >> 2] >> ((j & 3) * 8)) & 0xffu);
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j) e[j] = (col0 + j < shape.N) ? em[j] : 0;
                }
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const bool tlive = (col0 + g * 8 < shape.N) ? (tm[g] != 0) : false;
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const int jj = g * 8 + j;
                    v[jj] = tlive ? v[jj] * static_cast<float>(e[jj]) : 0.f;
                  }
                }
              }
              float* crow = epi.C + b * epi.stride_c + static_cast<long long>(row) * epi.ldc + col0;
              const bool vec = ((reinterpret_cast<uintptr_t>(crow) & 15) == 0) && (col0 + 32 <= shape.N);
              if (vec) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  __stcs(reinterpret_cast<float4*>(crow + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < shape.N) crow[j] = v[j];
              }
            }
          } else if (EPI == kEpiMin) {
            // kernels/minbmm.cu:86-153: strict '<' in ascending column order keeps the
            // lowest column on ties; columns past N never compete.
            if (col0 + 32 <= shape.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (v[j] < best) { best = v[j]; best_col = col0 + j; }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j < shape.N && v[j] < best) { best = v[j]; best_col = col0 + j; }
            }
          } else {
            // top-k: only values that beat the row's current k-th best are staged; the
            // stage is merged into the row's list before it can overflow.
            const int valid = shape.N - col0;  // columns of this chunk that exist
#pragma unroll
            for (int j0 = 0; j0 < 32; j0 += 8) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int jj = j0 + j;
                if (row_ok && jj < valid && v[jj] > thr) {
                  stg_v[n_staged * kTileM + row_in_tile] = v[jj];
                  stg_i[n_staged * kTileM + row_in_tile] = col0 + jj;
                  ++n_staged;
                }
              }
              const bool full = n_staged > Traits::kTopkStage - 8;
              const uint32_t need = __ballot_sync(0xffffffffu, full);
              if (need) {
                const uint32_t listed = __ballot_sync(0xffffffffu, has_list);
                __syncwarp();
                thr = topk_merge_rows<TOPK_E>(need, listed, n_staged, thr, lv0, li0, epi.k, epi.index_offset,
                                              stg_v_w, stg_i_w);
                if (full) { n_staged = 0; has_list = true; }
                __syncwarp();
              }
            }
          }
        }
        if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1u; }
      }

      // ---- unit end
      if (EPI == kEpiMin) {
        if (row_ok && ok) {
          const float bz = best + 0.0f;  // -0 -> +0 so equal values share one key
          const unsigned long long key =
              (static_cast<unsigned long long>(float_to_ordered(bz)) << 32) | static_cast<uint32_t>(best_col);
          atomicMin(epi.keys + static_cast<long long>(b) * shape.M + row, key);
        }
      } else if (EPI == kEpiTopk) {
        if (ok) {
          const bool pending = row_ok && (n_staged > 0 || !has_list);
          const uint32_t need = __ballot_sync(0xffffffffu, pending);
          const uint32_t listed = __ballot_sync(0xffffffffu, has_list);
          __syncwarp();
          if (need)
            thr = topk_merge_rows<TOPK_E>(need, listed, n_staged, thr, lv0, li0, epi.k, epi.index_offset,
                                          stg_v_w, stg_i_w);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tcgen05_fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicOr(&g_fbmm_status[0], 1u);
  if (warp == 1) {
    tcgen05_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// keys -> (values, indices) for min_bmm
__global__ void fbmm_min_finalize_kernel(const unsigned long long* __restrict__ keys, float* __restrict__ values,
                                         long long* __restrict__ indices, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const unsigned long long key = keys[i];
  const uint32_t k = static_cast<uint32_t>(key >> 32);
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  values[i] = __uint_as_float(u);
  indices[i] = static_cast<long long>(static_cast<uint32_t>(key & 0xffffffffu));
}

}  // namespace fbmm

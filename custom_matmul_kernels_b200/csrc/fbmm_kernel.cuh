// Fused fp32 batched-matmul kernel for sm_100a: C[b] = A[b] @ B[b] with the epilogue
// chosen at compile time (store / masked store / masked row softmax / row-wise min+argmin /
// row-wise top-k).
//
// Replaces the reference's SIMT tile kernels (kernels/bmm.cu:185, kernels/mbmm.cu:209,
// kernels/minbmm.cu:348, kernels/topkbmm.cu:500 and their layout variants) with one
// persistent, warp-specialised kernel:
//
//   warp 0      TMA producer: raw fp32 operand tiles -> shared-memory ring
//   last warp   A loader: for K <= 128 the 128 x K block of A is loaded once per unit and
//               stays resident while the unit's column tiles stream past. It has a thread of
//               its own so that the ring keeps running across unit boundaries: the next
//               unit's B tiles are requested while the last tile of this unit is still being
//               multiplied, and each k-block of the next A is requested the moment the last
//               MMA that reads the old one has retired
//   warps 2-5   splitters: lo = x - tf32(x), written beside the raw tile (the raw tile
//               itself serves as the hi plane because the tensor core ignores the low
//               13 mantissa bits of a tf32 operand)
//   warp 1      MMA issuer: per 8-wide k-step two tcgen05.mma kind::tf32: A_hi x [B_hi | B_lo]
//               (N = 256: hi*hi lands in a "big" TMEM accumulator and hi*lo in a "small" one
//               beside it) and A_lo x B_hi (N = 128, into the small one). TMEM accumulation
//               truncates, and keeping the small terms apart keeps their bits
//   warps 6-9   epilogue: tcgen05.ld both accumulators, add them, then store / mask /
//               reduce. One thread owns one output row, so per-row min and top-k state
//               never crosses threads (the mask epilogue, which keeps no state, runs
//               warps 6-13, two per row quarter; so does the softmax epilogue, whose two
//               warps per row exchange their running maximum and sum once per unit).
//
// Work is cut into units (batch, 128-row block, run of column tiles); CTA i processes
// units i, i + gridDim.x, ... All four roles walk the same unit list.
//
// Variants (template parameters of the kernel): lo planes taken from global memory
// instead of the splitters (PRESPLIT), clusters of two CTAs on 256-row blocks with
// tcgen05.mma.cta_group::2 (PAIR; min and top-k on pre-split planes, K > 64), two resident row
// blocks of A per CTA sharing every B stage (DUAL; min on pre-split planes, K <= 64), and fp16 /
// bf16 operands multiplied as they are by kind::f16 (DT).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cfloat>
#include "sm100_primitives.cuh"

namespace fbmm {

constexpr int kTileM = 128;
constexpr int kKBlock = 32;  // fp32 elements per k-block: one 128-byte swizzle row
constexpr int kSplitThreads = 128;
constexpr int kTmemCols = 512;
constexpr long long kPaceWaitCycles = 4000000;  // longest a CTA holds back for the others (~2 ms)

enum EpilogueKind { kEpiStore = 0, kEpiMask = 1, kEpiMin = 2, kEpiTopk = 3, kEpiSoftmax = 4 };
// epilogues that take the three masks of mbmm
__host__ __device__ constexpr bool is_masked(int epi) { return epi == kEpiMask || epi == kEpiSoftmax; }
// Row softmax over the kept entries of a masked product: the unit's column tiles are swept
// twice (the row block of A stays in shared memory, B streams past again), first for the
// row maxima and sums, then for the probabilities, so the scores never reach global memory.
__host__ __device__ constexpr int sweeps(int epi) { return epi == kEpiSoftmax ? 2 : 1; }

// Epilogue warps. A warp may read only the 32 TMEM lanes (rows) 32 * (warp % 4) onwards, so
// four warps cover a tile. The mask epilogue runs two warps per row quarter, each on half of
// the tile's columns: one warp per scheduler cannot hide the latency of its own chain (TMEM
// load, shuffles, mask bytes from HBM, stores), which was what held mbmm back (c3 216 ->
// 199 us). The plain store epilogue is not what limits bmm and measured 6 % slower with
// eight warps; min and top-k keep one warp per row quarter because a row's state has one
// owner. The softmax epilogue is arithmetic-bound (32 exponentials per row and chunk in
// each sweep) and gains the most from the second warp (c3 operands: 555 -> 300 us); its two
// warps per row exchange their running (maximum, sum) once per unit.
__host__ __device__ constexpr int epilogue_warps(int epi) { return is_masked(epi) ? 8 : 4; }
// warps: 0 ring producer, 1 MMA issuer, 2-5 splitters, then the epilogue warps, then one warp
// that loads the resident A blocks
__host__ __device__ constexpr int block_threads(int epi) { return 192 + 32 * epilogue_warps(epi) + 32; }

// Device status word (bit 0: a bounded wait ran out).
__device__ unsigned int g_fbmm_status[4];

// Optional per-role wait-time counters (cycles), compiled in only for tuning builds.
#ifdef FBMM_PROFILE
__device__ long long g_fbmm_prof[24];
// timeline of CTA 0: per role a list of clock64() stamps (tile boundaries)
__device__ long long g_fbmm_trace[4][1024];
#define FBMM_TRACE_DECL int trace_n_ = 0, trace2_n_ = 0
#define FBMM_TRACE2(role) if (blockIdx.x == 0 && trace2_n_ < 1024) g_fbmm_trace[role][trace2_n_++] = clock64()
#define FBMM_TRACE(role) if (blockIdx.x == 0 && trace_n_ < 1024) g_fbmm_trace[role][trace_n_++] = clock64()
#define FBMM_TRACE_TAG(role, tag) if (blockIdx.x == 0 && threadIdx.x == 192 && trace2_n_ < 1024) g_fbmm_trace[role][trace2_n_++] = (clock64() << 3) | (tag)
#define FBMM_PROF_DECL long long prof_t0_ = 0, prof_acc_[4] = {0, 0, 0, 0}, prof_x_[4] = {0, 0, 0, 0}, prof_x0_ = 0
#ifdef FBMM_PROFILE_LIGHT
#define FBMM_PROF_XBEGIN()
#define FBMM_PROF_XEND(i)
#else
#define FBMM_PROF_XBEGIN() prof_x0_ = clock64()
#define FBMM_PROF_XEND(i) prof_x_[i] += clock64() - prof_x0_
#endif
#define FBMM_PROF_XFLUSH() if (blockIdx.x == 0) { for (int q_ = 0; q_ < 4; ++q_) g_fbmm_prof[16 + q_] = prof_x_[q_]; }
#ifdef FBMM_PROFILE_LIGHT
#define FBMM_PROF_BEGIN()
#define FBMM_PROF_END(i)
#else
#define FBMM_PROF_BEGIN() prof_t0_ = clock64()
#define FBMM_PROF_END(i) prof_acc_[i] += clock64() - prof_t0_
#endif
#define FBMM_PROF_MARK(i, c, n) long long prof_m0_ = clock64(); prof_acc_[c] += (n)
#define FBMM_PROF_MARK_END(i) prof_acc_[i] += clock64() - prof_m0_
#define FBMM_PROF_PHASE_DECL long long prof_p0_ = clock64()
#define FBMM_PROF_PHASE(i)                                                              \
  {                                                                                     \
    const long long now_ = clock64();                                                   \
    if (blockIdx.x == 0 && threadIdx.x == 192) g_fbmm_prof[20 + (i)] += now_ - prof_p0_; \
    prof_p0_ = now_;                                                                    \
  }
#define FBMM_PROF_FLUSH(base)                                                           \
  if (blockIdx.x == 0) {                                                                \
    for (int q_ = 0; q_ < 4; ++q_) g_fbmm_prof[(base) + q_] = prof_acc_[q_];            \
  }
#else
#define FBMM_TRACE_DECL
#define FBMM_TRACE(role)
#define FBMM_TRACE2(role)
#define FBMM_TRACE_TAG(role, tag)
#define FBMM_PROF_DECL
#define FBMM_PROF_XBEGIN()
#define FBMM_PROF_XEND(i)
#define FBMM_PROF_XFLUSH()
#define FBMM_PROF_BEGIN()
#define FBMM_PROF_END(i)
#define FBMM_PROF_MARK(i, c, n)
#define FBMM_PROF_MARK_END(i)
#define FBMM_PROF_FLUSH(base)
#define FBMM_PROF_PHASE_DECL
#define FBMM_PROF_PHASE(i)
#endif

struct GemmShape {
  int L, M, N, K;
  int a_mn;  // A stored [l][k][m] (m contiguous) instead of [l][m][k]
  int b_mn;  // B stored [l][k][n] (n contiguous) instead of [l][n][k]
  int a_bcast, b_bcast;  // the operand has one matrix that serves every batch (batch stride 0)
  int m_blocks;         // ceil(M / 128)
  int n_tiles;          // ceil(N / TILE_N)
  int n_chunks;         // column chunks per row block
  int tiles_per_chunk;  // column tiles per chunk
  long long num_units;  // L * m_blocks * n_chunks
  int chunk_major;      // unit order: 0 = chunks of one row block are consecutive,
                        // 1 = all row blocks of chunk 0 first, then chunk 1, ... (keeps the
                        // CTAs inside one L2-sized column range of B at a time)
  // Pacing of long sweeps (0 / null: off). A unit's column tiles are counted off in ranges of
  // `pace_tiles`; range number g of a CTA (counted over all its units) is not started before
  // every CTA has requested all tiles of its range g - 2. The CTAs then read the same
  // L2-sized part of B at about the same time instead of drifting apart over a long sweep,
  // after which each would fetch B from HBM for itself. Only a hint: a CTA that has waited
  // long enough goes on regardless. pace_counts[g] counts the CTAs done with range g (zeroed
  // by the host); needs n_chunks == 1 and one CTA per unit.
  int pace_tiles;
  int pace_slack;  // ranges a CTA may be ahead of the slowest one (>= 1)
  unsigned int* pace_counts;
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
  float softmax_scale_log2e;  // softmax epilogue: scale * log2(e), applied to the products before exp2
  int mask_tma;  // the element and thread masks of a tile come through shared memory by TMA (tensor maps
                 // tmap_em / tmap_tm are valid: n a multiple of 128, mask bases 16-byte aligned)
  // min
  unsigned long long* keys;  // [L][M] packed (ordered value << 32 | column)
  // top-k
  float* topk_values;         // [L][M][k] running lists, descending
  long long* topk_indices;    // [L][M][k]
  int k;
  long long index_offset;     // added to every column index written (column shards)
  long long topk_chunk_rows;  // rows between the lists of consecutive column chunks (0: one chunk)
  float* topk_scratch;        // running lists of the unit a CTA works on: per CTA 32 E entries x 128 rows of
                              // values, then as many int32 columns, entry-major (see topk_merge_own_rows)
  int2* topk_packed;          // when set, the lists are written here instead of topk_values / topk_indices:
                              // [L][M][k] pairs (value bits, int32 column WITHOUT index_offset; -1 = empty),
                              // the wire format of the column-sharded exchange
  // squared-l2 distance (min / top-k): squared norms of the row operand [L][M] and of the
  // column operand [L][N]; null for the inner product
  const float* row_norms;
  const float* col_norms;
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
// top-k helpers. Order of (value, index) pairs everywhere: larger value first, ties by
// ascending index. In the warp-wide routines element i of a list of 32 * E lives in lane
// (i % 32), slot (i / 32).
// --------------------------------------------------------------------------------------
// Bitwise operators on purpose: with the short-circuit forms the compiler emits branches,
// and a compare-exchange then costs four times as much.
__device__ __forceinline__ bool topk_before(float va, int ia, float vb, int ib) {
  return (va > vb) | ((va == vb) & (ia < ib));
}

// Two fp32 values rounded to nearest into one 32-bit word of fp16 (bf16 == false) or bf16.
__device__ __forceinline__ uint32_t pack_x16(float a, float b, bool bf16) {
  if (bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ uint16_t round_x16(float a, bool bf16) {
  return static_cast<uint16_t>(pack_x16(a, 0.f, bf16) & 0xffffu);
}

// Within each group of four lanes, turns "lane q holds 32 consecutive columns of its own
// row" into "lane q holds columns [8q, 8q+8) of each of the group's four rows":
// afterwards v[8i .. 8i+7] belongs to row (group base + i). A warp store of v[8i..] then
// writes eight complete 128-byte lines (four lanes per line) instead of touching 32 lines
// with one sector each, which is what the load/store unit is short of when the output is
// written at HBM speed. Two butterfly stages, 32 shuffles.
__device__ __forceinline__ void transpose_rows_in_lane_quads(float (&v)[32]) {
  const bool hi2 = (lane_id() & 2u) != 0;
  const bool hi1 = (lane_id() & 1u) != 0;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float send = hi2 ? v[j] : v[16 + j];
    const float recv = __shfl_xor_sync(0xffffffffu, send, 2);
    if (hi2) v[j] = recv; else v[16 + j] = recv;
  }
#pragma unroll
  for (int h = 0; h < 32; h += 16) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float send = hi1 ? v[h + j] : v[h + 8 + j];
      const float recv = __shfl_xor_sync(0xffffffffu, send, 1);
      if (hi1) v[h + j] = recv; else v[h + 8 + j] = recv;
    }
  }
}

constexpr int kTopkEmpty = 0x7fffffff;

// Stores the staged candidate (x, col) as one 8-byte entry at shared-memory byte address
// `addr` when `pred` is non-zero; predicated, so a warp never diverges over it.
__device__ __forceinline__ void topk_stage_if(uint32_t pred, uint32_t addr, float x, int col) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.u32 p, %0, 0;\n"
      "@p st.shared.v2.b32 [%1], {%2, %3};\n"
      "}\n"
      ::"r"(pred), "r"(addr), "r"(__float_as_uint(x)), "r"(col)
      : "memory");
}

// Sorts a bitonic sequence of 32 * E striped pairs (entry i in lane i % 32, slot i / 32)
// into descending order: the last log2(32 E) stages of the sorting network.
template <int E>
__device__ __forceinline__ void warp_bitonic_merge_desc(float (&v)[E], int (&ix)[E]) {
  const uint32_t lane = lane_id();
#pragma unroll
  for (int stride = 16 * E; stride > 0; stride >>= 1) {
    if (stride >= 32) {
      const int js = stride >> 5;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        if ((j & js) == 0 && !topk_before(v[j], ix[j], v[j | js], ix[j | js])) {
          const float tv = v[j]; v[j] = v[j | js]; v[j | js] = tv;
          const int tx = ix[j]; ix[j] = ix[j | js]; ix[j | js] = tx;
        }
      }
    } else {
      const bool lower = ((lane & stride) == 0);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float ov = __shfl_xor_sync(0xffffffffu, v[j], stride);
        const int oi = __shfl_xor_sync(0xffffffffu, ix[j], stride);
        const bool mine_first = topk_before(v[j], ix[j], ov, oi);
        if (mine_first != lower) { v[j] = ov; ix[j] = oi; }
      }
    }
  }
}

// Merges two descending striped lists of 32 * E entries each and keeps the best 32 * E in L:
// entry i of the result is the better of L[i] and G[32 E - 1 - i], which leaves the survivors
// as a bitonic sequence; log2(32 E) merge stages sort it. Order: larger value first, ties by
// lower index; empty entries (-inf, kTopkEmpty) sort last. The warp-wide counterpart of the
// reference's merge network (bitonic_sort_256, kernels/topkbmm.cu:98-183).
template <int E>
__device__ __forceinline__ void topk_merge_lists(float (&L)[E], int (&LI)[E], const float (&G)[E], const int (&GI)[E]) {
  const int partner = 31 - static_cast<int>(lane_id());
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const float bv = __shfl_sync(0xffffffffu, G[E - 1 - j], partner);
    const int bi = __shfl_sync(0xffffffffu, GI[E - 1 - j], partner);
    if (topk_before(bv, bi, L[j], LI[j])) { L[j] = bv; LI[j] = bi; }
  }
  warp_bitonic_merge_desc<E>(L, LI);
}

// Entry `pos` of a striped list, delivered to every lane.
template <int E>
__device__ __forceinline__ float topk_list_entry(const float (&L)[E], int pos) {
  float x = L[0];
#pragma unroll
  for (int j = 1; j < E; ++j)
    if ((pos >> 5) == j) x = L[j];
  return __shfl_sync(0xffffffffu, x, pos & 31);
}

// --------------------------------------------------------------------------------------
// Running top-k lists inside the fused kernel: one row per lane.
//
// An epilogue lane owns one row of the 128-row block (it reads that row's accumulator from
// tensor memory). Its running list lives in a per-CTA scratch area in global memory,
// entry-major: entry e of row r at [e * 128 + r], values and int32 columns in two arrays.
// A warp-wide access to "entry e of my row" is therefore one 128-byte line, and every lane
// can run the merge networks on its own row in registers with uniform addresses: no
// shuffles, 32 rows advance at once, nothing is shared between lanes. (A warp-wide merge of
// ONE row costs a chain of ~35 dependent shuffle stages at ~30 cycles each.) The lists go
// to the caller's [row][k] buffers once, when the unit ends. The reference keeps its lists
// in the output buffers under a per-row spin mutex (kernels/topkbmm.cu:13-47, 249-303).
// --------------------------------------------------------------------------------------

// Compare-exchange: afterwards (va, ia) is the entry that comes first.
__device__ __forceinline__ void topk_ce(float& va, int& ia, float& vb, int& ib) {
  const bool sw = topk_before(vb, ib, va, ia);
  const float tv = sw ? vb : va;
  const int ti = sw ? ib : ia;
  vb = sw ? va : vb;
  ib = sw ? ia : ib;
  va = tv;
  ia = ti;
}

// Compare-exchange with a run-time direction: (va, ia) comes first afterwards when `desc`.
__device__ __forceinline__ void topk_ce_dir(float& va, int& ia, float& vb, int& ib, bool desc) {
  const bool sw = topk_before(vb, ib, va, ia) == desc;
  const float tv = sw ? vb : va;
  const int ti = sw ? ib : ia;
  vb = sw ? va : vb;
  ib = sw ? ia : ib;
  va = tv;
  ia = ti;
}

// The merge stages with strides 4, 2, 1 on eight register pairs, all in one direction.
__device__ __forceinline__ void topk_merge8(float (&v)[8], int (&ix)[8], bool desc) {
#pragma unroll
  for (int st = 4; st > 0; st >>= 1) {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if ((e & st) == 0) topk_ce_dir(v[e], ix[e], v[e | st], ix[e | st], desc);
  }
}

// The merge stages with strides 16 to 1 on 32 register pairs (four groups of eight),
// descending: sorts a bitonic sequence of 32.
__device__ __forceinline__ void topk_merge32_desc(float (&v)[4][8], int (&ix)[4][8]) {
#pragma unroll
  for (int js = 2; js > 0; js >>= 1) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      if ((c & js) == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) topk_ce(v[c][e], ix[c][e], v[c | js][e], ix[c | js][e]);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < 4; ++c) {
#pragma unroll
    for (int st = 4; st > 0; st >>= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if ((e & st) == 0) topk_ce(v[c][e], ix[c][e], v[c][e | st], ix[c][e | st]);
    }
  }
}

__device__ __forceinline__ void topk_slots_load8(const int2* slots, int first, float (&v)[8], int (&ix)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const int2 t = slots[(first + e) * kTileM];
    v[e] = __int_as_float(t.x);
    ix[e] = t.y;
  }
}
__device__ __forceinline__ void topk_slots_store8(int2* slots, int first, const float (&v)[8], const int (&ix)[8]) {
#pragma unroll
  for (int e = 0; e < 8; ++e) slots[(first + e) * kTileM] = make_int2(__float_as_int(v[e]), ix[e]);
}

// Bitonic sorting network over the 32 staging slots of one lane (slots kTileM entries
// apart, so the lanes of a warp never meet in a bank), descending. Three trips through
// shared memory, each doing in registers every stage that stays inside what it loaded:
// groups of 8 (sizes 2, 4, 8), pairs of groups (size 16), all four groups (size 32).
__device__ __forceinline__ void thread_sort32_desc(int2* slots) {
#pragma unroll 1
  for (int g = 0; g < 4; ++g) {
    float v[8];
    int ix[8];
    topk_slots_load8(slots, 8 * g, v, ix);
#pragma unroll
    for (int e = 0; e < 8; e += 2) topk_ce_dir(v[e], ix[e], v[e + 1], ix[e + 1], (e & 2) == 0);
#pragma unroll
    for (int st = 2; st > 0; st >>= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if ((e & st) == 0) topk_ce_dir(v[e], ix[e], v[e | st], ix[e | st], (e & 4) == 0);
    }
    topk_merge8(v, ix, (g & 1) == 0);
    topk_slots_store8(slots, 8 * g, v, ix);
  }
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    float v[2][8];
    int ix[2][8];
    topk_slots_load8(slots, 16 * h, v[0], ix[0]);
    topk_slots_load8(slots, 16 * h + 8, v[1], ix[1]);
    const bool desc = h == 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) topk_ce_dir(v[0][e], ix[0][e], v[1][e], ix[1][e], desc);
    topk_merge8(v[0], ix[0], desc);
    topk_merge8(v[1], ix[1], desc);
    topk_slots_store8(slots, 16 * h, v[0], ix[0]);
    topk_slots_store8(slots, 16 * h + 8, v[1], ix[1]);
  }
  {
    float v[4][8];
    int ix[4][8];
#pragma unroll
    for (int c = 0; c < 4; ++c) topk_slots_load8(slots, 8 * c, v[c], ix[c]);
    topk_merge32_desc(v, ix);
#pragma unroll
    for (int c = 0; c < 4; ++c) topk_slots_store8(slots, 8 * c, v[c], ix[c]);
  }
}

// Every lane merges its own row's staged candidates (n_staged of them, at most 32, in the
// lane's staging slots) into its own list and returns the row's new k-th value.
// The list has room for 32 E entries in blocks of 32; the first ceil(k / 32) blocks are
// kept (sorted, descending), the rest always read as empty.
//   1. the candidates are padded to 32 and sorted in place in the staging slots;
//   2. first pass over the list, eight entries of every block at a time: the last block
//      meets the candidates in reverse order (keeping the better of each pair leaves the
//      best 32 E of list and candidates as a bitonic sequence), then the merge stages
//      whose stride is a multiple of 32 run across the blocks;
//   3. second pass, block by block: strides 16 to 1, all in registers. Blocks past the
//      k-th entry hold nothing that can reach the first k places any more and are dropped.
// `listed` (warp-uniform): the lists have been written in this unit; otherwise they start
// empty. sv / si: entry 0 of the lane's own row in the scratch arrays.
template <int E>
__device__ __noinline__ float topk_merge_own_rows(bool listed, int n_staged, float* sv, int* si, int k, int2* stg_own) {
  const int live_blocks = (k + 31) >> 5;
  FBMM_PROF_PHASE_DECL;
  for (int sl = n_staged; sl < 32; ++sl) stg_own[sl * kTileM] = make_int2(__float_as_int(-INFINITY), kTopkEmpty);
  __syncwarp();
  thread_sort32_desc(stg_own);
  FBMM_PROF_PHASE(0);
  if (E == 1) {
    // one block: it meets the candidates and is sorted in a single trip
    float v[4][8];
    int ix[4][8];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[c][e] = -INFINITY;
        ix[c][e] = kTopkEmpty;
        if (listed) {
          v[c][e] = sv[(8 * c + e) * kTileM];
          ix[c][e] = si[(8 * c + e) * kTileM];
        }
        const int2 cand = stg_own[(31 - (8 * c + e)) * kTileM];
        if (topk_before(__int_as_float(cand.x), cand.y, v[c][e], ix[c][e])) {
          v[c][e] = __int_as_float(cand.x);
          ix[c][e] = cand.y;
        }
      }
    }
    topk_merge32_desc(v, ix);
    float kth1 = -INFINITY;
    const int at = (k - 1) & 31;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sv[(8 * c + e) * kTileM] = v[c][e];
        si[(8 * c + e) * kTileM] = ix[c][e];
        if (8 * c + e == at) kth1 = v[c][e];
      }
    }
    return kth1;
  }
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    float v[E][8];
    int ix[E][8];
#pragma unroll
    for (int b = 0; b < E; ++b) {
      const bool use = listed && b < live_blocks;  // warp-uniform
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[b][e] = -INFINITY;
        ix[b][e] = kTopkEmpty;
        if (use) {
          v[b][e] = sv[(32 * b + 8 * c + e) * kTileM];
          ix[b][e] = si[(32 * b + 8 * c + e) * kTileM];
        }
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      // list entry 32 E - 32 + j meets candidate 31 - j
      const int2 cand = stg_own[(31 - (8 * c + e)) * kTileM];
      if (topk_before(__int_as_float(cand.x), cand.y, v[E - 1][e], ix[E - 1][e])) {
        v[E - 1][e] = __int_as_float(cand.x);
        ix[E - 1][e] = cand.y;
      }
    }
#pragma unroll
    for (int js = E >> 1; js > 0; js >>= 1) {
#pragma unroll
      for (int b = 0; b < E; ++b) {
        if ((b & js) == 0) {
#pragma unroll
          for (int e = 0; e < 8; ++e) topk_ce(v[b][e], ix[b][e], v[b | js][e], ix[b | js][e]);
        }
      }
    }
#pragma unroll
    for (int b = 0; b < E; ++b) {
      if (b < live_blocks) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sv[(32 * b + 8 * c + e) * kTileM] = v[b][e];
          si[(32 * b + 8 * c + e) * kTileM] = ix[b][e];
        }
      }
    }
  }
  FBMM_PROF_PHASE(1);
  float kth = -INFINITY;
#pragma unroll 1
  for (int b = 0; b < live_blocks; ++b) {
    float v[4][8];
    int ix[4][8];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        v[c][e] = sv[(32 * b + 8 * c + e) * kTileM];
        ix[c][e] = si[(32 * b + 8 * c + e) * kTileM];
      }
    }
    topk_merge32_desc(v, ix);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sv[(32 * b + 8 * c + e) * kTileM] = v[c][e];
        si[(32 * b + 8 * c + e) * kTileM] = ix[c][e];
      }
    }
    if (b == ((k - 1) >> 5)) {  // the block that holds the k-th entry
      const int at = (k - 1) & 31;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (8 * c + e == at) kth = v[c][e];
      }
    }
  }
  FBMM_PROF_PHASE(2);
  return kth;
}

// Copies the warp's 32 finished lists from the scratch area to the caller's layout
// (values [row][k] fp32, indices [row][k] int64 with `index_offset` added, empty entries
// -inf / -1), 32 entries of every row at a time through the warp's staging slots: a lane
// parks its own row's entries with the column rotated by the slot number, so that both
// the row-wise writes and the entry-wise reads spread over the banks, and the global
// stores run along the entries of one row. `rows_valid`: rows of this warp that exist.
__device__ __forceinline__ void topk_write_out(const float* sv, const int* si, int k, long long index_offset,
                                               float* lv0, long long* li0, int2* lp0, int rows_valid, int2* stg_w) {
  const int lane = static_cast<int>(lane_id());
  for (int e0 = 0; e0 < k; e0 += 32) {
#pragma unroll 8
    for (int j = 0; j < 32; ++j)
      stg_w[j * kTileM + ((lane + j) & 31)] = make_int2(__float_as_int(sv[(e0 + j) * kTileM]), si[(e0 + j) * kTileM]);
    __syncwarp();
    if (e0 + lane < k) {
#pragma unroll 4
      for (int r = 0; r < rows_valid; ++r) {
        const int2 e = stg_w[lane * kTileM + ((r + lane) & 31)];
        if (lp0 != nullptr) {
          lp0[static_cast<long long>(r) * k + e0 + lane] = make_int2(e.x, e.y == kTopkEmpty ? -1 : e.y);
        } else {
          lv0[static_cast<long long>(r) * k + e0 + lane] = __int_as_float(e.x);
          li0[static_cast<long long>(r) * k + e0 + lane] = (e.y == kTopkEmpty) ? -1ll : static_cast<long long>(e.y) + index_offset;
        }
      }
    }
    __syncwarp();
  }
}

// Shared-memory plan, computed identically on the host (launch size) and in the kernel.
//   [A region: kblocks x (hi 16 KB | lo 16 KB)]      only when A stays resident
//   [ring: stages x stage_bytes]                     stage = (A hi | A lo |) B hi | B lo
//   [top-k staging] [barriers]
constexpr int kTileN = 128;
constexpr int kMaxStages = 8;
constexpr int kMaxResidentKBlocks = 4;  // A stays resident up to K = 128
constexpr uint32_t kPlaneBytes = kTileM * kKBlock * 4;  // one 128 x 32 fp32 plane: 16 KB
constexpr uint32_t kTopkStageSlots = 32;                // staged candidates per row
constexpr uint32_t kTopkStageBytes = kTopkStageSlots * kTileM * 8u;

constexpr uint32_t kBarrierBytes = 512;
constexpr uint32_t kSmemLimit = 232448;  // 227 KB per CTA on sm_100

// Mask tiles of the mask epilogue (mbmm): the 128 x 128 element-mask bytes of a tile and its
// 16 x 16 thread-mask bytes, brought in by TMA two tiles ahead of the epilogue, which would
// otherwise wait out a trip to HBM for every chunk of every tile.
constexpr uint32_t kMaskStages = 2;
constexpr uint32_t kMaskElemBytes = kTileM * 128u;       // 128 rows x 128 columns, one byte each
constexpr uint32_t kMaskThreadBytes = 16u * 16u;         // one byte per 8 x 8 tile
constexpr uint32_t kMaskStageBytes = kMaskElemBytes + 512u;
// Softmax: the two epilogue warps that share a row (one per half of a tile's columns) exchange
// their running (maximum, sum) between the sweeps: [unit parity][column half][128 rows] x 8 bytes.
constexpr uint32_t kSoftmaxExchangeBytes = 2u * 2u * kTileM * 8u;

struct SmemPlan {
  uint32_t a_bytes, stage_bytes, stages, epi_bytes, total;
};
// `planes`: 2 for fp32 operands (hi and lo), 1 for 16-bit ones. `epi_extra`: what the epilogue
// keeps in shared memory (top-k staging, or the mask tiles).
// `pair`: a CTA of a pair keeps one whole plane of each B tile plus half a plane (see PAIR below).
__host__ __device__ inline SmemPlan make_smem_plan(bool a_resident, int kblocks, bool topk, uint32_t planes = 2u,
                                                   bool mask_tiles = false, bool pair = false,
                                                   bool softmax = false) {
  SmemPlan p;
  const uint32_t b_bytes = pair ? kPlaneBytes + kPlaneBytes / 2u : planes * kPlaneBytes;
  p.a_bytes = a_resident ? static_cast<uint32_t>(kblocks) * planes * kPlaneBytes : 0u;
  p.stage_bytes = (a_resident ? 0u : planes * kPlaneBytes) + b_bytes;
  p.epi_bytes = topk ? kTopkStageBytes : (mask_tiles ? kMaskStages * kMaskStageBytes : 0u);
  if (softmax) p.epi_bytes += kSoftmaxExchangeBytes;
  const uint32_t fixed = p.a_bytes + p.epi_bytes + kBarrierBytes + 1024u /* alignment slack */;
  uint32_t st = (kSmemLimit - fixed) / p.stage_bytes;
  p.stages = st > static_cast<uint32_t>(kMaxStages) ? static_cast<uint32_t>(kMaxStages) : st;
  p.total = fixed + p.stages * p.stage_bytes;
  return p;
}

struct Barriers {
  uint64_t full[kMaxStages];    // TMA landed in ring stage
  uint64_t split[kMaxStages];   // lo plane(s) of ring stage written
  uint64_t empty[kMaxStages];   // MMAs done reading ring stage
  uint64_t acc_full[2];         // accumulator stage complete
  uint64_t acc_empty[2];        // accumulator stage drained by the epilogue
  uint64_t a_full[kMaxResidentKBlocks];   // resident A k-block landed
  uint64_t a_split[kMaxResidentKBlocks];  // its lo plane written
  uint64_t a_empty[kMaxResidentKBlocks];  // last MMA of the unit done reading it
  uint64_t mask_full[kMaskStages];        // mask tile landed
  uint64_t mask_empty[kMaskStages];       // epilogue done reading it
  uint64_t xchg;                          // softmax: every epilogue warp has posted its (max, sum)
  uint32_t tmem_base;
  uint32_t abort_flag;
};
static_assert(sizeof(Barriers) <= kBarrierBytes, "barrier block too large");

// lo plane of `bytes` bytes of fp32 at `hi`, written to `lo` (same layout), by the 128
// splitter threads.
__device__ __forceinline__ void split_plane(const uint8_t* hi, uint8_t* lo, uint32_t bytes, int st) {
  const float4* src = reinterpret_cast<const float4*>(hi);
  float4* dst = reinterpret_cast<float4*>(lo);
#pragma unroll 8
  for (int i = st; i < static_cast<int>(bytes / 16); i += kSplitThreads) {
    const float4 x = src[i];
    dst[i] = make_float4(split_lo(x.x), split_lo(x.y), split_lo(x.z), split_lo(x.w));
  }
}

// PRESPLIT: lo planes were computed once by fbmm_split_lo_kernel into global scratch with
// the operands' own strides; TMA then brings hi and lo of everything that streams through
// the ring, and a ring stage is ready the moment its copies land. A resident row block of
// A is still split in shared memory (once per unit, so there is nothing to save).
//
// PAIR: the kernel runs as clusters of two CTAs on 256-row blocks, and the even CTA issues
// tcgen05.mma.cta_group::2 for both. What limits the single-CTA kernel is not the tensor
// core's arithmetic but the rate at which one thread can hand it instructions: an MMA costs
// the issuing thread 65 cycles or more whatever its shape, and with K = 8 per tf32
// instruction the 128 x 128 x 8 product (64 cycles of arithmetic) is issue-bound. A pair MMA
// does the work of two: M = 256 (128 rows of A from each CTA's own shared memory, 128
// accumulator rows in each CTA's own TMEM), and its N operand rows are taken half from each
// CTA. The three tf32 products of a k-step then take two instructions for 256 x 128 outputs:
//   wide    A_hi x [B_hi | B_lo], N = 256: the even CTA holds the tile's B_hi plane, the odd
//           CTA its B_lo plane, at the same shared-memory offset, so the instruction's first
//           128 result columns are hi*hi (the big accumulator) and the other 128 are hi*lo
//           (the small one) in both CTAs;
//   narrow  A_lo x B_hi, N = 128: the even CTA supplies columns 0-63 of B_hi, the odd CTA
//           columns 64-127 (a second copy of 8 KB per CTA, at a common offset).
// Measured on resident operands: 762 cycles per 256 x 128 x 32 k-block of a pair (4 wide + 4
// narrow, commits included) against 1057 per 128 x 128 x 32 in a single CTA: both SMs of a
// pair are busy for those 762 cycles, so per SM the gain is 1057 / 762 = 1.39, all of it from
// the narrow MMA (64 cycles as half of a pair, 112 alone). Each CTA loads its own operands (24 KB of B per k-block instead of 32 KB, no
// cluster fan-out of any copy); completion bytes of both CTAs are counted on the even CTA's
// barrier, barriers that gate the MMAs live in the even CTA (the peer arrives on them through
// the cluster window) and every commit goes to both CTAs. Needs pre-split planes and fp32
// operands; used by the reducing epilogues (min, top-k) for problems of more than 128 rows.
//
// DT: element type of the operands. 0 = fp32 (everything above). 1 = fp16, 2 = bf16: the
// operands are multiplied as they are by tcgen05.mma.kind::f16 (fp32 accumulation), one MMA
// per k-step into the big accumulator only; a k-block is 64 elements (still 128 bytes per
// row), there are no lo planes and nothing to split, so these variants are instantiated with
// PRESPLIT = true and load the hi planes only. Both operands must be k-contiguous. The
// lo-plane slots of the shared-memory plan stay unused.
//
// DUAL: two resident row blocks of A per CTA (a 256-row unit) take turns on the two accumulator
// stages, so that every ring stage of B serves 256 rows before it is released: half the operand
// bytes per output pulled out of L2 into the SM, which is what bounds the K <= 64 kernels (with
// the MMAs, the accumulator loads and the epilogue arithmetic compiled out they still took three
// quarters of their time). The ring walks real column tiles; the MMA thread and the epilogue walk
// "virtual tiles" (column tile, row block), row block 0 always on accumulator stage 0. A stage is
// waited for by the first row block and released by the second. Needs both blocks' hi and lo
// planes resident (2 x kblocks <= 4 slots: K <= 64), B's planes by TMA, a single CTA; min epilogue.
template <int EPI, int TOPK_E, bool A_RES, bool PRESPLIT, int DT = 0, bool PAIR = false, bool DUAL = false>
__global__ void __launch_bounds__(block_threads(EPI), 1)
fbmm_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_a_lo, const __grid_constant__ CUtensorMap tmap_b_lo,
                 const __grid_constant__ CUtensorMap tmap_em, const __grid_constant__ CUtensorMap tmap_tm,
                 const GemmShape shape, const EpiArgs epi) {
  constexpr int TILE_N = kTileN;
  constexpr int kAccStages = 2;
  static_assert(2 * kAccStages * TILE_N <= kTmemCols, "TMEM budget");

  constexpr bool kHalf = DT != 0;
  static_assert(!kHalf || PRESPLIT, "16-bit variants: PRESPLIT = true");
  static_assert(!PAIR || (PRESPLIT && !kHalf && (EPI == kEpiMin || EPI == kEpiTopk)),
                "pair variants: fp32 operands with pre-split planes, reducing epilogues");
  static_assert(!DUAL || (EPI == kEpiMin && A_RES && PRESPLIT && !PAIR && !kHalf),
                "dual row blocks: min epilogue, A resident, pre-split planes, single CTA, fp32");
  constexpr int kRb = DUAL ? 2 : 1;  // row blocks of A a CTA keeps resident
  constexpr int kKElems = kHalf ? 2 * kKBlock : kKBlock;  // elements of K per k-block (128 bytes)
  const int kblocks = (shape.K + kKElems - 1) / kKElems;
  constexpr uint32_t kPlanes = kHalf ? 1u : 2u;  // planes per operand tile in shared memory
  const bool mask_tma = is_masked(EPI) && epi.mask_tma != 0;
  constexpr int kSweeps = sweeps(EPI);
  const SmemPlan plan = make_smem_plan(A_RES, kblocks * kRb, EPI == kEpiTopk, kPlanes, mask_tma, PAIR, EPI == kEpiSoftmax);
  const uint32_t stages = plan.stages;
  constexpr uint32_t kBPlane = kPlaneBytes;  // one plane of a B tile
  // offsets inside a ring stage. Single CTA: (A hi | A lo |) B hi | B lo. Pair: (A hi | A lo |)
  // this CTA's plane of the wide operand (B hi in the even CTA, B lo in the odd one) | its 64
  // columns of B hi for the narrow MMA.
  const uint32_t off_a_hi = 0, off_a_lo = kPlaneBytes;
  const uint32_t off_b_hi = A_RES ? 0u : kPlanes * kPlaneBytes;
  const uint32_t off_b_lo = off_b_hi + kBPlane;
  const uint32_t off_b_narrow = off_b_hi + kBPlane;  // pair only

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_region = smem;
  uint8_t* ring = smem + plan.a_bytes;
  uint8_t* epi_smem = ring + stages * plan.stage_bytes;
  Barriers* bars = reinterpret_cast<Barriers*>(epi_smem + plan.epi_bytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = lane_id();
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;  // 0 = the CTA that issues the MMAs
  constexpr uint32_t kCtas = PAIR ? 2u : 1u;
  // the barrier block of both CTAs of a pair in the cluster window
  const uint32_t bars_cta0 = PAIR ? map_to_cta(smem_u32(bars), 0) : smem_u32(bars);
  const uint32_t bars_cta1 = PAIR ? map_to_cta(smem_u32(bars), 1) : smem_u32(bars);
  auto bar_off = [&](const uint64_t* b) -> uint32_t { return smem_u32(b) - smem_u32(bars); };

  if (threadIdx.x == 0) {
    bars->abort_flag = 0;
    for (int s = 0; s < kMaxStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->split[s], (kSplitThreads / 32) * kCtas);       // one arrival per splitter warp
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&bars->acc_full[s], 1);
      mbar_init(&bars->acc_empty[s], epilogue_warps(EPI) * kCtas);  // one arrival per epilogue warp
    }
    for (int s = 0; s < kMaxResidentKBlocks; ++s) {
      mbar_init(&bars->a_full[s], 1);
      mbar_init(&bars->a_split[s], (kSplitThreads / 32) * kCtas);
      mbar_init(&bars->a_empty[s], 1);
    }
    for (int s = 0; s < static_cast<int>(kMaskStages); ++s) {
      mbar_init(&bars->mask_full[s], 1);
      mbar_init(&bars->mask_empty[s], epilogue_warps(EPI));
    }
    mbar_init(&bars->xchg, epilogue_warps(EPI));
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (PRESPLIT && !kHalf) {
      tma_prefetch_desc(&tmap_a_lo);
      tma_prefetch_desc(&tmap_b_lo);
    }
    if (mask_tma) {
      tma_prefetch_desc(&tmap_em);
      tma_prefetch_desc(&tmap_tm);
    }
  }
  if (warp == 1) {
    if (PAIR) {
      tmem_alloc_pair(&bars->tmem_base, kTmemCols);
      tmem_relinquish_alloc_permit_pair();
    } else {
      tmem_alloc(&bars->tmem_base, kTmemCols);
      tmem_relinquish_alloc_permit();
    }
  }
  tcgen05_fence_before_sync();
  if (PAIR) cluster_sync_all(); else __syncthreads();
  tcgen05_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  const long long units = shape.num_units;
  // a pair walks the unit list as one worker
  const long long unit_first = PAIR ? (blockIdx.x >> 1) : blockIdx.x;
  const long long unit_step = PAIR ? (gridDim.x >> 1) : gridDim.x;
  // first row of this CTA inside row block `mb` (row blocks are 256 rows for pairs)
  // (with DUAL a unit is 256 rows too; its second row block starts kTileM rows further on)
  auto row_base = [&](int mb) -> int {
    return PAIR ? mb * 2 * kTileM + static_cast<int>(cta_rank) * kTileM : (DUAL ? mb * 2 * kTileM : mb * kTileM);
  };

  // Decodes unit u into batch, row block and column-tile range.
  auto decode = [&](long long u, int& b, int& mb, int& t0, int& t1) {
    const long long row_blocks = static_cast<long long>(shape.L) * shape.m_blocks;
    const int c = static_cast<int>(shape.chunk_major ? u / row_blocks : u % shape.n_chunks);
    const long long r = shape.chunk_major ? u % row_blocks : u / shape.n_chunks;
    mb = static_cast<int>(r % shape.m_blocks);
    b = static_cast<int>(r / shape.m_blocks);
    t0 = c * shape.tiles_per_chunk;
    t1 = min(shape.n_tiles, t0 + shape.tiles_per_chunk);
  };
  // Block-mask test of the mask epilogue (kernels/mbmm.cu:251-255): a zero byte means
  // the 128x128 tile is neither loaded nor multiplied. (Every role asks once per tile. Keeping
  // the bytes of a row block as a bit window in registers instead was measured and is slower:
  // the four registers it pins cost the epilogue and the MMA thread more than the loads do.)
  auto tile_live = [&](int b, int mb, int t) -> bool {
    if (!is_masked(EPI)) return true;
    if (mb * kTileM >= shape.M) return false;
    return epi.block_mask[b * epi.bm_stride + static_cast<long long>(mb) * epi.bm_cols + t] != 0;
  };
  // First and last live tile of a unit; false when the unit has none.
  auto live_range = [&](int b, int mb, int t0, int t1, int& first, int& last) -> bool {
    if (!is_masked(EPI)) { first = t0; last = t1 - 1; return t0 < t1; }
    first = -1; last = -1;
    for (int t = t0; t < t1; ++t)
      if (tile_live(b, mb, t)) { if (first < 0) first = t; last = t; }
    return first >= 0;
  };

  // The column operand is re-read by every row block, so it should outlive everything
  // else in L2. A resident row block of A is read exactly once (first out); a streamed one
  // is re-read for every column tile of the unit and keeps the default priority.
  const uint64_t a_policy = A_RES ? kL2EvictFirst : kL2EvictLast;
  // One TMA box into this CTA's shared memory. `bar` is a local barrier; with `to_leader` the
  // completion bytes are counted on the same barrier of the pair's even CTA instead.
  auto tma_issue = [&](uint8_t* dst, const CUtensorMap* map, uint64_t* bar, bool to_leader, int c0, int c1, int c2,
                       uint64_t policy) {
    if (PAIR && to_leader) tma_load_3d_pair(dst, map, bars_cta0 + bar_off(bar), c0, c1, c2, policy);
    else tma_load_3d(dst, map, bar, c0, c1, c2, policy);
  };
  // this CTA's 128 rows of A of row block mb, k-block kb
  auto load_a = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, bool to_leader, int kb, int mb, int b,
                    int row_off = 0) {
    if (shape.a_bcast) b = 0;
    if (!shape.a_mn) {
      tma_issue(dst, map, bar, to_leader, kb * kKElems, row_base(mb) + row_off, b, a_policy);
    } else {
#pragma unroll
      for (int c = 0; c < kTileM / 32; ++c)
        tma_issue(dst + c * 4096, map, bar, to_leader, row_base(mb) + row_off + c * 32, kb * kKBlock, b, a_policy);
    }
  };
  // `ncols` columns (a multiple of 32) of an operand plane of B starting at column `col`, k-block kb.
  // K-major tensor maps of the pair kernels have boxes of 64 rows, the others of 128.
  auto load_b_cols = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, bool to_leader, int kb, int col, int ncols,
                         int b) {
    if (shape.b_bcast) b = 0;
    if (!shape.b_mn) {
      constexpr int kBox = PAIR ? TILE_N / 2 : TILE_N;
      for (int c = 0; c < ncols; c += kBox)
        tma_issue(dst + c * 128, map, bar, to_leader, kb * kKElems, col + c, b, kL2EvictLast);
    } else {
      for (int c = 0; c < ncols; c += 32)
        tma_issue(dst + c * 128, map, bar, to_leader, col + c, kb * kKBlock, b, kL2EvictLast);
    }
  };
  // the 128 columns of B tile t, k-block kb (single CTA)
  auto load_b = [&](const CUtensorMap* map, uint8_t* dst, uint64_t* bar, int kb, int t, int b) {
    load_b_cols(map, dst, bar, false, kb, t * TILE_N, TILE_N, b);
  };

  // Barriers that gate the MMAs live in the pair's even CTA: the peer arrives through the
  // cluster window, the issuer waits with cluster scope, and commits go to both CTAs.
  // One arrival per warp, by lane 0 once every lane has got there: an arrival through the
  // cluster window costs hundreds of cycles when 128 threads queue up for it.
  auto warp_arrive = [&](uint64_t* bar) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
  };
  auto warp_arrive_leader = [&](uint64_t* bar) {
    __syncwarp();
    if (lane == 0) {
      if (PAIR && cta_rank != 0) mbar_arrive_cluster(bars_cta0 + bar_off(bar)); else mbar_arrive(bar);
    }
  };
  // every wait of a pair kernel whose arrivals can come through the cluster (the peer's
  // arrivals, pair commits, the peer's copies) uses the cluster-scope form
  auto wait_gate = [&](uint64_t* bar, uint32_t parity) -> bool {
    return PAIR ? mbar_wait_cluster(bar, parity, abort_flag) : mbar_wait(bar, parity, abort_flag);
  };
  auto commit_all = [&](uint64_t* bar) {
    if (PAIR) {
      umma_commit_pair(bars_cta0 + bar_off(bar));
      umma_commit_pair(bars_cta1 + bar_off(bar));
    } else {
      umma_commit(bar);
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, mstage = 0, mphase = 0;
      bool ok = true;
      FBMM_PROF_DECL;
      const long long prof_start = clock64();
      long long pace_seq = 0;  // number of this CTA's next range
      const long long pace_ranges = shape.pace_tiles > 0 ? (shape.n_tiles + shape.pace_tiles - 1) / shape.pace_tiles : 0;
      for (long long u = unit_first; u < units && ok; u += unit_step) {
        int b, mb, t0, t1, first, last;
        decode(u, b, mb, t0, t1);
        if (!live_range( b, mb, t0, t1, first, last)) continue;
        for (int sweep = 0; sweep < kSweeps; ++sweep)
        for (int t = first; t <= last && ok; ++t) {
          if (!tile_live(b, mb, t)) continue;
          if (shape.pace_tiles > 0 && cta_rank == 0 && (t - t0) % shape.pace_tiles == 0) {
            if (pace_seq > 0) atomicAdd(shape.pace_counts + pace_seq - 1, 1u);  // the range before is requested
            if (pace_seq >= shape.pace_slack) {
              // CTAs that have a unit of the ordinal the awaited range belongs to
              const long long g = pace_seq - shape.pace_slack;
              const long long ahead = units - (g / pace_ranges) * unit_step;
              const unsigned int expected = static_cast<unsigned int>(ahead < unit_step ? ahead : unit_step);
              const volatile unsigned int* cnt = shape.pace_counts + g;
              const long long w0 = clock64();
              while (*cnt < expected && clock64() - w0 < kPaceWaitCycles) __nanosleep(256);
            }
            ++pace_seq;
          }
          if (mask_tma) {
            // the tile's mask bytes, as soon as the epilogue has let go of the stage
            ok = mbar_wait(&bars->mask_empty[mstage], mphase ^ 1u, abort_flag);
            if (!ok) break;
            uint8_t* ms = epi_smem + mstage * kMaskStageBytes;
            const int mask_b = epi.em_stride == 0 ? 0 : b;  // shared masks have no batch axis
            mbar_arrive_expect_tx(&bars->mask_full[mstage], kMaskElemBytes + kMaskThreadBytes);
            tma_load_3d(ms, &tmap_em, &bars->mask_full[mstage], t * TILE_N, row_base(mb), mask_b, kL2EvictFirst);
            tma_load_3d(ms + kMaskElemBytes, &tmap_tm, &bars->mask_full[mstage], t * (TILE_N / 8), row_base(mb) / 8,
                        mask_b, kL2EvictFirst);
            if (++mstage == kMaskStages) { mstage = 0; mphase ^= 1u; }
          }
          for (int kb = 0; kb < kblocks; ++kb) {
            FBMM_PROF_BEGIN();
            ok = wait_gate(&bars->empty[stage], phase ^ 1u);
            FBMM_PROF_END(0);
            if (!ok) break;
            uint8_t* sb = ring + stage * plan.stage_bytes;
            if (PAIR) {
              // each CTA brings its own operands; the even CTA's barrier counts the bytes of both
              constexpr uint32_t kMyBytes = (A_RES ? 0u : 2u * kPlaneBytes) + kPlaneBytes + kPlaneBytes / 2u;
              if (cta_rank == 0) mbar_arrive_expect_tx(&bars->full[stage], 2u * kMyBytes);
              if (!A_RES) {
                load_a(&tmap_a, sb + off_a_hi, &bars->full[stage], true, kb, mb, b);
                load_a(&tmap_a_lo, sb + off_a_lo, &bars->full[stage], true, kb, mb, b);
              }
              const int col = t * TILE_N;
              // wide operand: B hi in the even CTA, B lo in the odd one; narrow: this CTA's 64 columns of B hi
              load_b_cols(cta_rank == 0 ? &tmap_b : &tmap_b_lo, sb + off_b_hi, &bars->full[stage], true, kb, col, TILE_N, b);
              load_b_cols(&tmap_b, sb + off_b_narrow, &bars->full[stage], true, kb,
                          col + static_cast<int>(cta_rank) * (TILE_N / 2), TILE_N / 2, b);
            } else {
              // bytes that land in the stage
              constexpr uint32_t kStageTx = ((A_RES ? 0u : kPlaneBytes) + kBPlane) * ((PRESPLIT && !kHalf) ? 2u : 1u);
              mbar_arrive_expect_tx(&bars->full[stage], kStageTx);
              if (!A_RES) {
                load_a(&tmap_a, sb + off_a_hi, &bars->full[stage], false, kb, mb, b);
                if (PRESPLIT && !kHalf) load_a(&tmap_a_lo, sb + off_a_lo, &bars->full[stage], false, kb, mb, b);
              }
              load_b(&tmap_b, sb + off_b_hi, &bars->full[stage], kb, t, b);
              if (PRESPLIT && !kHalf) load_b(&tmap_b_lo, sb + off_b_lo, &bars->full[stage], kb, t, b);
            }
            if (++stage == stages) { stage = 0; phase ^= 1u; }
          }
        }
      }
      // the last range counts too: CTAs with one more unit wait for it
      if (shape.pace_tiles > 0 && pace_seq > 0) atomicAdd(shape.pace_counts + pace_seq - 1, 1u);
#ifdef FBMM_PROFILE
      prof_acc_[1] = clock64() - prof_start;
#endif
      (void)prof_start;
      FBMM_PROF_FLUSH(0);
      if (!ok) {
        // Give copies already in flight a bounded time to land before the CTA leaves.
        const long long t0c = clock64();
        while (clock64() - t0c < 2000000LL) {}
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && cta_rank == 0) {
      // A ring stage holds the B hi plane directly followed by the B lo plane, so one MMA
      // of width 2 * TILE_N over both computes hi*hi into the big accumulator and hi*lo
      // into the small one next to it while reading A_hi once.
      static_assert(2 * TILE_N <= 256, "the merged hi|lo MMA needs 2 * TILE_N <= 256");
      const uint32_t idesc = make_idesc_tf32(kTileM, TILE_N, shape.a_mn != 0, shape.b_mn != 0);
      const uint32_t idesc_wide = make_idesc_tf32(kTileM, 2 * TILE_N, shape.a_mn != 0, shape.b_mn != 0);
      const uint32_t a_lbo = shape.a_mn ? 4096u : 16u, a_sbo = shape.a_mn ? 512u : 1024u;
      const uint32_t b_lbo = shape.b_mn ? 4096u : 16u, b_sbo = shape.b_mn ? 512u : 1024u;
      const uint32_t a_kstep = shape.a_mn ? 1024u : 32u, b_kstep = shape.b_mn ? 1024u : 32u;
      // One thread has to issue an MMA every 64 cycles, so the shared-memory descriptors are
      // kept as two 32-bit halves: the upper half (stride offset, version, layout type) is a
      // constant per operand, the lower half is (address >> 4) | (lbo >> 4) << 16 and moves
      // by a constant per k-step. Building each descriptor from scratch made the issuing
      // thread, not the tensor core, the limit.
      const uint32_t a_desc_hi = (a_sbo >> 4) | (1u << 14) | ((shape.a_mn ? 1u : 2u) << 29);
      const uint32_t b_desc_hi = (b_sbo >> 4) | (1u << 14) | ((shape.b_mn ? 1u : 2u) << 29);
      const uint32_t a_lbo_bits = ((a_lbo >> 4) & 0x3fffu) << 16, b_lbo_bits = ((b_lbo >> 4) & 0x3fffu) << 16;
      const uint32_t a_step = a_kstep >> 4, b_step = b_kstep >> 4;
      auto pack = [](uint32_t lo, uint32_t hi) -> uint64_t {
        uint64_t d;
        asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
        return d;
      };
      // pair: M = 256 over both CTAs; N counts the operand rows of both CTAs together
      const uint32_t idesc_pair_wide = make_idesc_tf32(2 * kTileM, 2 * TILE_N, shape.a_mn != 0, shape.b_mn != 0);
      const uint32_t idesc_pair_narrow = make_idesc_tf32(2 * kTileM, TILE_N, shape.a_mn != 0, shape.b_mn != 0);
      uint32_t stage = 0, phase = 0, acc_stage = 0, acc_phase = 0, a_phase = 0;
      bool ok = true;
      FBMM_PROF_DECL;
      FBMM_TRACE_DECL;
      for (long long u = unit_first; u < units && ok; u += unit_step) {
        int b, mb, t0, t1, first, last;
        decode(u, b, mb, t0, t1);
        if (!live_range( b, mb, t0, t1, first, last)) continue;
        for (int sweep = 0; sweep < kSweeps; ++sweep)
        for (int t = first; t <= last && ok; ++t) {
          if (!tile_live(b, mb, t)) continue;
          // (DUAL: the tile's ring stages are walked once per row block, from the same start)
          const uint32_t stage_t = stage, phase_t = phase;
          for (int rb = 0; rb < kRb && ok; ++rb) {
          stage = stage_t;
          phase = phase_t;
          FBMM_TRACE(0);
          FBMM_PROF_BEGIN();
          ok = wait_gate(&bars->acc_empty[acc_stage], acc_phase ^ 1u);
          FBMM_PROF_END(0);
          if (!ok) break;
          tcgen05_fence_after_sync();
          const uint32_t acc_big = tmem_base + acc_stage * (2 * TILE_N);
          const uint32_t acc_small = acc_big + TILE_N;
          for (int kb = 0; kb < kblocks; ++kb) {
            const int a_slot = rb * kblocks + kb;  // resident slot of this row block's k-block
            if (A_RES && t == first && sweep == 0) {
              // 16-bit operands are used as they land; fp32 ones once their lo plane exists
              FBMM_PROF_BEGIN();
              ok = wait_gate(kHalf ? &bars->a_full[a_slot] : &bars->a_split[a_slot], a_phase);
              FBMM_PROF_END(3);
              if (!ok) break;
            }
            if (rb == 0) {  // (the second row block finds the stage as the first left it)
              FBMM_PROF_BEGIN();
              ok = wait_gate(PRESPLIT ? &bars->full[stage] : &bars->split[stage], phase);
              FBMM_PROF_END(1);
              if (!ok) break;
            }
            // (no tcgen05 fence here: the operands reach shared memory through the async
            // proxy, or through writers that ran fence.proxy.async before arriving)
            FBMM_PROF_BEGIN();
            const uint32_t sb = smem_u32(ring + stage * plan.stage_bytes);
            const uint32_t sa = A_RES ? smem_u32(a_region + a_slot * kPlanes * kPlaneBytes) : sb;
            // Issue order: all four k-steps of one operand-plane combination before the
            // next combination, so that consecutive MMAs walk the same 128-byte
            // shared-memory rows.
            const uint32_t first_kb = kb == 0 ? 0u : 1u;
            const uint32_t a_hi0 = ((sa + off_a_hi) >> 4) | a_lbo_bits, a_lo0 = ((sa + off_a_lo) >> 4) | a_lbo_bits;
            const uint32_t b_hi0 = ((sb + off_b_hi) >> 4) | b_lbo_bits, b_lo0 = ((sb + off_b_lo) >> 4) | b_lbo_bits;
            if (kHalf) {
              const uint32_t idesc_half = make_idesc_f16(kTileM, TILE_N, DT == 2);
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)  // big (+)= A * B, 16 elements of K per MMA
                umma_f16(acc_big, pack(a_hi0 + ks * a_step, a_desc_hi), pack(b_hi0 + ks * b_step, b_desc_hi),
                         idesc_half, ks == 0 ? first_kb : 1u);
              (void)a_lo0; (void)b_lo0; (void)acc_small; (void)idesc; (void)idesc_wide;
            } else if (PAIR) {
              const uint32_t b_nar0 = ((sb + off_b_narrow) >> 4) | b_lbo_bits;
#pragma unroll
              for (int ks = 0; ks < kKBlock / 8; ++ks)  // [big | small] (+)= A_hi * [B_hi (even CTA) | B_lo (odd CTA)]
                umma_tf32_pair(acc_big, pack(a_hi0 + ks * a_step, a_desc_hi), pack(b_hi0 + ks * b_step, b_desc_hi),
                               idesc_pair_wide, ks == 0 ? first_kb : 1u);
#pragma unroll
              for (int ks = 0; ks < kKBlock / 8; ++ks)  // small += A_lo * B_hi (64 columns from each CTA)
                umma_tf32_pair(acc_small, pack(a_lo0 + ks * a_step, a_desc_hi), pack(b_nar0 + ks * b_step, b_desc_hi),
                               idesc_pair_narrow, 1u);
              (void)b_lo0;
            } else {
#pragma unroll
              for (int ks = 0; ks < kKBlock / 8; ++ks)  // [big | small] (+)= A_hi * [B_hi | B_lo]
                umma_tf32(acc_big, pack(a_hi0 + ks * a_step, a_desc_hi), pack(b_hi0 + ks * b_step, b_desc_hi),
                          idesc_wide, ks == 0 ? first_kb : 1u);
#pragma unroll
              for (int ks = 0; ks < kKBlock / 8; ++ks)  // small += A_lo * B_hi
                umma_tf32(acc_small, pack(a_lo0 + ks * a_step, a_desc_hi), pack(b_hi0 + ks * b_step, b_desc_hi), idesc,
                          1u);
              (void)b_lo0;
            }
            if (rb == kRb - 1) commit_all(&bars->empty[stage]);  // the last row block releases the stage
            if (A_RES && t == last && sweep == kSweeps - 1) commit_all(&bars->a_empty[a_slot]);
            FBMM_PROF_END(2);
            if (++stage == stages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          commit_all(&bars->acc_full[acc_stage]);
          if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1u; }
          }  // row blocks
        }
        a_phase ^= 1u;
      }
      FBMM_PROF_FLUSH(4);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ hi/lo splitters
    if (kHalf || (PRESPLIT && !A_RES)) {
      // nothing to split: every lo plane arrives by TMA, or (16-bit operands) there is none
    } else {
    const int st = static_cast<int>(threadIdx.x) - 64;
    uint32_t stage = 0, phase = 0, a_phase = 0;
    bool ok = true;
    FBMM_PROF_DECL;
    for (long long u = unit_first; u < units && ok; u += unit_step) {
      int b, mb, t0, t1, first, last;
      decode(u, b, mb, t0, t1);
      if (!live_range( b, mb, t0, t1, first, last)) continue;
      for (int sweep = 0; sweep < kSweeps; ++sweep)
      for (int t = first; t <= last && ok; ++t) {
        if (!tile_live(b, mb, t)) continue;
        if (PRESPLIT && (t != first || sweep != 0)) break;  // only the unit's resident A block needs splitting
        for (int kb = 0; kb < (DUAL ? 2 * kblocks : kblocks); ++kb) {  // (DUAL: kb counts resident slots)
          if (A_RES && t == first && sweep == 0) {
            ok = mbar_wait(&bars->a_full[kb], a_phase, abort_flag);
            if (!ok) break;
            uint8_t* ab = a_region + kb * 2 * kPlaneBytes;
            split_plane(ab + off_a_hi, ab + off_a_lo, kPlaneBytes, st);
            fence_proxy_async_smem();
            warp_arrive_leader(&bars->a_split[kb]);
          }
          if (PRESPLIT) continue;
          FBMM_PROF_BEGIN();
          ok = mbar_wait(&bars->full[stage], phase, abort_flag);
          FBMM_PROF_END(0);
          if (!ok) break;
          FBMM_PROF_BEGIN();
          uint8_t* sb = ring + stage * plan.stage_bytes;
          if (!A_RES) split_plane(sb + off_a_hi, sb + off_a_lo, kPlaneBytes, st);
          split_plane(sb + off_b_hi, sb + off_b_lo, kBPlane, st);
          FBMM_PROF_END(1);
          FBMM_PROF_BEGIN();
          fence_proxy_async_smem();
          warp_arrive_leader(&bars->split[stage]);
          FBMM_PROF_END(2);
          if (++stage == stages) { stage = 0; phase ^= 1u; }
        }
      }
      a_phase ^= 1u;
    }
    if (st == 0) { FBMM_PROF_FLUSH(8); }
    }
  } else if (warp < 6u + epilogue_warps(EPI)) {
    // ------------------------------------------------------------------ epilogue
    const uint32_t quarter = warp & 3u;  // TMEM lanes this warp may read
    // 32-column chunks of a tile this warp handles
    constexpr int kChunksPerWarp = (TILE_N / 32) / (epilogue_warps(EPI) / 4);
    const int chunk_first = static_cast<int>((warp - 6u) >> 2) * kChunksPerWarp;
    const int chunk_end = chunk_first + kChunksPerWarp;
    const int row_in_tile = static_cast<int>(quarter * 32u + lane);
    const uint32_t lane_base = (quarter * 32u) << 16;
    uint32_t acc_stage = 0, acc_phase = 0, mstage = 0, mphase = 0;
    uint32_t xparity = 0;  // softmax: parity of the exchange barrier = which half of its buffer is in use
    bool ok = true;
    FBMM_PROF_DECL;
    FBMM_TRACE_DECL;

    // 256-bit stores need every row start of C 32-byte aligned
    const bool c_lines_ok = (EPI == kEpiStore || is_masked(EPI)) && ((epi.ldc & 7) == 0) &&
                            ((epi.stride_c & 7) == 0) && ((reinterpret_cast<uintptr_t>(epi.C) & 31) == 0);
    // 8-byte reads of the element mask need its rows 8-byte aligned
    const bool em_lines_ok = (EPI == kEpiMask) && ((shape.N & 7) == 0) && ((epi.em_stride & 7) == 0) &&
                             ((reinterpret_cast<uintptr_t>(epi.element_mask) & 7) == 0);
    // top-k staging: 8-byte (value, column) entries, slot-major [slot][row]
    int2* stg = reinterpret_cast<int2*>(epi_smem);
    for (long long u = unit_first; u < units && ok; u += unit_step) {
      int b, mb, t0, t1;
      decode(u, b, mb, t0, t1);
      const int row = row_base(mb) + row_in_tile;
      const bool row_ok = row < shape.M;

      // squared-l2 mode: this row's squared norm
      const bool l2 = (EPI == kEpiMin || EPI == kEpiTopk) && epi.row_norms != nullptr;
      float row_norm = (l2 && row_ok) ? epi.row_norms[static_cast<long long>(b) * shape.M + row] : 0.f;
      // per-unit reduction state
      float best = INFINITY;
      int best_col = t0 * TILE_N;
      // DUAL: the same for this thread's row of the unit's second row block (row + kTileM); the two
      // sets change places around every virtual tile of that block
      const bool row_ok_o = DUAL && row + kTileM < shape.M;
      float row_norm_o = (DUAL && l2 && row_ok_o) ? epi.row_norms[static_cast<long long>(b) * shape.M + row + kTileM] : 0.f;
      float best_o = INFINITY;
      int best_col_o = t0 * TILE_N;
      // top-k: current k-th best of this row (+inf for rows past M, which never stage)
      float thr = row_ok ? -INFINITY : INFINITY;
      const uint32_t stg_base = smem_u32(stg + row_in_tile);
      uint32_t stg_slot = stg_base;  // address of this row's next free staging slot
      bool has_list = false;  // warp-uniform: the lists of this unit have been written
      // output lists of this warp's first row (rows of a warp are consecutive)
      const long long warp_row0 = (shape.tiles_per_chunk > 0 ? (t0 / shape.tiles_per_chunk) : 0) * epi.topk_chunk_rows +
                                  static_cast<long long>(b) * shape.M + row_base(mb) + static_cast<int>(quarter) * 32;
      const bool packed_out = (EPI == kEpiTopk) && epi.topk_packed != nullptr;
      float* lv0 = (EPI == kEpiTopk && !packed_out) ? epi.topk_values + warp_row0 * epi.k : nullptr;
      long long* li0 = (EPI == kEpiTopk && !packed_out) ? epi.topk_indices + warp_row0 * epi.k : nullptr;
      int2* lp0 = packed_out ? epi.topk_packed + warp_row0 * epi.k : nullptr;
      int2* stg_w = stg + quarter * 32;
      // running list of this lane's row in the CTA's scratch area
      float* sv = nullptr;
      int* si = nullptr;
      if (EPI == kEpiTopk) {
        constexpr long long kListEntries = 32ll * TOPK_E * kTileM;
        sv = epi.topk_scratch + static_cast<long long>(blockIdx.x) * 2 * kListEntries + row_in_tile;
        si = reinterpret_cast<int*>(sv + kListEntries);
      }

      // softmax: running maximum (in the exp2 domain) and sum of this row over the kept entries
      float sm_max = -INFINITY, sm_sum = 0.f, sm_inv = 0.f;

      for (int sweep = 0; sweep < kSweeps; ++sweep) {
      if (EPI == kEpiSoftmax && sweep == 1) {
        // The other half of this row's columns went through another warp: post this warp's
        // (maximum, sum), wait until all eight warps have, and fold the partner's in.
        float2* xb = reinterpret_cast<float2*>(epi_smem + plan.epi_bytes - kSoftmaxExchangeBytes) + xparity * 2 * kTileM;
        const int half = static_cast<int>((warp - 6u) >> 2);
        xb[half * kTileM + row_in_tile] = make_float2(sm_max, sm_sum);
        warp_arrive(&bars->xchg);
        ok = mbar_wait(&bars->xchg, xparity, abort_flag);
        if (!ok) break;
        const float2 o = xb[(half ^ 1) * kTileM + row_in_tile];
        xparity ^= 1u;
        const float mx = fmaxf(sm_max, o.x);
        if (mx == -INFINITY) {  // the row keeps nothing: all zeros
          sm_max = 0.f;
          sm_inv = 0.f;
        } else {
          sm_sum = sm_sum * ex2_approx(sm_max - mx) + o.y * ex2_approx(o.x - mx);
          sm_max = mx;
          sm_inv = sm_sum > 0.f ? 1.f / sm_sum : 0.f;
        }
      }
      for (int t = t0; t < t1 && ok; ++t) {
      for (int rb = 0; rb < kRb && ok; ++rb) {  // (one pass unless DUAL)
        if (DUAL && rb == 1) {
          float tf = best; best = best_o; best_o = tf;
          int ti = best_col; best_col = best_col_o; best_col_o = ti;
          tf = row_norm; row_norm = row_norm_o; row_norm_o = tf;
        }
        const int col_tile = t * TILE_N;
        FBMM_TRACE_TAG(3, 0);
        const bool live = tile_live(b, mb, t);
        if (live) { FBMM_TRACE_TAG(3, 1); }  // loads and MMAs happen for this tile
        if (!live) {
          // masked-out block: the product is defined as zero (mbmm.py:74 pre-zeroes C).
          FBMM_PROF_BEGIN();
          if (EPI == kEpiMask || (EPI == kEpiSoftmax && sweep == 1)) {
            const int c_end = min(shape.N, col_tile + TILE_N);
            if (kHalf) {
              // 16-bit C: element-wise zeros over this warp's columns of the row
              if (row_ok) {
                uint16_t* crow16 = reinterpret_cast<uint16_t*>(epi.C) + b * epi.stride_c + static_cast<long long>(row) * epi.ldc;
                for (int c = col_tile + chunk_first * 32; c < min(c_end, col_tile + chunk_end * 32); ++c) crow16[c] = 0;
              }
            } else if (c_lines_ok && col_tile + TILE_N <= shape.N) {
              // four lanes per row: every store instruction writes eight whole lines
              const int q = static_cast<int>(lane & 3u);
              const int row_g = row_base(mb) + static_cast<int>(quarter) * 32 + static_cast<int>(lane & ~3u);
              float* cbase = epi.C + b * epi.stride_c + static_cast<long long>(row_g) * epi.ldc + col_tile + 8 * q;
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (row_g + i < shape.M)
#pragma unroll
                  for (int c = 0; c < kChunksPerWarp * 32; c += 32)
                    st_global_v8_streaming(cbase + static_cast<long long>(i) * epi.ldc + chunk_first * 32 + c, 0.f, 0.f,
                                           0.f, 0.f, 0.f, 0.f, 0.f, 0.f);
            } else if (row_ok) {
              float* crow = epi.C + b * epi.stride_c + static_cast<long long>(row) * epi.ldc;
              for (int c = col_tile + chunk_first * 32; c < min(c_end, col_tile + chunk_end * 32); ++c) crow[c] = 0.f;
            }
          }
          FBMM_PROF_END(3);
          FBMM_TRACE_TAG(3, 2);
          continue;
        }
        // Mask bytes of a 32-column chunk for this lane after the lane-quad transpose (lane q
        // of a quad: columns [8q, 8q + 8) of the quad's four rows). They are fetched one
        // chunk ahead -- the first chunk's before the wait for the accumulator -- because
        // with one epilogue warp per scheduler a trip to L2 or HBM is otherwise waited out
        // in full on every chunk.
        unsigned char tmv_n[4] = {0, 0, 0, 0};
        uint2 e8_n[4] = {};
        auto mask_line_ok = [&](int col0) -> bool {
          return EPI == kEpiMask && c_lines_ok && em_lines_ok && col0 + 32 <= shape.N;
        };
        auto mask_fetch = [&](int col0) {
          const int q = static_cast<int>(lane & 3u);
          const int row_g = row_base(mb) + static_cast<int>(quarter) * 32 + static_cast<int>(lane & ~3u);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int r = min(row_g + i, shape.M - 1);
            tmv_n[i] = epi.thread_mask[b * epi.tm_stride + static_cast<long long>(r >> 3) * epi.tm_cols + (col0 >> 3) + q];
            e8_n[i] = *reinterpret_cast<const uint2*>(epi.element_mask + b * epi.em_stride +
                                                      static_cast<long long>(r) * shape.N + col0 + 8 * q);
          }
        };
        if (!mask_tma && mask_line_ok(col_tile + chunk_first * 32)) mask_fetch(col_tile + chunk_first * 32);
        const uint8_t* mask_tile = epi_smem + mstage * kMaskStageBytes;
        if (mask_tma) {
          FBMM_PROF_BEGIN();
          ok = mbar_wait(&bars->mask_full[mstage], mphase, abort_flag);
          FBMM_PROF_END(2);
          if (!ok) break;
        }
        FBMM_TRACE_TAG(3, 3);
        FBMM_PROF_BEGIN();
        ok = wait_gate(&bars->acc_full[acc_stage], acc_phase);
        FBMM_PROF_END(0);
        if (!ok) break;
        FBMM_TRACE_TAG(3, 4);
        tcgen05_fence_after_sync();
        FBMM_PROF_BEGIN();
        const uint32_t acc_big = tmem_base + acc_stage * (2 * TILE_N) + lane_base;
        const uint32_t acc_small = acc_big + TILE_N;
#pragma unroll 1
        for (int c = chunk_first; c < chunk_end; ++c) {
          uint32_t rb[32], rs[32];
          unsigned char tmv[4];
          uint2 e8[4];
          // softmax: the 32 element-mask bytes of this thread's row in the chunk, as 8 words, with
          // the bytes of a dropped 8 x 8 tile (zero thread-mask byte), of columns past N and of
          // rows past M cleared: a non-zero byte is a kept entry. Read before the TMEM loads: after
          // the last chunk's loads the mask stage goes back to the producer.
          uint32_t ew[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
          uint32_t any_kept = 0;
          if (EPI == kEpiSoftmax) {
            const int kc0 = col_tile + c * 32;
            uint32_t tmw = 0;
            if (mask_tma) {
              // (rows past M and columns past N arrive zero-filled)
              const uint4 e0 = *reinterpret_cast<const uint4*>(mask_tile + row_in_tile * 128 + c * 32);
              const uint4 e1 = *reinterpret_cast<const uint4*>(mask_tile + row_in_tile * 128 + c * 32 + 16);
              tmw = *reinterpret_cast<const uint32_t*>(mask_tile + kMaskElemBytes + (row_in_tile >> 3) * 16 + c * 4);
              ew[0] = e0.x; ew[1] = e0.y; ew[2] = e0.z; ew[3] = e0.w;
              ew[4] = e1.x; ew[5] = e1.y; ew[6] = e1.z; ew[7] = e1.w;
            } else if (row_ok) {
              const unsigned char* tm =
                  epi.thread_mask + b * epi.tm_stride + static_cast<long long>(row >> 3) * epi.tm_cols + (kc0 >> 3);
              const unsigned char* em = epi.element_mask + b * epi.em_stride + static_cast<long long>(row) * shape.N + kc0;
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (kc0 + j < shape.N) ew[j >> 2] |= static_cast<uint32_t>(em[j]) << ((j & 3) * 8);
#pragma unroll
              for (int g = 0; g < 4; ++g)
                if (kc0 + 8 * g < shape.N) tmw |= static_cast<uint32_t>(tm[g]) << (g * 8);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (((tmw >> (g * 8)) & 0xffu) == 0u) ew[2 * g] = ew[2 * g + 1] = 0u;
#pragma unroll
            for (int g = 0; g < 8; ++g) any_kept |= ew[g];
          }
          if (EPI == kEpiMask && mask_tma) {
            // lane q of a quad: columns [8q, 8q + 8) of the quad's four rows, which share one
            // 8-row thread-mask tile
            const int q = static_cast<int>(lane & 3u);
            const int row_l = static_cast<int>(quarter) * 32 + static_cast<int>(lane & ~3u);
            const unsigned char tb = mask_tile[kMaskElemBytes + (row_l >> 3) * 16 + c * 4 + q];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              tmv[i] = tb;
              e8[i] = *reinterpret_cast<const uint2*>(mask_tile + (row_l + i) * 128 + c * 32 + 8 * q);
            }
          } else if (EPI == kEpiMask) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { tmv[i] = tmv_n[i]; e8[i] = e8_n[i]; }
            if (c + 1 < chunk_end && mask_line_ok(col_tile + (c + 1) * 32)) mask_fetch(col_tile + (c + 1) * 32);
          }
          FBMM_PROF_XBEGIN();
          tmem_ld_32x32b_x32(acc_big + c * 32, rb);
          if (!kHalf) tmem_ld_32x32b_x32(acc_small + c * 32, rs);
          tmem_ld_wait();
          FBMM_PROF_XEND(0);
          FBMM_PROF_XBEGIN();
          if (c == chunk_end - 1) {
            // both accumulators of this stage are now in registers: hand the stage back
            FBMM_PROF_XEND(1);
            FBMM_PROF_XBEGIN();
            tcgen05_fence_before_sync();
            warp_arrive_leader(&bars->acc_empty[acc_stage]);
            if (mask_tma) warp_arrive(&bars->mask_empty[mstage]);  // its mask bytes too
            FBMM_PROF_XEND(2);
            FBMM_PROF_XBEGIN();
          }
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = kHalf ? __uint_as_float(rb[j]) : __uint_as_float(rb[j]) + __uint_as_float(rs[j]);
          const int col0 = col_tile + c * 32;
          if (l2) {
            // squared_l2 of the reference (kernels/bmm_helpers.cu:28-35) in GEMM form:
            // |a - b|^2 = |a|^2 + |b|^2 - 2 a.b, clamped at 0 against cancellation.
            const float* cn = epi.col_norms + static_cast<long long>(b) * shape.N + col0;
            if (col0 + 32 <= shape.N && (reinterpret_cast<uintptr_t>(cn) & 15) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                const float4 n4 = __ldg(reinterpret_cast<const float4*>(cn + j));
                v[j] = fmaxf(fmaf(-2.f, v[j], row_norm + n4.x), 0.f);
                v[j + 1] = fmaxf(fmaf(-2.f, v[j + 1], row_norm + n4.y), 0.f);
                v[j + 2] = fmaxf(fmaf(-2.f, v[j + 2], row_norm + n4.z), 0.f);
                v[j + 3] = fmaxf(fmaf(-2.f, v[j + 3], row_norm + n4.w), 0.f);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const float nj = (col0 + j < shape.N) ? __ldg(cn + j) : 0.f;
                v[j] = fmaxf(fmaf(-2.f, v[j], row_norm + nj), 0.f);
              }
            }
          }

          if (EPI == kEpiStore || EPI == kEpiMask) {
            const bool line_path = c_lines_ok && col0 + 32 <= shape.N && (EPI != kEpiMask || em_lines_ok);
            if (line_path) {
              // Whole warp (rows past M included: their lanes still carry the shuffles).
              // After the transpose lane q of each lane quad holds columns [8q, 8q+8) of
              // the quad's four rows, so masks are read and C is written 4 lanes per row.
              transpose_rows_in_lane_quads(v);
              const int q = static_cast<int>(lane & 3u);
              const int row_g = row_base(mb) + static_cast<int>(quarter) * 32 + static_cast<int>(lane & ~3u);
              float* cbase = epi.C + b * epi.stride_c + static_cast<long long>(row_g) * epi.ldc + col0 + 8 * q;
              if (EPI == kEpiMask) {
                // kernels/mbmm.cu:360-363 (8x8 tile skip) and :111-133 (element multiply);
                // the mask bytes (tmv, e8) were fetched one chunk ahead
#pragma unroll
                for (int i = 0; i < 4; ++i) {
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const uint32_t w = j < 4 ? e8[i].x : e8[i].y;
                    // byte -> float without the conversion unit: 0x4B0000bb is 2^23 + bb
                    const float ef = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540u | (j & 3))) - 8388608.0f;
                    v[8 * i + j] = tmv[i] != 0 ? v[8 * i + j] * ef : 0.f;
                  }
                }
              }
              if (kHalf) {
                // C has the operands' type: eight columns are one 16-byte store, four lanes
                // cover 64 contiguous bytes of a row
                uint16_t* cb16 = reinterpret_cast<uint16_t*>(epi.C) + b * epi.stride_c +
                                 static_cast<long long>(row_g) * epi.ldc + col0 + 8 * q;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  if (row_g + i < shape.M)
                    __stcs(reinterpret_cast<uint4*>(cb16 + static_cast<long long>(i) * epi.ldc),
                           make_uint4(pack_x16(v[8 * i], v[8 * i + 1], DT == 2), pack_x16(v[8 * i + 2], v[8 * i + 3], DT == 2),
                                      pack_x16(v[8 * i + 4], v[8 * i + 5], DT == 2), pack_x16(v[8 * i + 6], v[8 * i + 7], DT == 2)));
              } else {
#pragma unroll
              for (int i = 0; i < 4; ++i)
                if (row_g + i < shape.M)
                  st_global_v8_streaming(cbase + static_cast<long long>(i) * epi.ldc, v[8 * i], v[8 * i + 1],
                                         v[8 * i + 2], v[8 * i + 3], v[8 * i + 4], v[8 * i + 5], v[8 * i + 6],
                                         v[8 * i + 7]);
              }
            } else if (row_ok && col0 < shape.N) {
              // ragged right edge or storage that is not 32-byte friendly: one row per thread
              if (EPI == kEpiMask) {
                const unsigned char* tm = epi.thread_mask + b * epi.tm_stride +
                                          static_cast<long long>(row >> 3) * epi.tm_cols + (col0 >> 3);
                const unsigned char* em = epi.element_mask + b * epi.em_stride +
                                          static_cast<long long>(row) * shape.N + col0;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const bool tlive = (col0 + g * 8 < shape.N) ? (tm[g] != 0) : false;
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const int jj = g * 8 + j;
                    const float ef = (col0 + jj < shape.N) ? static_cast<float>(em[jj]) : 0.f;
                    v[jj] = tlive ? v[jj] * ef : 0.f;
                  }
                }
              }
              float* crow = epi.C + b * epi.stride_c + static_cast<long long>(row) * epi.ldc + col0;
              if (kHalf) {
                // 16-bit C: element-wise
                uint16_t* crow16 = reinterpret_cast<uint16_t*>(epi.C) + b * epi.stride_c +
                                   static_cast<long long>(row) * epi.ldc + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < shape.N) crow16[j] = round_x16(v[j], DT == 2);
              } else if (col0 + 32 <= shape.N && (reinterpret_cast<uintptr_t>(crow) & 15) == 0) {
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                  __stcs(reinterpret_cast<float4*>(crow + j), make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]));
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < shape.N) crow[j] = v[j];
              }
            }
          } else if (EPI == kEpiSoftmax) {
            // This thread's row, 32 columns; scores go to the exp2 domain, s = (a.b) * scale * log2(e),
            // and dropped entries to -inf, whose exponential is an exact 0.
#pragma unroll
            for (int j = 0; j < 32; ++j)
              v[j] = (ew[j >> 2] & (0xffu << ((j & 3) * 8))) != 0u ? v[j] * epi.softmax_scale_log2e : -INFINITY;
            if (sweep == 0) {
              if (any_kept != 0u) {
                // (trees, not chains: a warp or two per scheduler cannot hide a 32-deep dependency)
                float x[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) x[j] = fmaxf(v[j], v[j + 16]);
#pragma unroll
                for (int w = 8; w > 0; w >>= 1)
#pragma unroll
                  for (int j = 0; j < w; ++j) x[j] = fmaxf(x[j], x[j + w]);
                if (x[0] > sm_max) {
                  sm_sum *= ex2_approx(sm_max - x[0]);  // exp2(-inf) = 0 on the first kept chunk
                  sm_max = x[0];
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = ex2_approx(v[j] - sm_max);
#pragma unroll
                for (int w = 16; w > 0; w >>= 1)
#pragma unroll
                  for (int j = 0; j < w; ++j) v[j] += v[j + w];
                sm_sum += v[0];
              }
            } else {
              // (sm_max is finite here: a row that keeps nothing got 0 at the start of the sweep)
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = ex2_approx(v[j] - sm_max) * sm_inv;
              const bool line_path = c_lines_ok && col0 + 32 <= shape.N;
              if (line_path) {
                // whole warp: after the transpose lane q of a lane quad holds columns [8q, 8q + 8)
                // of the quad's four rows, and every store instruction writes eight whole lines
                transpose_rows_in_lane_quads(v);
                const int q = static_cast<int>(lane & 3u);
                const int row_g = row_base(mb) + static_cast<int>(quarter) * 32 + static_cast<int>(lane & ~3u);
                float* cbase = epi.C + b * epi.stride_c + static_cast<long long>(row_g) * epi.ldc + col0 + 8 * q;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  if (row_g + i < shape.M)
                    st_global_v8_streaming(cbase + static_cast<long long>(i) * epi.ldc, v[8 * i], v[8 * i + 1], v[8 * i + 2],
                                           v[8 * i + 3], v[8 * i + 4], v[8 * i + 5], v[8 * i + 6], v[8 * i + 7]);
              } else if (row_ok && col0 < shape.N) {
                float* crow = epi.C + b * epi.stride_c + static_cast<long long>(row) * epi.ldc + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (col0 + j < shape.N) crow[j] = v[j];
              }
            }
          } else if (EPI == kEpiMin) {
            // kernels/minbmm.cu:86-153 keeps the first index under a strict '<'. Here: the
            // chunk minimum by a comparison tree, then -- only when it beats the running
            // best -- the lowest column that holds it. Columns past N never compete.
            if (col0 + 32 > shape.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j >= shape.N) v[j] = INFINITY;
            }
            float m16[16], m8[8], m4[4];
#pragma unroll
            for (int j = 0; j < 16; ++j) m16[j] = fminf(v[2 * j], v[2 * j + 1]);
#pragma unroll
            for (int j = 0; j < 8; ++j) m8[j] = fminf(m16[2 * j], m16[2 * j + 1]);
#pragma unroll
            for (int j = 0; j < 4; ++j) m4[j] = fminf(m8[2 * j], m8[2 * j + 1]);
            const float m = fminf(fminf(m4[0], m4[1]), fminf(m4[2], m4[3]));
            if (m < best) {
              best = m;
              int jj = 0;
#pragma unroll
              for (int j = 31; j >= 0; --j)
                if (v[j] == m) jj = j;
              best_col = col0 + jj;
            }
          } else {
            // top-k: only values that beat the row's current k-th best are staged; the
            // stage is merged into the row's list before it can overflow. Groups of 8
            // columns in which no row of the warp has a candidate are skipped outright
            // (a threshold raised by a merge inside the chunk only makes the group test
            // conservative: the values themselves are compared with the current one).
            constexpr int kSlotStride = kTileM * 8;
            if (col0 + 32 > shape.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (col0 + j >= shape.N) v[j] = -INFINITY;  // never greater than a threshold
            }
            // which groups of 8 columns hold, in any row of the warp, a value above that row's
            // threshold: one OR-reduction over the warp answers for all four groups
            uint32_t mine = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int j0 = 8 * g;
              const float mx = fmaxf(fmaxf(fmaxf(v[j0], v[j0 + 1]), fmaxf(v[j0 + 2], v[j0 + 3])),
                                     fmaxf(fmaxf(v[j0 + 4], v[j0 + 5]), fmaxf(v[j0 + 6], v[j0 + 7])));
              mine |= (mx > thr ? 1u : 0u) << g;
            }
            const uint32_t groups = __reduce_or_sync(0xffffffffu, mine);
            if (groups != 0) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if ((groups >> g) & 1u) {  // warp-uniform
                  const int j0 = 8 * g;
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const uint32_t hit = v[j0 + j] > thr ? 1u : 0u;
                    topk_stage_if(hit, stg_slot, v[j0 + j], col0 + j0 + j);
                    stg_slot += hit * kSlotStride;
                  }
                  // at most 8 slots were taken since the last check: merge while 8 are still free
                  const int n_staged = static_cast<int>(stg_slot - stg_base) / kSlotStride;
                  const bool full = n_staged > static_cast<int>(kTopkStageSlots) - 8;
                  if (__any_sync(0xffffffffu, full)) {
                    // every lane merges what its row has staged: the call costs the same for
                    // one row as for 32
                    FBMM_PROF_MARK(2, 3, 1);
                    const float kth = topk_merge_own_rows<TOPK_E>(has_list, n_staged, sv, si, epi.k, stg + row_in_tile);
                    FBMM_PROF_MARK_END(2);
                    if (row_ok) thr = kth;
                    stg_slot = stg_base;
                    has_list = true;
                  }
                }
              }
            }
          }
          FBMM_PROF_XEND(1);
        }
        FBMM_PROF_END(1);
        FBMM_TRACE_TAG(3, 5);
        if (threadIdx.x == 192) { FBMM_TRACE(1); }
        if (++acc_stage == kAccStages) { acc_stage = 0; acc_phase ^= 1u; }
        if (mask_tma && ++mstage == kMaskStages) { mstage = 0; mphase ^= 1u; }
        if (DUAL && rb == 1) {
          float tf = best; best = best_o; best_o = tf;
          int ti = best_col; best_col = best_col_o; best_col_o = ti;
          tf = row_norm; row_norm = row_norm_o; row_norm_o = tf;
        }
      }  // row blocks
      }
      }  // sweeps

      // ---- unit end
      if (EPI == kEpiMin) {
        if (row_ok && ok) {
          const float bz = best + 0.0f;  // -0 -> +0 so equal values share one key
          const unsigned long long key =
              (static_cast<unsigned long long>(float_to_ordered(bz)) << 32) | static_cast<uint32_t>(best_col);
          atomicMin(epi.keys + static_cast<long long>(b) * shape.M + row, key);
        }
        if (DUAL && row_ok_o && ok) {
          const float bz = best_o + 0.0f;
          const unsigned long long key =
              (static_cast<unsigned long long>(float_to_ordered(bz)) << 32) | static_cast<uint32_t>(best_col_o);
          atomicMin(epi.keys + static_cast<long long>(b) * shape.M + row + kTileM, key);
        }
      } else if (EPI == kEpiTopk) {
        if (ok) {
          const int n_staged = static_cast<int>(stg_slot - stg_base) / (kTileM * 8);
          if (__any_sync(0xffffffffu, n_staged > 0) || !has_list)
            topk_merge_own_rows<TOPK_E>(has_list, n_staged, sv, si, epi.k, stg + row_in_tile);
          __syncwarp();
          const int rows_valid = min(32, shape.M - (row_base(mb) + static_cast<int>(quarter) * 32));
          topk_write_out(sv, si, epi.k, epi.index_offset, lv0, li0, lp0, rows_valid, stg_w);
        }
      }
    }
    if (threadIdx.x == 6 * 32) { FBMM_PROF_FLUSH(12); FBMM_PROF_XFLUSH(); }
  } else {
    // ------------------------------------------------------------------ resident A loader
    if (A_RES && lane == 0) {
      uint32_t a_phase = 0;
      bool ok = true;
      for (long long u = unit_first; u < units && ok; u += unit_step) {
        int b, mb, t0, t1, first, last;
        decode(u, b, mb, t0, t1);
        if (!live_range( b, mb, t0, t1, first, last)) continue;
        for (int slot = 0; slot < kblocks * kRb && ok; ++slot) {  // slot = row block * kblocks + k-block
          const int rb = slot / kblocks, kb = slot - rb * kblocks;
          // free as soon as the previous unit's last tile has finished with that k-block
          ok = wait_gate(&bars->a_empty[slot], a_phase ^ 1u);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars->a_full[slot], kPlaneBytes);
          load_a(&tmap_a, a_region + slot * kPlanes * kPlaneBytes + off_a_hi, &bars->a_full[slot], false, kb, mb, b,
                 rb * kTileM);
        }
        a_phase ^= 1u;
      }
      if (!ok) {
        const long long t0c = clock64();
        while (clock64() - t0c < 2000000LL) {}
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tcgen05_fence_before_sync();
  // a pair leaves together: the issuer reads the peer's shared memory and signals its barriers
  if (PAIR) cluster_sync_all(); else __syncthreads();
  if (threadIdx.x == 0 && *abort_flag != 0) atomicOr(&g_fbmm_status[0], 1u);
  if (warp == 1) {
    tcgen05_fence_after_sync();
    if (PAIR) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// lo plane of a whole operand: lo[i] = x[i] - tf32(x[i]) over `count` floats (both pointers
// 16-byte aligned; the last count % 4 floats are handled one by one).
__global__ void fbmm_split_lo_kernel(const float* __restrict__ src, float* __restrict__ lo, long long count) {
  const long long count4 = count >> 2;
  const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const float4* src4 = reinterpret_cast<const float4*>(src);
  float4* lo4 = reinterpret_cast<float4*>(lo);
  for (long long i = tid; i < count4; i += stride) {
    const float4 x = src4[i];
    lo4[i] = make_float4(split_lo(x.x), split_lo(x.y), split_lo(x.z), split_lo(x.w));
  }
  if (tid < (count & 3)) lo[4 * count4 + tid] = split_lo(src[4 * count4 + tid]);
}

// hi and lo planes of an operand stored [l][k][n] (n contiguous, pitch `ld`), written
// transposed as [l][n][kp] (k contiguous, kp >= K a multiple of 4, zero beyond K): hi is a
// copy, lo = x - tf32(x). A column tile of a very wide operand then is one contiguous piece
// of memory instead of K pieces a whole row of the operand apart. Block 32 x 8, tile 32 x 32.
__global__ void fbmm_split_transpose_kernel(const float* __restrict__ src, float* __restrict__ hi,
                                            float* __restrict__ lo, int K, int N, int kp, long long ld, long long stride) {
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const long long l = blockIdx.z;
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int k = k0 + j, n = n0 + static_cast<int>(threadIdx.x);
    tile[j][threadIdx.x] = (k < K && n < N) ? src[l * stride + static_cast<long long>(k) * ld + n] : 0.f;
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    const int n = n0 + j, k = k0 + static_cast<int>(threadIdx.x);
    if (n < N && k < kp) {
      const float x = tile[threadIdx.x][j];
      const long long at = (l * N + n) * kp + k;
      hi[at] = x;
      lo[at] = split_lo(x);
    }
  }
}

// Squared norms of the rows of an operand: out[l][r] = sum_k x[l][r][k]^2. `ld` is the pitch
// of the stored rows; mn_major != 0 means the storage runs along r (element (r, k) at
// k * ld + r), else along k (r * ld + k). One warp per row for k-contiguous storage, one
// thread per row otherwise; both read coalesced.
__global__ void fbmm_sqnorm_kernel(const float* __restrict__ x, float* __restrict__ out, int L, int rows, int K,
                                   long long ld, long long stride, int mn_major) {
  const long long total = static_cast<long long>(L) * rows;
  if (mn_major) {
    const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float* p = x + (i / rows) * stride + (i % rows);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const float a = p[static_cast<long long>(k) * ld];
      acc = fmaf(a, a, acc);
    }
    out[i] = acc;
  } else {
    const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    if (i >= total) return;  // whole warps leave together
    const float* p = x + (i / rows) * stride + (i % rows) * ld;
    float acc = 0.f;
    for (int k = static_cast<int>(lane_id()); k < K; k += 32) {
      const float a = p[k];
      acc = fmaf(a, a, acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane_id() == 0) out[i] = acc;
  }
}

// The same for k-contiguous fp16 (bf16 == 0) or bf16 rows, one warp per row, fp32 sums.
__global__ void fbmm_sqnorm_x16_kernel(const uint16_t* __restrict__ x, float* __restrict__ out, int L, int rows, int K,
                                       long long ld, long long stride, int bf16) {
  const long long total = static_cast<long long>(L) * rows;
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (i >= total) return;  // whole warps leave together
  const uint16_t* p = x + (i / rows) * stride + (i % rows) * ld;
  float acc = 0.f;
  for (int k = static_cast<int>(lane_id()); k < K; k += 32) {
    const uint16_t raw = p[k];
    const float a = bf16 ? __uint_as_float(static_cast<uint32_t>(raw) << 16) : __half2float(__ushort_as_half(raw));
    acc = fmaf(a, a, acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane_id() == 0) out[i] = acc;
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

// k-means centroid update, the step after min_bmm with the l2 distance has assigned every
// point to its nearest centroid: sums[c][:] += X[i][:] and counts[c] += 1 for c = assign[i]
// (integer counts: exact for any number of points).
// One warp per point; the additions are fire-and-forget reductions that resolve in L2,
// where the k x d sums live. Summation order, and with it the last bits of the result,
// varies from run to run. Points with an assignment outside [0, k) are skipped.
__global__ void fbmm_kmeans_accumulate_kernel(const float* __restrict__ x, long long ldx,
                                              const long long* __restrict__ assign, long long n, int d, int k,
                                              float* __restrict__ sums, unsigned int* __restrict__ counts) {
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x & 31u);
  for (long long i = warp; i < n; i += warps) {
    const long long c = assign[i];
    if (c < 0 || c >= k) continue;
    const float* row = x + i * ldx;
    float* dst = sums + c * d;
    for (int j = lane; j < d; j += 32) atomicAdd(dst + j, row[j]);
    if (lane == 0) atomicAdd(counts + c, 1u);
  }
}

// The same with the k x d sums and the k counts of a CTA's points first gathered in shared
// memory (dynamic: (k * d + k) floats) and added to the global ones once at the end. With
// few clusters every point of the plain kernel lands on the same few lines in L2; here the
// contended additions stay on chip.
__global__ void fbmm_kmeans_accumulate_smem_kernel(const float* __restrict__ x, long long ldx,
                                                   const long long* __restrict__ assign, long long n, int d, int k,
                                                   float* __restrict__ sums, unsigned int* __restrict__ counts) {
  extern __shared__ float part[];  // [k * d] sums, then [k] counts (unsigned int, all-zero bits = 0 either way)
  unsigned int* part_counts = reinterpret_cast<unsigned int*>(part + k * d);
  const int cells = k * d + k;
  for (int i = threadIdx.x; i < cells; i += blockDim.x) part[i] = 0.f;
  __syncthreads();
  const long long warp = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long warps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x & 31u);
  for (long long i = warp; i < n; i += warps) {
    const long long c = assign[i];
    if (c < 0 || c >= k) continue;
    const float* row = x + i * ldx;
    float* dst = part + c * d;
    for (int j = lane; j < d; j += 32) atomicAdd(dst + j, row[j]);
    if (lane == 0) atomicAdd(part_counts + c, 1u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < k * d; i += blockDim.x) {
    const float v = part[i];
    if (v != 0.f) atomicAdd(sums + i, v);
  }
  for (int i = threadIdx.x; i < k; i += blockDim.x) {
    const unsigned int c = part_counts[i];
    if (c != 0u) atomicAdd(counts + i, c);
  }
}

// centroids[c][:] = sums[c][:] / counts[c]; a centroid no point chose keeps its old place.
// counts_out (or null) receives the cluster sizes as fp32.
__global__ void fbmm_kmeans_finalize_kernel(const float* __restrict__ sums, const unsigned int* __restrict__ counts,
                                            float* __restrict__ centroids, long long ldc, int d, long long total,
                                            float* __restrict__ counts_out) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long c = i / d;
  const int j = static_cast<int>(i - c * d);
  const unsigned int cnt = counts[c];
  if (cnt > 0u) centroids[c * ldc + j] = sums[i] / static_cast<float>(cnt);
  if (j == 0 && counts_out != nullptr) counts_out[c] = static_cast<float>(cnt);
}

}  // namespace fbmm

// Row-wise min / top-k of the l1 distance matrix D[m, n] = sum_k |A[m, k] - B[k, n]| without
// writing D: the reference's `distance="l1"` mode (kernels/bmm_helpers.cu:46-52 substituted for
// __DISTANCE_FN__ in kernels/minbmm.cu and kernels/topkbmm.cu; chosen in minbmm.py:16-17 and
// topkbmm.py:19-20).
//
// |a - b| has no matrix-product form, so this mode cannot use the tensor cores: it is a plain
// SIMT tile kernel (fp32 pipes: one subtract and one add of the absolute value per term), and the
// B200 parts of the library it shares are the epilogues. A CTA of 256 threads walks units
// (batch, 128-row block, run of column tiles) like the tensor-core kernel does. Per column tile:
//   * A and B tiles of 16 k each go through shared memory, k-major ([k][row], rows padded to 132
//     floats), fetched one k-block ahead into registers;
//   * thread (ty, tx) of the 16 x 16 grid accumulates rows {4 ty + i, 64 + 4 ty + i} x columns
//     {4 tx + j, 64 + 4 tx + j} (8 x 8 outputs; both operand reads are float4 and free of bank
//     conflicts);
//   * min: every thread keeps, for each of its 8 rows, the best of its own columns over the whole
//     unit (ascending columns and a strict '<' keep the first index, kernels/minbmm.cu:86-153);
//     at unit end the 16 threads of a row combine by shuffles (ties to the lower column) and one
//     of them issues the same packed 64-bit atomicMin as the tensor-core kernel;
//   * top-k: the tile is parked in shared memory ([row][132]) and the first four warps take over
//     as row owners, thread = row, exactly as the tensor-core epilogue reads TMEM: threshold
//     filter, predicated staging, every lane merging its own row's list (topk_merge_own_rows),
//     lists written out at unit end (topk_write_out) -- values only go where those routines put
//     them, so the outputs, the packed wire format and the chunk merge are shared.
// K tails are zero-filled in both operands (|0 - 0| adds nothing); columns past N never compete.
#pragma once
#include "fbmm_kernel.cuh"

namespace fbmm {

struct L1Operand {
  const float* ptr;
  long long ld, stride;  // pitch of stored rows and batch stride, in elements (stride 0: shared by all batches)
  int mn_major;          // 1: contiguous along M / N, 0: along K
  int rows;              // M or N
};

constexpr int kL1KBlock = 16;
constexpr int kL1Pitch = kTileM + 4;  // floats per k-row of an operand tile, and per row of the parked tile
constexpr int kL1Threads = 256;
constexpr uint32_t kL1OperandBytes = 2u * kL1KBlock * kL1Pitch * 4u;
constexpr uint32_t kL1TileBytes = kTileM * kL1Pitch * 4u;
__host__ __device__ constexpr uint32_t l1_smem_bytes(int epi) {
  return kL1OperandBytes + (epi == kEpiTopk ? kL1TileBytes + kTopkStageBytes : 0u) + 16u;
}

// This thread's share of one 128 x 16 operand tile, fetched into registers: rows row0 .. row0 + 127
// of the operand, k0 .. k0 + 15. Out-of-range rows and k read as zero.
struct L1Fetch {
  float4 v[2];
};
__device__ __forceinline__ L1Fetch l1_fetch(const L1Operand& op, const float* base, int row0, int k0, int K, int t) {
  L1Fetch f;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (op.mn_major) {
      // rows are contiguous: 32 lanes x 4 rows, k = t / 32 (+ 8)
      const int k = k0 + (t >> 5) + 8 * h;
      const int r = row0 + (t & 31) * 4;
      if (k < K) {
        const float* p = base + static_cast<long long>(k) * op.ld + r;
        if (r + 3 < op.rows) {
          const float4 q = *reinterpret_cast<const float4*>(p);
          x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (r + i < op.rows) x[i] = p[i];
        }
      }
    } else {
      // k is contiguous: 4 lanes x 4 k per row, row = t / 4 (+ 64)
      const int r = row0 + (t >> 2) + 64 * h;
      const int k = k0 + (t & 3) * 4;
      if (r < op.rows) {
        const float* p = base + static_cast<long long>(r) * op.ld + k;
        if (k + 3 < K) {
          const float4 q = *reinterpret_cast<const float4*>(p);
          x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (k + i < K) x[i] = p[i];
        }
      }
    }
    f.v[h] = make_float4(x[0], x[1], x[2], x[3]);
  }
  return f;
}
// ... and parked in the shared-memory tile [k][kL1Pitch].
__device__ __forceinline__ void l1_park(const L1Operand& op, const L1Fetch& f, float* tile, int t) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (op.mn_major) {
      *reinterpret_cast<float4*>(tile + ((t >> 5) + 8 * h) * kL1Pitch + (t & 31) * 4) = f.v[h];
    } else {
      float* p = tile + ((t & 3) * 4) * kL1Pitch + (t >> 2) + 64 * h;
      p[0] = f.v[h].x;
      p[kL1Pitch] = f.v[h].y;
      p[2 * kL1Pitch] = f.v[h].z;
      p[3 * kL1Pitch] = f.v[h].w;
    }
  }
}

template <int EPI, int TOPK_E>
__global__ void __launch_bounds__(kL1Threads, EPI == kEpiTopk ? 1 : 2)
fbmm_l1_kernel(const L1Operand opa, const L1Operand opb, const GemmShape shape, const EpiArgs epi) {
  static_assert(EPI == kEpiMin || EPI == kEpiTopk, "the l1 mode has the reducing epilogues only");
  extern __shared__ __align__(16) uint8_t l1_smem[];
  float* As = reinterpret_cast<float*>(l1_smem);
  float* Bs = As + kL1KBlock * kL1Pitch;
  float* Cs = reinterpret_cast<float*>(l1_smem + kL1OperandBytes);           // top-k: the parked tile
  int2* stg = reinterpret_cast<int2*>(l1_smem + kL1OperandBytes + kL1TileBytes);  // top-k: staging slots

  const int t = static_cast<int>(threadIdx.x);
  const int tx = t & 15, ty = t >> 4;
  const uint32_t lane = lane_id();
  const int warp = t >> 5;

  for (long long u = blockIdx.x; u < shape.num_units; u += gridDim.x) {
    // unit -> batch, row block, column tiles (as in the tensor-core kernel)
    const long long row_blocks = static_cast<long long>(shape.L) * shape.m_blocks;
    const int chunk = static_cast<int>(shape.chunk_major ? u / row_blocks : u % shape.n_chunks);
    const long long rb = shape.chunk_major ? u % row_blocks : u / shape.n_chunks;
    const int mb = static_cast<int>(rb % shape.m_blocks);
    const int b = static_cast<int>(rb / shape.m_blocks);
    const int t0 = chunk * shape.tiles_per_chunk;
    const int t1 = min(shape.n_tiles, t0 + shape.tiles_per_chunk);
    const int row0 = mb * kTileM;
    const float* a_base = opa.ptr + static_cast<long long>(b) * opa.stride;
    const float* b_base = opb.ptr + static_cast<long long>(b) * opb.stride;

    // ---- per-unit reduction state
    // min: best (value, column) of this thread's own columns for each of its 8 rows
    float best[8];
    int best_col[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { best[i] = INFINITY; best_col[i] = t0 * kTileN; }
    // top-k (row owners, threads 0..127): as the tensor-core epilogue keeps it
    const int row_in_tile = t;  // owners only
    const bool owner = EPI == kEpiTopk && t < kTileM;
    const bool row_ok = row0 + row_in_tile < shape.M;
    float thr = (owner && row_ok) ? -INFINITY : INFINITY;
    const uint32_t stg_base = smem_u32(stg + (owner ? row_in_tile : 0));
    uint32_t stg_slot = stg_base;
    bool has_list = false;
    float* sv = nullptr;
    int* si = nullptr;
    if (owner) {
      constexpr long long kListEntries = 32ll * TOPK_E * kTileM;
      sv = epi.topk_scratch + static_cast<long long>(blockIdx.x) * 2 * kListEntries + row_in_tile;
      si = reinterpret_cast<int*>(sv + kListEntries);
    }

    for (int tile = t0; tile < t1; ++tile) {
      const int col0 = tile * kTileN;
      float acc[8][8];
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

      L1Fetch fa = l1_fetch(opa, a_base, row0, 0, shape.K, t);
      L1Fetch fb = l1_fetch(opb, b_base, col0, 0, shape.K, t);
      for (int k0 = 0; k0 < shape.K; k0 += kL1KBlock) {
        __syncthreads();  // everyone is done with the tiles of the k-block before
        l1_park(opa, fa, As, t);
        l1_park(opb, fb, Bs, t);
        __syncthreads();
        if (k0 + kL1KBlock < shape.K) {
          fa = l1_fetch(opa, a_base, row0, k0 + kL1KBlock, shape.K, t);
          fb = l1_fetch(opb, b_base, col0, k0 + kL1KBlock, shape.K, t);
        }
#pragma unroll
        for (int k = 0; k < kL1KBlock; ++k) {
          const float4 a0 = *reinterpret_cast<const float4*>(As + k * kL1Pitch + 4 * ty);
          const float4 a1 = *reinterpret_cast<const float4*>(As + k * kL1Pitch + 64 + 4 * ty);
          const float4 b0 = *reinterpret_cast<const float4*>(Bs + k * kL1Pitch + 4 * tx);
          const float4 b1 = *reinterpret_cast<const float4*>(Bs + k * kL1Pitch + 64 + 4 * tx);
          const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
          const float bb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] += fabsf(a[i] - bb[j]);  // kernels/bmm_helpers.cu:46-52
        }
      }

      if (EPI == kEpiMin) {
        // this thread's columns in ascending order: 4 tx + j, then 64 + 4 tx + j
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int col = col0 + (j < 4 ? 4 * tx + j : 64 + 4 * tx + (j - 4));
            if (col < shape.N && acc[i][j] < best[i]) { best[i] = acc[i][j]; best_col[i] = col; }
          }
        }
      } else {
        // park the tile, rows as the owners will read them
        __syncthreads();  // (the owners may still be reading the tile before)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i < 4 ? 4 * ty + i : 64 + 4 * ty + (i - 4);
          *reinterpret_cast<float4*>(Cs + r * kL1Pitch + 4 * tx) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
          *reinterpret_cast<float4*>(Cs + r * kL1Pitch + 64 + 4 * tx) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
        }
        __syncthreads();
        if (owner) {
          // the tensor-core kernel's top-k epilogue, fed from shared memory instead of TMEM
          constexpr int kSlotStride = kTileM * 8;
          for (int c = 0; c < kTileN / 32; ++c) {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const float4 q = *reinterpret_cast<const float4*>(Cs + row_in_tile * kL1Pitch + c * 32 + j);
              v[j] = q.x; v[j + 1] = q.y; v[j + 2] = q.z; v[j + 3] = q.w;
            }
            const int cc0 = col0 + c * 32;
            if (cc0 + 32 > shape.N) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (cc0 + j >= shape.N) v[j] = -INFINITY;
            }
            uint32_t mine = 0;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int j0 = 8 * g;
              const float mx = fmaxf(fmaxf(fmaxf(v[j0], v[j0 + 1]), fmaxf(v[j0 + 2], v[j0 + 3])),
                                     fmaxf(fmaxf(v[j0 + 4], v[j0 + 5]), fmaxf(v[j0 + 6], v[j0 + 7])));
              mine |= (mx > thr ? 1u : 0u) << g;
            }
            const uint32_t groups = __reduce_or_sync(0xffffffffu, mine);
            if (groups == 0) continue;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              if ((groups >> g) & 1u) {  // warp-uniform
                const int j0 = 8 * g;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const uint32_t hit = v[j0 + j] > thr ? 1u : 0u;
                  topk_stage_if(hit, stg_slot, v[j0 + j], cc0 + j0 + j);
                  stg_slot += hit * kSlotStride;
                }
                const int n_staged = static_cast<int>(stg_slot - stg_base) / kSlotStride;
                const bool full = n_staged > static_cast<int>(kTopkStageSlots) - 8;
                if (__any_sync(0xffffffffu, full)) {
                  const float kth = topk_merge_own_rows<TOPK_E>(has_list, n_staged, sv, si, epi.k, stg + row_in_tile);
                  if (row_ok) thr = kth;
                  stg_slot = stg_base;
                  has_list = true;
                }
              }
            }
          }
        }
      }
    }

    // ---- unit end
    if (EPI == kEpiMin) {
      // the 16 threads of a row (same ty: one half of a warp) combine; ties go to the lower column
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float v = best[i];
        int c = best_col[i];
#pragma unroll
        for (int w = 8; w > 0; w >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, v, w);
          const int oc = __shfl_xor_sync(0xffffffffu, c, w);
          if (ov < v || (ov == v && oc < c)) { v = ov; c = oc; }
        }
        const int row = row0 + (i < 4 ? 4 * ty + i : 64 + 4 * ty + (i - 4));
        if (tx == 0 && row < shape.M) {
          const float bz = v + 0.0f;  // -0 -> +0 so equal values share one key
          const unsigned long long key =
              (static_cast<unsigned long long>(float_to_ordered(bz)) << 32) | static_cast<uint32_t>(c);
          atomicMin(epi.keys + static_cast<long long>(b) * shape.M + row, key);
        }
      }
    } else if (owner) {
      const int n_staged = static_cast<int>(stg_slot - stg_base) / (kTileM * 8);
      if (__any_sync(0xffffffffu, n_staged > 0) || !has_list)
        topk_merge_own_rows<TOPK_E>(has_list, n_staged, sv, si, epi.k, stg + row_in_tile);
      __syncwarp();
      const long long warp_row0 = (shape.tiles_per_chunk > 0 ? (t0 / shape.tiles_per_chunk) : 0) * epi.topk_chunk_rows +
                                  static_cast<long long>(b) * shape.M + row0 + warp * 32;
      const bool packed_out = epi.topk_packed != nullptr;
      float* lv0 = !packed_out ? epi.topk_values + warp_row0 * epi.k : nullptr;
      long long* li0 = !packed_out ? epi.topk_indices + warp_row0 * epi.k : nullptr;
      int2* lp0 = packed_out ? epi.topk_packed + warp_row0 * epi.k : nullptr;
      const int rows_valid = max(0, min(32, shape.M - (row0 + warp * 32)));
      topk_write_out(sv, si, epi.k, epi.index_offset, lv0, li0, lp0, rows_valid, stg + warp * 32);
    }
    (void)lane;
  }
}

}  // namespace fbmm

// Host side of libfbmm.so: argument validation, tensor-map construction, work
// decomposition and launches behind the C ABI declared in include/fbmm.h.
#include <algorithm>
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/fbmm.h"
#include "fbmm_kernel.cuh"
#include "fbmm_l1_kernel.cuh"

namespace {

using namespace fbmm;

thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define FBMM_CUDA(call)                                                                   \
  do {                                                                                    \
    cudaError_t e_ = (call);                                                              \
    if (e_ != cudaSuccess) return fail(FBMM_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); \
  } while (0)

// ---------------------------------------------------------------------------------------
// per-device state
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

constexpr int kMaxDevices = 64;
struct DeviceState {
  bool ready = false;
  int sms = 0;
};
std::mutex g_mu;
DeviceState g_dev[kMaxDevices];
EncodeTiledFn g_encode = nullptr;

template <int EPI, int E, bool AR, bool PS, bool PR = false>
int set_one_attr() {
  FBMM_CUDA(cudaFuncSetAttribute(fbmm_gemm_kernel<EPI, E, AR, PS, 0, PR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSmemLimit)));
  return FBMM_OK;
}

template <int EPI, int E>
int set_smem_attr() {
  int rc;
  if ((rc = set_one_attr<EPI, E, false, false>()) != FBMM_OK) return rc;
  if ((rc = set_one_attr<EPI, E, true, false>()) != FBMM_OK) return rc;
  if (EPI == kEpiMin || EPI == kEpiTopk) {
    constexpr bool kPs = (EPI == kEpiMin || EPI == kEpiTopk);
    if ((rc = set_one_attr<EPI, E, false, kPs>()) != FBMM_OK) return rc;
    if ((rc = set_one_attr<EPI, E, true, kPs>()) != FBMM_OK) return rc;
    if ((rc = set_one_attr<EPI, E, false, kPs, kPs>()) != FBMM_OK) return rc;
    if ((rc = set_one_attr<EPI, E, true, kPs, kPs>()) != FBMM_OK) return rc;
  }
  if (EPI == kEpiMin) {
    constexpr bool kMin = EPI == kEpiMin;
    FBMM_CUDA(cudaFuncSetAttribute(fbmm_gemm_kernel<EPI, E, true, kMin, 0, false, kMin>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemLimit)));
  }
  return FBMM_OK;
}

int device_state(DeviceState** out) {
  int dev = 0;
  FBMM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FBMM_ERR_INVALID, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& st = g_dev[dev];
  if (!st.ready) {
    cudaDeviceProp prop;
    FBMM_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
      return fail(FBMM_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                  prop.major, prop.minor);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      FBMM_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
      if (fn == nullptr) return fail(FBMM_ERR_CUDA, "cuTensorMapEncodeTiled not available");
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    int rc;
    if ((rc = set_smem_attr<kEpiStore, 1>()) != FBMM_OK) return rc;
    if ((rc = set_smem_attr<kEpiMask, 1>()) != FBMM_OK) return rc;
    if ((rc = set_smem_attr<kEpiSoftmax, 1>()) != FBMM_OK) return rc;
    if ((rc = set_smem_attr<kEpiMin, 1>()) != FBMM_OK) return rc;
    if ((rc = set_smem_attr<kEpiTopk, 1>()) != FBMM_OK) return rc;
    if ((rc = set_smem_attr<kEpiTopk, 2>()) != FBMM_OK) return rc;
    if ((rc = set_smem_attr<kEpiTopk, 4>()) != FBMM_OK) return rc;
    st.sms = prop.multiProcessorCount;
    st.ready = true;
  }
  *out = &st;
  return FBMM_OK;
}

// SM count for the workspace queries; falls back to the B200 figure when no device can
// be asked (the queries must work on a machine without a GPU).
int sm_count_or_default() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 148; }
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
    cudaGetLastError();
    return 148;
  }
  return sms;
}

// ---------------------------------------------------------------------------------------
// operands
// ---------------------------------------------------------------------------------------
struct Operand {
  const float* ptr;
  bool mn_major;     // contiguous along M/N (true) or along K (false)
  long long ld;      // pitch of stored rows (elements)
  long long stride;  // batch stride (elements)
  int rows;          // M or N
};

int check_operand(const char* name, const Operand& op, int k, int l) {
  if (op.ptr == nullptr) return fail(FBMM_ERR_INVALID, "%s is null", name);
  const long long inner = op.mn_major ? op.rows : k;
  if (op.ld < inner) return fail(FBMM_ERR_INVALID, "%s pitch %lld smaller than its row length %lld", name, op.ld, inner);
  if ((reinterpret_cast<uintptr_t>(op.ptr) & 15u) != 0) return fail(FBMM_ERR_ALIGN, "%s is not 16-byte aligned", name);
  if ((op.ld & 3) != 0) return fail(FBMM_ERR_ALIGN, "%s pitch %lld is not a multiple of 4 elements", name, op.ld);
  if (l > 1 && (op.stride & 3) != 0)
    return fail(FBMM_ERR_ALIGN, "%s batch stride %lld is not a multiple of 4 elements", name, op.stride);
  if (l > 1 && op.stride < 0) return fail(FBMM_ERR_INVALID, "%s batch stride is negative", name);
  // a batch stride of 0 with l > 1 is a broadcast: one matrix serves every batch
  return FBMM_OK;
}

bool is_broadcast(const Operand& op, int l) { return l > 1 && op.stride == 0; }

// 3-D tiled tensor map over one operand. K-major: dims (k, rows, l), box (32, box_rows, 1),
// 128-byte swizzle. MN-major: dims (rows, k, l), box (32, 32, 1), 128-byte swizzle with
// 32-byte atoms (the only MN-major layout tcgen05 takes for tf32). A broadcast operand
// (batch stride 0) is described as a single batch; the kernel then asks for batch 0 only.
//
// Encoding a map costs a driver call, and a serving loop calls with the same buffers over
// and over, so the last few maps are kept, keyed by everything that goes into them.
struct TensorMapKey {
  const void* ptr;
  long long ld, stride;
  int rows, k, l, box_rows, kind;  // kind: 0 fp32 K-major, 1 fp32 MN-major, 2 fp16, 3 bf16
  bool operator==(const TensorMapKey& o) const {
    return ptr == o.ptr && ld == o.ld && stride == o.stride && rows == o.rows && k == o.k && l == o.l &&
           box_rows == o.box_rows && kind == o.kind;
  }
};
constexpr int kTensorMapCacheSize = 32;
struct TensorMapCache {
  TensorMapKey keys[kTensorMapCacheSize];
  CUtensorMap maps[kTensorMapCacheSize];
  int used = 0, next = 0;
  unsigned long long hits = 0, misses = 0;
};
std::mutex g_tm_mu;
TensorMapCache g_tm_cache;

bool tensor_map_lookup(const TensorMapKey& key, CUtensorMap* out) {
  std::lock_guard<std::mutex> lock(g_tm_mu);
  for (int i = 0; i < g_tm_cache.used; ++i)
    if (g_tm_cache.keys[i] == key) {
      *out = g_tm_cache.maps[i];
      ++g_tm_cache.hits;
      return true;
    }
  ++g_tm_cache.misses;
  return false;
}
void tensor_map_remember(const TensorMapKey& key, const CUtensorMap& map) {
  std::lock_guard<std::mutex> lock(g_tm_mu);
  const int at = g_tm_cache.next;
  g_tm_cache.keys[at] = key;
  g_tm_cache.maps[at] = map;
  g_tm_cache.next = (at + 1) % kTensorMapCacheSize;
  if (g_tm_cache.used < kTensorMapCacheSize) ++g_tm_cache.used;
}

int make_tensor_map(CUtensorMap* map, const Operand& op, int k, int l, int box_rows) {
  const TensorMapKey key{op.ptr, op.ld, l > 1 ? op.stride : 0, op.rows, k, l, box_rows, op.mn_major ? 1 : 0};
  if (tensor_map_lookup(key, map)) return FBMM_OK;
  cuuint64_t dims[3];
  cuuint32_t box[3];
  if (op.mn_major) {
    dims[0] = static_cast<cuuint64_t>(op.rows);
    dims[1] = static_cast<cuuint64_t>(k);
    box[0] = 32; box[1] = 32;
  } else {
    dims[0] = static_cast<cuuint64_t>(k);
    dims[1] = static_cast<cuuint64_t>(op.rows);
    box[0] = 32; box[1] = static_cast<cuuint32_t>(box_rows);
  }
  const bool one_batch = l == 1 || is_broadcast(op, l);
  dims[2] = one_batch ? 1u : static_cast<cuuint64_t>(l);
  box[2] = 1;
  const cuuint64_t pitch_bytes = static_cast<cuuint64_t>(op.ld) * 4u;
  cuuint64_t strides[2] = {pitch_bytes, one_batch ? pitch_bytes * dims[1] : static_cast<cuuint64_t>(op.stride) * 4u};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(op.ptr), dims, strides,
                              box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              op.mn_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FBMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  tensor_map_remember(key, *map);
  return FBMM_OK;
}

// Tensor map over a uint8 mask [l or 1][rows][cols] (cols contiguous), box (box_cols, box_rows, 1),
// no swizzle. cols must be a multiple of 16 and the base 16-byte aligned.
int make_mask_map(CUtensorMap* map, const unsigned char* ptr, int rows, int cols, int l, bool shared, int box_rows,
                  int box_cols) {
  const TensorMapKey key{ptr, cols, shared ? 0 : static_cast<long long>(rows) * cols, rows, box_cols, l, box_rows, 4};
  if (tensor_map_lookup(key, map)) return FBMM_OK;
  const bool one_batch = shared || l == 1;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), one_batch ? 1u : static_cast<cuuint64_t>(l)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows) * static_cast<cuuint64_t>(cols)};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<unsigned char*>(ptr), dims, strides, box,
                              elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FBMM_ERR_CUDA, "cuTensorMapEncodeTiled (mask) failed with CUresult %d", static_cast<int>(r));
  tensor_map_remember(key, *map);
  return FBMM_OK;
}

// The mask epilogue takes its element and thread masks through shared memory by TMA when
// their rows can be addressed that way: n a multiple of 128 (element rows of n bytes and
// thread rows of n / 8 bytes are then multiples of 16) and both bases 16-byte aligned.
bool masks_fit_tma(const EpiArgs& e, int n) {
  return n % 128 == 0 && (reinterpret_cast<uintptr_t>(e.element_mask) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(e.thread_mask) & 15u) == 0;
}

int make_mask_maps(CUtensorMap* em, CUtensorMap* tm, const EpiArgs& e, int l, int m, int n) {
  const bool shared = e.em_stride == 0;
  int rc;
  if ((rc = make_mask_map(em, e.element_mask, m, n, l, shared, kTileM, kTileN)) != FBMM_OK) return rc;
  return make_mask_map(tm, e.thread_mask, (m + 7) / 8, n / 8, l, shared, kTileM / 8, kTileN / 8);
}

int parse_layout(int letter, bool* transposed) {
  if (letter == 'n' || letter == 'N') { *transposed = false; return FBMM_OK; }
  if (letter == 't' || letter == 'T') { *transposed = true; return FBMM_OK; }
  return fail(FBMM_ERR_INVALID, "layout must be 'n' or 't', got %d", letter);
}

int check_dims(int l, int m, int n, int k) {
  if (l <= 0 || m <= 0 || n <= 0 || k <= 0)
    return fail(FBMM_ERR_INVALID, "l, m, n, k must be positive, got %d %d %d %d", l, m, n, k);
  return FBMM_OK;
}

// A problem in "row" form: rows come from operand `a` (M of them), columns from `b`.
struct RowProblem {
  Operand a, b;
  int L, M, N, K;
};

// Builds the row-form problem of the reference's (A, B, dim) call. dim == 2 reduces over
// the columns of A @ B; dim == 1 reduces over its rows, which is the row-wise reduction of
// B^T @ A^T: the operands swap and their storage is reread with the other majorness.
int make_row_problem(RowProblem* p, const float* A, int a_layout, long long lda, long long stride_a, const float* B,
                     int b_layout, long long ldb, long long stride_b, int l, int m, int n, int k, int dim) {
  bool at, bt;
  int rc;
  if ((rc = parse_layout(a_layout, &at)) != FBMM_OK) return rc;
  if ((rc = parse_layout(b_layout, &bt)) != FBMM_OK) return rc;
  // storage majorness of the two matrices as given
  const Operand opA{A, at, lda, stride_a, m};   // 'n': [m][k] K-major; 't': [k][m] MN-major
  const Operand opB{B, !bt, ldb, stride_b, n};  // 'n': [k][n] MN-major; 't': [n][k] K-major
  if (dim == 2) {
    p->a = opA; p->b = opB; p->M = m; p->N = n;
  } else if (dim == 1) {
    p->a = opB; p->b = opA; p->M = n; p->N = m;
  } else {
    return fail(FBMM_ERR_INVALID, "dim must be 1 or 2 (counted on the 3-D product), got %d", dim);
  }
  p->L = l; p->K = k;
  return FBMM_OK;
}

// Column chunking: with few row blocks, split the column sweep so that every SM has
// work. Models the makespan of each chunk count (`overhead_tiles` is the cost of one
// extra unit in tile-times) and takes the SMALLEST count within 5% of the best: extra
// chunks cost scratch memory and merge work, so they must pay for themselves.
void choose_chunks(int L, int m_blocks, int n_tiles, int sms, int overhead_tiles, int max_chunks, int* n_chunks,
                   int* tiles_per_chunk) {
  const long long base = static_cast<long long>(L) * m_blocks;
  const int limit = n_tiles < max_chunks ? n_tiles : max_chunks;
  auto cost_of = [&](int c, int* cc_out, int* tpc_out) -> long long {
    const int tpc = (n_tiles + c - 1) / c;
    const int cc = (n_tiles + tpc - 1) / tpc;
    const long long units = base * cc;
    const long long waves = (units + sms - 1) / sms;
    *cc_out = cc;
    *tpc_out = tpc;
    return waves * (tpc + overhead_tiles);
  };
  long long best_cost = -1;
  int cc, tpc;
  for (int c = 1; c <= limit; ++c) {
    const long long cost = cost_of(c, &cc, &tpc);
    if (best_cost < 0 || cost < best_cost) best_cost = cost;
  }
  for (int c = 1; c <= limit; ++c) {
    const long long cost = cost_of(c, &cc, &tpc);
    if (cost * 100 <= best_cost * 105) break;
  }
  *n_chunks = cc;
  *tiles_per_chunk = tpc;
}

constexpr int kStoreOverheadTiles = 1;
constexpr int kMinOverheadTiles = 1;
constexpr int kTopkOverheadTiles = 12;
constexpr int kMaxChunks = 64;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Number of floats between an operand's first and last element, storage gaps included.
long long operand_span(const Operand& op, int k, int l) {
  const long long outer = op.mn_major ? k : op.rows;
  const long long inner = op.mn_major ? op.rows : k;
  return (l > 1 ? static_cast<long long>(l - 1) * op.stride : 0) + (outer - 1) * op.ld + inner;
}

// Pre-splitting pays when every operand tile is fetched many times (each lo plane costs one
// extra read and write of the operand) and the storage has no large gaps.
bool presplit_worthwhile(const RowProblem& p) {
  if (p.M < 1024 || p.N < 1024) return false;
  const long long dense_a = static_cast<long long>(p.L) * p.M * p.K, dense_b = static_cast<long long>(p.L) * p.N * p.K;
  return operand_span(p.a, p.K, p.L) <= 2 * dense_a && operand_span(p.b, p.K, p.L) <= 2 * dense_b;
}

// The column operand streams past every row block. Its hi and lo planes together must stay
// L2-sized while the CTAs pass over them: over a long sweep the CTAs drift apart, and a
// stream that L2 cannot hold is then re-read from HBM per CTA, where doubling it costs more
// than it saves. Wider operands need the sweep cut into column ranges (min_bmm) or paced
// (top-k with one chunk per row block).
bool b_planes_fit_l2(const RowProblem& p) { return operand_span(p.b, p.K, p.L) * 8 <= 96ll * 1024 * 1024; }

bool a_stays_resident(int k) { return (k + kKBlock - 1) / kKBlock <= kMaxResidentKBlocks; }

// A column operand stored with n contiguous has the K pieces of a column tile one whole row
// of the operand apart. Once the operand is large, every tile then touches dozens of pages
// out of a set no TLB holds (measured on a 1 GB operand with K = 256: 134 instead of 223
// TFLOP/s; from 64 MB up the k-contiguous form is 10-15 % faster). Such an operand is
// copied, while it is being split anyway, into k-contiguous hi and lo planes.
bool b_gets_repacked(const RowProblem& p) {
  return p.b.mn_major && p.L <= 65535 && operand_span(p.b, p.K, p.L) * 4 >= (64ll << 20);
}
int repacked_pitch(int k) { return (k + 3) / 4 * 4; }
size_t repacked_plane_bytes(const RowProblem& p) {
  return align_up(static_cast<size_t>(p.L) * p.N * repacked_pitch(p.K) * 4, 256);
}

// Room for the pre-split planes: the column operand's lo plane (or both its planes when it
// is repacked), and the row operand's lo plane only when it streams through the ring
// (K > 128); a resident row block is split in shared memory.
size_t presplit_bytes(const RowProblem& p) {
  const size_t a = a_stays_resident(p.K) ? 0 : align_up(static_cast<size_t>(operand_span(p.a, p.K, p.L)) * 4, 256);
  if (b_gets_repacked(p)) return a + 2 * repacked_plane_bytes(p);
  return a + align_up(static_cast<size_t>(operand_span(p.b, p.K, p.L)) * 4, 256);
}

size_t norms_bytes(const RowProblem& p) {
  return align_up(static_cast<size_t>(p.L) * p.M * 4, 256) + align_up(static_cast<size_t>(p.L) * p.N * 4, 256);
}

// Squared norms of both operands of a row-form problem into `scratch` (norms_bytes);
// fills the epilogue arguments.
int launch_norms(cudaStream_t stream, const RowProblem& p, void* scratch, EpiArgs* e) {
  float* rn = static_cast<float*>(scratch);
  float* cn = reinterpret_cast<float*>(static_cast<char*>(scratch) + align_up(static_cast<size_t>(p.L) * p.M * 4, 256));
  const Operand* ops[2] = {&p.a, &p.b};
  float* outs[2] = {rn, cn};
  for (int i = 0; i < 2; ++i) {
    const Operand& op = *ops[i];
    const long long total = static_cast<long long>(p.L) * op.rows;
    const int threads = 256;
    const long long work = op.mn_major ? total : total * 32;
    const long long blocks = (work + threads - 1) / threads;
    fbmm_sqnorm_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(op.ptr, outs[i], p.L, op.rows, p.K, op.ld,
                                                                              p.L > 1 ? op.stride : 0, op.mn_major ? 1 : 0);
  }
  FBMM_CUDA(cudaGetLastError());
  e->row_norms = rn;
  e->col_norms = cn;
  return FBMM_OK;
}

// `l1_ok`: the entry point has the SIMT l1 path behind it (fp32 min and top-k); the 16-bit entries do not.
int check_distance(int distance, bool l1_ok = true) {
  if (distance == FBMM_DIST_L1 && !l1_ok)
    return fail(FBMM_ERR_UNSUPPORTED, "FBMM_DIST_L1 is available for fp32 operands only");
  if (distance != FBMM_DIST_INNER && distance != FBMM_DIST_L2 && distance != FBMM_DIST_L1)
    return fail(FBMM_ERR_INVALID, "distance must be FBMM_DIST_INNER (0), FBMM_DIST_L2 (1) or FBMM_DIST_L1 (2), got %d", distance);
  return FBMM_OK;
}

// The l1 mode: the SIMT kernel of fbmm_l1_kernel.cuh on the same units, outputs and scratch as
// the tensor-core kernel. Top-k CTAs own a slot of running lists each, so there are at most `sms`
// of them; min CTAs are small enough for two per SM.
template <int EPI, int E>
int launch_l1(cudaStream_t stream, const DeviceState& st, const RowProblem& p, const GemmShape& shape, const EpiArgs& epi) {
  L1Operand oa{p.a.ptr, p.a.ld, p.L > 1 ? p.a.stride : 0, p.a.mn_major ? 1 : 0, p.M};
  L1Operand ob{p.b.ptr, p.b.ld, p.L > 1 ? p.b.stride : 0, p.b.mn_major ? 1 : 0, p.N};
  const uint32_t smem = l1_smem_bytes(EPI);
  static std::mutex mu;
  static bool attr_set[kMaxDevices] = {};
  {
    int dev = 0;
    FBMM_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(mu);
    if (!attr_set[dev]) {
      FBMM_CUDA(cudaFuncSetAttribute(fbmm_l1_kernel<EPI, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
      attr_set[dev] = true;
    }
  }
  const long long workers = EPI == kEpiTopk ? st.sms : 2ll * st.sms;
  const unsigned grid = static_cast<unsigned>(shape.num_units < workers ? shape.num_units : workers);
  fbmm_l1_kernel<EPI, E><<<grid, kL1Threads, smem, stream>>>(oa, ob, shape, epi);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}

// CTA pairs (clusters of two, tcgen05 cta_group::2; see the kernel's PAIR notes) work on
// 256-row blocks and need pre-split planes: they are what the reducing ops run on whenever
// the caller's workspace has room for the planes.
// Measured against the single-CTA pre-split kernels (same operands, one B200): K = 128 (4 k-blocks
// per tile) and K = 256 (A streams) run 2-3 % faster as pairs; K = 64 runs 25 % slower, because
// with two k-blocks per tile the accumulator hand-off between the issuing CTA and BOTH epilogues
// (one of them across the cluster) comes round too often. Pairs are used from K = 65 up.
bool pairs_apply(const RowProblem& p, bool presplit) { return presplit && p.M > kTileM && p.K > 2 * kKBlock; }
// Two resident row blocks of A per CTA (the kernel's DUAL notes): min on pre-split planes, at most
// two k-blocks, at least 256 rows.
bool dual_rows_apply(const RowProblem& p, bool presplit) {
#ifdef FBMM_NO_DUAL
  return false;
#endif
  return presplit && p.M >= 2 * kTileM && 2 * ((p.K + kKBlock - 1) / kKBlock) <= kMaxResidentKBlocks;
}
int rows_per_block(bool pairs) { return pairs ? 2 * kTileM : kTileM; }
int unit_workers(int sms, bool pairs) { return pairs ? sms / 2 : sms; }

// Launches the fused kernel. `lo_scratch` (or null) is room for the lo planes of both
// operands (presplit_bytes): when given, they are computed here by one element-wise pass
// each and the kernel runs without its splitter stage, as CTA pairs if `pairs` (the shape
// must then have been laid out in 256-row blocks).
template <int EPI, int E>
int launch_gemm(cudaStream_t stream, const DeviceState& st, const RowProblem& p, GemmShape shape, const EpiArgs& epi,
                void* lo_scratch = nullptr, bool pairs = false, bool dual = false) {
  CUtensorMap ta, tb, ta_lo, tb_lo;
  int rc;
  EpiArgs epi_args = epi;
  if (pairs && lo_scratch == nullptr) return fail(FBMM_ERR_INVALID, "internal: pair kernels need pre-split planes");
  const int b_box = pairs ? kTileN / 2 : kTileN;  // the pair kernels fetch B in pieces of 64 columns
  if ((rc = make_tensor_map(&ta, p.a, p.K, p.L, kTileM)) != FBMM_OK) return rc;
  const bool presplit = lo_scratch != nullptr && (EPI == kEpiMin || EPI == kEpiTopk);
  if (presplit) {
    const bool a_too = !a_stays_resident(p.K);
    const long long span_a = operand_span(p.a, p.K, p.L), span_b = operand_span(p.b, p.K, p.L);
    float* a_lo = static_cast<float*>(lo_scratch);
    float* b_lo = a_too ? reinterpret_cast<float*>(static_cast<char*>(lo_scratch) + align_up(static_cast<size_t>(span_a) * 4, 256))
                        : static_cast<float*>(lo_scratch);
    const int threads = 256;
    const int blocks = st.sms * 8;
    if (a_too) fbmm_split_lo_kernel<<<blocks, threads, 0, stream>>>(p.a.ptr, a_lo, span_a);
    Operand oa = p.a, ob_hi = p.b, ob_lo = p.b;
    if (b_gets_repacked(p)) {
      // both planes of the column operand, k-contiguous, in the scratch: [hi][lo]
      const int kp = repacked_pitch(p.K);
      float* b_hi = b_lo;
      b_lo = reinterpret_cast<float*>(reinterpret_cast<char*>(b_hi) + repacked_plane_bytes(p));
      const dim3 grid(static_cast<unsigned>((p.N + 31) / 32), static_cast<unsigned>((kp + 31) / 32), static_cast<unsigned>(p.L));
      fbmm_split_transpose_kernel<<<grid, dim3(32, 8, 1), 0, stream>>>(p.b.ptr, b_hi, b_lo, p.K, p.N, kp, p.b.ld,
                                                                       p.L > 1 ? p.b.stride : 0);
      ob_hi.ptr = b_hi;
      ob_hi.mn_major = false;
      ob_hi.ld = kp;
      ob_hi.stride = static_cast<long long>(p.N) * kp;
      ob_lo = ob_hi;
      shape.b_mn = 0;
      shape.b_bcast = 0;  // the repacked planes hold one copy per batch
    } else {
      fbmm_split_lo_kernel<<<blocks, threads, 0, stream>>>(p.b.ptr, b_lo, span_b);
    }
    ob_lo.ptr = b_lo;
    FBMM_CUDA(cudaGetLastError());
    ta_lo = ta;
    if (a_too) {
      oa.ptr = a_lo;
      if ((rc = make_tensor_map(&ta_lo, oa, p.K, p.L, kTileM)) != FBMM_OK) return rc;
    }
    if ((rc = make_tensor_map(&tb, ob_hi, p.K, p.L, b_box)) != FBMM_OK) return rc;
    if ((rc = make_tensor_map(&tb_lo, ob_lo, p.K, p.L, b_box)) != FBMM_OK) return rc;
  } else {
    if ((rc = make_tensor_map(&tb, p.b, p.K, p.L, b_box)) != FBMM_OK) return rc;
    ta_lo = ta;
    tb_lo = tb;
  }
  const int workers = unit_workers(st.sms, pairs);
  const long long active = shape.num_units < workers ? shape.num_units : workers;
  const int kblocks = (p.K + kKBlock - 1) / kKBlock;
  // Up to K = 128 the row block of A stays in shared memory for the whole unit.
  const bool a_resident = a_stays_resident(p.K);
  // mask tiles by TMA when the masks allow it (the kernel reads them from global memory otherwise)
  CUtensorMap tem = ta, ttm = ta;
  if (is_masked(EPI) && masks_fit_tma(epi, p.N)) {
    if ((rc = make_mask_maps(&tem, &ttm, epi, p.L, p.M, p.N)) != FBMM_OK) return rc;
    epi_args.mask_tma = 1;
  }
  if (dual && !(EPI == kEpiMin && presplit && a_resident && !pairs && 2 * kblocks <= kMaxResidentKBlocks))
    return fail(FBMM_ERR_INVALID, "internal: two resident row blocks need the pre-split min kernel and K <= 64");
  const SmemPlan plan = make_smem_plan(a_resident, dual ? 2 * kblocks : kblocks, EPI == kEpiTopk, 2u, epi_args.mask_tma != 0, pairs,
                                       EPI == kEpiSoftmax);
  if (plan.stages < 2) return fail(FBMM_ERR_INVALID, "internal: shared-memory plan has %u stages", plan.stages);
  // min / top-k have pre-split variants; store / mask never use them
  constexpr bool kHasPresplit = (EPI == kEpiMin || EPI == kEpiTopk);
  const bool ps = kHasPresplit && presplit;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(active) * (pairs ? 2u : 1u), 1, 1);
  cfg.blockDim = dim3(block_threads(EPI), 1, 1);
  cfg.dynamicSmemBytes = plan.total;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = pairs ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
#define FBMM_LAUNCH(AR, PS, PR) \
  FBMM_CUDA(cudaLaunchKernelEx(&cfg, fbmm_gemm_kernel<EPI, E, AR, PS, 0, PR>, ta, tb, ta_lo, tb_lo, tem, ttm, shape, epi_args))
  if (dual) {
    constexpr bool kMin = EPI == kEpiMin;  // (the only epilogue with this variant)
    FBMM_CUDA(cudaLaunchKernelEx(&cfg, fbmm_gemm_kernel<EPI, E, true, kMin, 0, false, kMin>, ta, tb, ta_lo, tb_lo, tem, ttm, shape,
                                 epi_args));
  } else if (ps && pairs) {
    if (a_resident) FBMM_LAUNCH(true, kHasPresplit, kHasPresplit); else FBMM_LAUNCH(false, kHasPresplit, kHasPresplit);
  } else if (a_resident) {
    if (ps) FBMM_LAUNCH(true, kHasPresplit, false); else FBMM_LAUNCH(true, false, false);
  } else {
    if (ps) FBMM_LAUNCH(false, kHasPresplit, false); else FBMM_LAUNCH(false, false, false);
  }
#undef FBMM_LAUNCH
  return FBMM_OK;
}

GemmShape base_shape(const RowProblem& p, bool pairs = false) {
  GemmShape s{};
  s.L = p.L; s.M = p.M; s.N = p.N; s.K = p.K;
  s.a_mn = p.a.mn_major ? 1 : 0;
  s.b_mn = p.b.mn_major ? 1 : 0;
  s.a_bcast = is_broadcast(p.a, p.L) ? 1 : 0;
  s.b_bcast = is_broadcast(p.b, p.L) ? 1 : 0;
  s.m_blocks = (p.M + rows_per_block(pairs) - 1) / rows_per_block(pairs);
  s.n_tiles = (p.N + kTileN - 1) / kTileN;
  return s;
}

}  // namespace

// =======================================================================================
// C ABI
// =======================================================================================
extern "C" {

int fbmm_version(void) { return 1000; }

#ifdef FBMM_PROFILE
// Tuning builds only: copies the per-role wait counters of CTA 0 to `out` (24 values).
int fbmm_debug_read_profile(long long* out) {
  FBMM_CUDA(cudaDeviceSynchronize());
  FBMM_CUDA(cudaMemcpyFromSymbol(out, fbmm::g_fbmm_prof, 24 * sizeof(long long)));
  return FBMM_OK;
}
// Tuning builds only: the tile timeline of CTA 0 (4 roles x 1024 stamps); clears it afterwards.
int fbmm_debug_read_trace(long long* out) {
  FBMM_CUDA(cudaDeviceSynchronize());
  FBMM_CUDA(cudaMemcpyFromSymbol(out, fbmm::g_fbmm_trace, 4 * 1024 * sizeof(long long)));
  static long long zeros[4 * 1024];
  FBMM_CUDA(cudaMemcpyToSymbol(fbmm::g_fbmm_trace, zeros, sizeof(zeros)));
  return FBMM_OK;
}
#endif

const char* fbmm_last_error(void) { return g_err; }

int fbmm_check(void* stream) {
  FBMM_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  unsigned int status[4] = {0, 0, 0, 0};
  FBMM_CUDA(cudaMemcpyFromSymbol(status, fbmm::g_fbmm_status, sizeof(status)));
  if (status[0] != 0) {
    const unsigned int zero[4] = {0, 0, 0, 0};
    FBMM_CUDA(cudaMemcpyToSymbol(fbmm::g_fbmm_status, zero, sizeof(zero)));
    return fail(FBMM_ERR_DEVICE, "a kernel gave up on a bounded wait (status 0x%x)", status[0]);
  }
  return FBMM_OK;
}

int fbmm_bmm_f32(void* stream, const float* A, int a_layout, long long lda, long long stride_a, const float* B,
                 int b_layout, long long ldb, long long stride_b, float* C, long long ldc, long long stride_c, int l,
                 int m, int n, int k) {
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if (C == nullptr) return fail(FBMM_ERR_INVALID, "C is null");
  if (ldc < n) return fail(FBMM_ERR_INVALID, "ldc %lld smaller than n %d", ldc, n);
  RowProblem p;
  if ((rc = make_row_problem(&p, A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, l, m, n, k, 2)) != FBMM_OK) return rc;
  if ((rc = check_operand("A", p.a, k, l)) != FBMM_OK) return rc;
  if ((rc = check_operand("B", p.b, k, l)) != FBMM_OK) return rc;
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape(p);
  choose_chunks(l, s.m_blocks, s.n_tiles, st->sms, kStoreOverheadTiles, kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  EpiArgs e{};
  e.C = C; e.ldc = ldc; e.stride_c = stride_c;
  return launch_gemm<kEpiStore, 1>(static_cast<cudaStream_t>(stream), *st, p, s, e);
}

int fbmm_mbmm_f32(void* stream, const float* A, int a_layout, long long lda, long long stride_a, const float* B,
                  int b_layout, long long ldb, long long stride_b, float* C, long long ldc, long long stride_c,
                  const unsigned char* block_mask, const unsigned char* thread_mask,
                  const unsigned char* element_mask, int share_mask, int l, int m, int n, int k) {
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if (C == nullptr) return fail(FBMM_ERR_INVALID, "C is null");
  if (ldc < n) return fail(FBMM_ERR_INVALID, "ldc %lld smaller than n %d", ldc, n);
  if (block_mask == nullptr || thread_mask == nullptr || element_mask == nullptr)
    return fail(FBMM_ERR_INVALID, "a mask pointer is null");
  RowProblem p;
  if ((rc = make_row_problem(&p, A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, l, m, n, k, 2)) != FBMM_OK) return rc;
  if ((rc = check_operand("A", p.a, k, l)) != FBMM_OK) return rc;
  if ((rc = check_operand("B", p.b, k, l)) != FBMM_OK) return rc;
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape(p);
  choose_chunks(l, s.m_blocks, s.n_tiles, st->sms, kStoreOverheadTiles, kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  EpiArgs e{};
  e.C = C; e.ldc = ldc; e.stride_c = stride_c;
  e.block_mask = block_mask; e.thread_mask = thread_mask; e.element_mask = element_mask;
  e.bm_cols = (n + 127) / 128;
  e.tm_cols = (n + 7) / 8;
  e.bm_stride = share_mask ? 0 : static_cast<long long>((m + 127) / 128) * e.bm_cols;
  e.tm_stride = share_mask ? 0 : static_cast<long long>((m + 7) / 8) * e.tm_cols;
  e.em_stride = share_mask ? 0 : static_cast<long long>(m) * n;
  return launch_gemm<kEpiMask, 1>(static_cast<cudaStream_t>(stream), *st, p, s, e);
}

int fbmm_mbmm_softmax_f32(void* stream, const float* A, int a_layout, long long lda, long long stride_a, const float* B,
                          int b_layout, long long ldb, long long stride_b, float* P, long long ldp, long long stride_p,
                          const unsigned char* block_mask, const unsigned char* thread_mask,
                          const unsigned char* element_mask, int share_mask, float scale, int l, int m, int n, int k) {
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if (P == nullptr) return fail(FBMM_ERR_INVALID, "P is null");
  if (ldp < n) return fail(FBMM_ERR_INVALID, "ldp %lld smaller than n %d", ldp, n);
  if (block_mask == nullptr || thread_mask == nullptr || element_mask == nullptr)
    return fail(FBMM_ERR_INVALID, "a mask pointer is null");
  if (!(scale == scale) || scale == INFINITY || scale == -INFINITY) return fail(FBMM_ERR_INVALID, "scale must be finite");
  RowProblem p;
  if ((rc = make_row_problem(&p, A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, l, m, n, k, 2)) != FBMM_OK) return rc;
  if ((rc = check_operand("A", p.a, k, l)) != FBMM_OK) return rc;
  if ((rc = check_operand("B", p.b, k, l)) != FBMM_OK) return rc;
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape(p);
  // one CTA owns whole rows: the row's maximum and sum live in its registers across the sweep
  s.n_chunks = 1;
  s.tiles_per_chunk = s.n_tiles;
  s.num_units = static_cast<long long>(l) * s.m_blocks;
  EpiArgs e{};
  e.C = P; e.ldc = ldp; e.stride_c = stride_p;
  e.block_mask = block_mask; e.thread_mask = thread_mask; e.element_mask = element_mask;
  e.bm_cols = (n + 127) / 128;
  e.tm_cols = (n + 7) / 8;
  e.bm_stride = share_mask ? 0 : static_cast<long long>((m + 127) / 128) * e.bm_cols;
  e.tm_stride = share_mask ? 0 : static_cast<long long>((m + 7) / 8) * e.tm_cols;
  e.em_stride = share_mask ? 0 : static_cast<long long>(m) * n;
  e.softmax_scale_log2e = scale * 1.4426950408889634f;
  return launch_gemm<kEpiSoftmax, 1>(static_cast<cudaStream_t>(stream), *st, p, s, e);
}

size_t fbmm_min_bmm_workspace_bytes(int l, int m, int n, int k, int dim, int distance) {
  (void)k;
  if (l <= 0 || m <= 0 || n <= 0) return 0;
  const long long rows = static_cast<long long>(l) * (dim == 1 ? n : m);
  size_t need = static_cast<size_t>(rows) * sizeof(unsigned long long);
  if (distance == FBMM_DIST_L2)
    need = align_up(need, 256) + align_up(static_cast<size_t>(l) * m * 4, 256) + align_up(static_cast<size_t>(l) * n * 4, 256);
  return need;
}

int fbmm_min_bmm_f32(void* stream_, const float* A, int a_layout, long long lda, long long stride_a, const float* B,
                     int b_layout, long long ldb, long long stride_b, float* values, long long* indices, int l, int m,
                     int n, int k, int dim, int distance, void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if ((rc = check_distance(distance)) != FBMM_OK) return rc;
  if (values == nullptr || indices == nullptr) return fail(FBMM_ERR_INVALID, "values or indices is null");
  RowProblem p;
  if ((rc = make_row_problem(&p, A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, l, m, n, k, dim)) != FBMM_OK) return rc;
  if ((rc = check_operand("A", dim == 2 ? p.a : p.b, k, l)) != FBMM_OK) return rc;
  if ((rc = check_operand("B", dim == 2 ? p.b : p.a, k, l)) != FBMM_OK) return rc;
  const size_t need = fbmm_min_bmm_workspace_bytes(l, m, n, k, dim, distance);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(FBMM_ERR_WORKSPACE, "min_bmm needs %zu workspace bytes, got %zu", need, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return fail(FBMM_ERR_ALIGN, "workspace is not 16-byte aligned");
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  // room behind the op's own scratch for the lo planes? then the operands are split once up
  // front and the kernel runs as CTA pairs on 256-row blocks
  const size_t lo_off = align_up(need, 256);
  const bool l1 = distance == FBMM_DIST_L1;  // SIMT kernel: no planes, no pairs
  const bool presplit = !l1 && presplit_worthwhile(p) && (b_planes_fit_l2(p) || p.L == 1) &&
                        workspace_bytes >= lo_off + presplit_bytes(p);
  const bool pairs = pairs_apply(p, presplit);
  // K <= 64 on pre-split planes: two resident row blocks of A per CTA share every B stage
  const bool dual = dual_rows_apply(p, presplit) && !pairs;
  GemmShape s = base_shape(p, pairs || dual);
  // (an l1 tile costs so many fp32 instructions that an extra unit costs nothing beside it: the
  // column sweep is cut as finely as balances the 2 x sms CTAs best)
  choose_chunks(l, s.m_blocks, s.n_tiles, l1 ? 2 * st->sms : unit_workers(st->sms, pairs), l1 ? 0 : kMinOverheadTiles,
                kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  const long long rows = static_cast<long long>(l) * p.M;
  unsigned long long* keys = static_cast<unsigned long long*>(workspace);
  FBMM_CUDA(cudaMemsetAsync(keys, 0xff, static_cast<size_t>(rows) * 8, stream));
  EpiArgs e{};
  e.keys = keys;
  if (distance == FBMM_DIST_L2 &&
      (rc = launch_norms(stream, p, static_cast<char*>(workspace) + align_up(static_cast<size_t>(rows) * 8, 256), &e)) != FBMM_OK)
    return rc;
  void* lo_scratch = nullptr;
  if (presplit) {
    lo_scratch = static_cast<char*>(workspace) + lo_off;
    // B's two planes should stay in L2 while every row block passes over them. What L2
    // keeps of data that all SMs share is about half its size, so wider B is swept in
    // column ranges of at most 40 MB (hi + lo), all row blocks per range; the packed
    // atomicMin keys make the ranges independent.
    const long long b_bytes = operand_span(p.b, p.K, p.L) * 8;
    const long long limit = 40ll * 1024 * 1024;
    if (b_bytes > limit && p.L == 1) {
      const int want = static_cast<int>((b_bytes + limit - 1) / limit);
      if (want > s.n_chunks && want <= s.n_tiles) {
        s.tiles_per_chunk = (s.n_tiles + want - 1) / want;
        s.n_chunks = (s.n_tiles + s.tiles_per_chunk - 1) / s.tiles_per_chunk;
        s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
      }
      s.chunk_major = 1;
    }
  }
  if (l1) rc = launch_l1<kEpiMin, 1>(stream, *st, p, s, e);
  else rc = launch_gemm<kEpiMin, 1>(stream, *st, p, s, e, lo_scratch, pairs, dual);
  if (rc != FBMM_OK) return rc;
  const int threads = 256;
  const long long blocks = (rows + threads - 1) / threads;
  fbmm_min_finalize_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(keys, values, indices, rows);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}

size_t fbmm_presplit_workspace_bytes(int l, int m, int n, int k, int dim, int a_layout, long long lda,
                                     long long stride_a, int b_layout, long long ldb, long long stride_b) {
  if (l <= 0 || m <= 0 || n <= 0 || k <= 0) return 0;
  RowProblem p;
  if (make_row_problem(&p, nullptr, a_layout, lda, stride_a, nullptr, b_layout, ldb, stride_b, l, m, n, k, dim) != FBMM_OK)
    return 0;
  if (p.a.ld < (p.a.mn_major ? p.M : k) || p.b.ld < (p.b.mn_major ? p.N : k)) return 0;
  if (!presplit_worthwhile(p)) return 0;
  return presplit_bytes(p);
}

// Running lists of the units in flight: one area per CTA (at most one CTA per SM), 32 E
// entries x 128 rows of fp32 values and as many int32 columns.
static size_t topk_scratch_bytes(int sms, int topk) {
  const size_t list_slots = topk <= 32 ? 32 : (topk <= 64 ? 64 : 128);  // 32 E, as chosen at launch
  return static_cast<size_t>(sms) * list_slots * kTileM * 8;
}

// Pacing of a one-chunk sweep (GemmShape::pace_tiles): ranges of about 16 MB of the column
// operand's two planes, and one counter per range and per unit a worker goes through.
struct PacePlan {
  int tiles;
  size_t count_bytes;
};
static PacePlan pace_plan(int l, int m_blocks, int n_tiles, int k, int workers) {
  const long long tile_bytes = 2ll * kTileN * ((k + kKBlock - 1) / kKBlock * kKBlock) * 4;
  PacePlan pp;
  pp.tiles = static_cast<int>(std::max(1ll, (16ll << 20) / tile_bytes));
  const long long ranges = (n_tiles + pp.tiles - 1) / pp.tiles;
  const long long per_cta = (static_cast<long long>(l) * m_blocks + workers - 1) / workers;
  pp.count_bytes = align_up(static_cast<size_t>(per_cta * ranges) * sizeof(unsigned int), 256);
  return pp;
}

// Work split and workspace layout of one top-k call, for single CTAs (128-row blocks) or CTA
// pairs (256-row blocks): [per-chunk lists, only when a row block's columns are cut into
// chunks][squared norms, l2 only][running lists of the CTAs][pacing counters, one chunk only].
struct TopkLayout {
  int m_blocks, n_tiles, n_chunks, tiles_per_chunk;
  size_t lists_values_bytes, lists_bytes, norms_off, scratch_off, pace_off, own;
  PacePlan pace;
};
static TopkLayout topk_layout(int l, int rows_pb, int cols, int k, int topk, int distance, int sms, bool pairs) {
  TopkLayout lay{};
  lay.m_blocks = (rows_pb + rows_per_block(pairs) - 1) / rows_per_block(pairs);
  lay.n_tiles = (cols + kTileN - 1) / kTileN;
  choose_chunks(l, lay.m_blocks, lay.n_tiles, unit_workers(sms, pairs), kTopkOverheadTiles, kMaxChunks, &lay.n_chunks,
                &lay.tiles_per_chunk);
  size_t at = 0;
  if (lay.n_chunks > 1) {
    const size_t entries = static_cast<size_t>(lay.n_chunks) * l * rows_pb * topk;
    lay.lists_values_bytes = align_up(entries * sizeof(float), 256);
    lay.lists_bytes = align_up(lay.lists_values_bytes + entries * sizeof(long long), 256);
    at = lay.lists_bytes;
  }
  lay.norms_off = at;
  if (distance == FBMM_DIST_L2) at += align_up(static_cast<size_t>(l) * rows_pb * 4, 256) + align_up(static_cast<size_t>(l) * cols * 4, 256);
  lay.scratch_off = at;
  at += topk_scratch_bytes(sms, topk);
  lay.pace_off = at;
  if (lay.n_chunks == 1) {
    lay.pace = pace_plan(l, lay.m_blocks, lay.n_tiles, k, unit_workers(sms, pairs));
    at += lay.pace.count_bytes;
  }
  lay.own = at;
  return lay;
}

size_t fbmm_topk_bmm_workspace_bytes(int l, int m, int n, int k, int topk, int dim, int distance) {
  if (l <= 0 || m <= 0 || n <= 0 || topk <= 0) return 0;
  const int rows_pb = dim == 1 ? n : m, cols = dim == 1 ? m : n;
  const int sms = sm_count_or_default();
  // which of the two layouts the call uses depends on the room it is given: enough for either
  const size_t single = topk_layout(l, rows_pb, cols, k, topk, distance, sms, false).own;
  const size_t pair = rows_pb > kTileM ? topk_layout(l, rows_pb, cols, k, topk, distance, sms, true).own : 0;
  return std::max(single, pair);
}

}  // extern "C"

namespace {

// Inputs and outputs of the candidate merge: lists either as two arrays (fp32 values, int64
// indices) or as one array of packed 8-byte pairs (value bits, int32 index; -1 = empty).
struct MergeIO {
  const float* cv;
  const long long* ci;
  const int2* cp;                // packed input; the index of group g gets g * group_index_stride added
  long long group_index_stride;
  float* ov;
  long long* oi;
  int2* op;                      // packed output (indices must fit 31 bits)
};
int launch_topk_merge(cudaStream_t stream, const MergeIO& io, int groups, long long rows, int topk);

// topk_bmm behind fbmm_topk_bmm_f32 (values + int64 indices with index_offset added) and
// fbmm_topk_bmm_packed_f32 (`packed` set: 8-byte pairs with plain int32 column indices).
int topk_bmm_impl(cudaStream_t stream, const float* A, int a_layout, long long lda, long long stride_a, const float* B,
                  int b_layout, long long ldb, long long stride_b, float* values, long long* indices, int2* packed, int l,
                  int m, int n, int k, int topk, int dim, int distance, long long index_offset, void* workspace,
                  size_t workspace_bytes) {
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if ((rc = check_distance(distance)) != FBMM_OK) return rc;
  if (topk <= 0 || topk > 128) return fail(FBMM_ERR_INVALID, "topk must be in 1..128, got %d", topk);
  if (packed == nullptr && (values == nullptr || indices == nullptr)) return fail(FBMM_ERR_INVALID, "values or indices is null");
  RowProblem p;
  if ((rc = make_row_problem(&p, A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, l, m, n, k, dim)) != FBMM_OK) return rc;
  if ((rc = check_operand("A", dim == 2 ? p.a : p.b, k, l)) != FBMM_OK) return rc;
  if ((rc = check_operand("B", dim == 2 ? p.b : p.a, k, l)) != FBMM_OK) return rc;
  if (static_cast<long long>(p.N) + index_offset > 0x7ffffffell || index_offset < 0)
    return fail(FBMM_ERR_INVALID, "column indices (offset %lld + %d columns) must stay below 2^31 - 1", index_offset, p.N);
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  if (workspace == nullptr) return fail(FBMM_ERR_WORKSPACE, "topk_bmm needs a workspace");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(FBMM_ERR_ALIGN, "workspace is not 256-byte aligned");
  // CTA pairs on pre-split planes when the workspace has room for the planes behind the op's
  // own scratch; a column operand wider than L2 also needs the one-chunk sweep, which can be paced
  TopkLayout lay = topk_layout(l, p.M, p.N, k, topk, distance, st->sms, true);
  const bool l1 = distance == FBMM_DIST_L1;  // SIMT kernel: no planes, no pairs, no pacing
  const bool presplit = !l1 && p.M > kTileM && presplit_worthwhile(p) && (b_planes_fit_l2(p) || lay.n_chunks == 1) &&
                        workspace_bytes >= lay.own + presplit_bytes(p);
  const bool pairs = pairs_apply(p, presplit);
  if (!pairs) lay = topk_layout(l, p.M, p.N, k, topk, distance, st->sms, false);
  if (workspace_bytes < lay.own)
    return fail(FBMM_ERR_WORKSPACE, "topk_bmm needs %zu workspace bytes, got %zu", lay.own, workspace_bytes);
  GemmShape s = base_shape(p, pairs);
  s.n_chunks = lay.n_chunks;
  s.tiles_per_chunk = lay.tiles_per_chunk;
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  const long long rows = static_cast<long long>(l) * p.M;
  char* ws = static_cast<char*>(workspace);
  EpiArgs e{};
  e.k = topk;
  e.index_offset = index_offset;
  if (s.n_chunks > 1) {
    e.topk_values = reinterpret_cast<float*>(ws);
    e.topk_indices = reinterpret_cast<long long*>(ws + lay.lists_values_bytes);
    e.topk_chunk_rows = rows;
  } else {
    e.topk_values = values;
    e.topk_indices = indices;
    e.topk_packed = packed;
    e.topk_chunk_rows = 0;
  }
  if (distance == FBMM_DIST_L2 && (rc = launch_norms(stream, p, ws + lay.norms_off, &e)) != FBMM_OK) return rc;
  e.topk_scratch = reinterpret_cast<float*>(ws + lay.scratch_off);
  void* lo_scratch = nullptr;
  if (presplit) {
    lo_scratch = ws + lay.own;
    if (!b_planes_fit_l2(p)) {
      s.pace_tiles = lay.pace.tiles;
      s.pace_slack = 2;
      s.pace_counts = reinterpret_cast<unsigned int*>(ws + lay.pace_off);
      FBMM_CUDA(cudaMemsetAsync(s.pace_counts, 0, lay.pace.count_bytes, stream));
    }
  }
  if (l1) {
    if (topk <= 32) rc = launch_l1<kEpiTopk, 1>(stream, *st, p, s, e);
    else if (topk <= 64) rc = launch_l1<kEpiTopk, 2>(stream, *st, p, s, e);
    else rc = launch_l1<kEpiTopk, 4>(stream, *st, p, s, e);
  } else if (topk <= 32) rc = launch_gemm<kEpiTopk, 1>(stream, *st, p, s, e, lo_scratch, pairs);  // E: blocks of 32 list entries per row
  else if (topk <= 64) rc = launch_gemm<kEpiTopk, 2>(stream, *st, p, s, e, lo_scratch, pairs);
  else rc = launch_gemm<kEpiTopk, 4>(stream, *st, p, s, e, lo_scratch, pairs);
  if (rc != FBMM_OK) return rc;
  if (s.n_chunks > 1) {
    MergeIO io{};
    io.cv = e.topk_values; io.ci = e.topk_indices;
    io.ov = values; io.oi = indices; io.op = packed;
    return launch_topk_merge(stream, io, s.n_chunks, rows, topk);
  }
  return FBMM_OK;
}

}  // namespace

extern "C" int fbmm_topk_bmm_f32(void* stream, const float* A, int a_layout, long long lda, long long stride_a,
                                 const float* B, int b_layout, long long ldb, long long stride_b, float* values,
                                 long long* indices, int l, int m, int n, int k, int topk, int dim, int distance,
                                 long long index_offset, void* workspace, size_t workspace_bytes) {
  return topk_bmm_impl(static_cast<cudaStream_t>(stream), A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, values,
                       indices, nullptr, l, m, n, k, topk, dim, distance, index_offset, workspace, workspace_bytes);
}

extern "C" int fbmm_topk_bmm_packed_f32(void* stream, const float* A, int a_layout, long long lda, long long stride_a,
                                        const float* B, int b_layout, long long ldb, long long stride_b,
                                        void* candidates, int l, int m, int n, int k, int topk, int dim, int distance,
                                        void* workspace, size_t workspace_bytes) {
  if (candidates == nullptr) return fail(FBMM_ERR_INVALID, "candidates is null");
  if ((reinterpret_cast<uintptr_t>(candidates) & 7u) != 0) return fail(FBMM_ERR_ALIGN, "candidates is not 8-byte aligned");
  // index_offset stays 0: packed indices are plain columns of this call's B
  return topk_bmm_impl(static_cast<cudaStream_t>(stream), A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, nullptr,
                       nullptr, static_cast<int2*>(candidates), l, m, n, k, topk, dim, distance, 0, workspace,
                       workspace_bytes);
}

// ---------------------------------------------------------------------------------------
// candidate merge (one warp per row)
// ---------------------------------------------------------------------------------------
namespace fbmm {

// One warp per row. The running list stays in registers (striped over the lanes); every
// group's list is already sorted, so it is merged whole by topk_merge_lists, and skipped
// when its best entry cannot beat the current k-th value. Entries carry their source slot
// (group * k + position) instead of the index, which is fetched at the end; equal values
// therefore keep the order (group, position), which is ascending index order when the
// groups cover ascending index ranges. Lists come as two arrays (fp32 values, int64 indices)
// or as packed pairs (value bits, int32 index local to the group's column range, to which
// group * group_index_stride is added); the result goes out in either form.
template <int E>
__global__ void __launch_bounds__(128) fbmm_topk_merge_kernel(const float* __restrict__ cv, const long long* __restrict__ ci,
                                                              const int2* __restrict__ cp, long long group_index_stride,
                                                              int groups, long long rows, int k, float* ov, long long* oi,
                                                              int2* op) {
  const long long row = static_cast<long long>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;  // whole warps leave together
  const int lane = static_cast<int>(lane_id());
  float L[E];
  int LI[E];
#pragma unroll
  for (int j = 0; j < E; ++j) { L[j] = -INFINITY; LI[j] = kTopkEmpty; }
  float thr = -INFINITY;
  for (int g = 0; g < groups; ++g) {
    const long long base = (static_cast<long long>(g) * rows + row) * k;
    float G[E];
    int GI[E];
#pragma unroll
    for (int j = 0; j < E; ++j) {
      const int i = j * 32 + lane;
      G[j] = -INFINITY;
      GI[j] = kTopkEmpty;
      if (i < k) {
        if (cp != nullptr) {
          const int2 e = cp[base + i];
          if (e.y >= 0) { G[j] = __int_as_float(e.x); GI[j] = g * k + i; }
        } else if (ci[base + i] >= 0) {
          G[j] = cv[base + i];
          GI[j] = g * k + i;
        }
      }
    }
    const float g0 = __shfl_sync(0xffffffffu, G[0], 0);
    if (g > 0 && !(g0 > thr)) continue;  // sorted: nothing in this group can enter
    topk_merge_lists<E>(L, LI, G, GI);
    thr = topk_list_entry<E>(L, k - 1);
  }
#pragma unroll
  for (int j = 0; j < E; ++j) {
    const int i = j * 32 + lane;
    if (i < k) {
      long long id = -1;
      if (LI[j] != kTopkEmpty) {
        const int g = LI[j] / k;
        const long long at = (static_cast<long long>(g) * rows + row) * k + (LI[j] % k);
        id = cp != nullptr ? static_cast<long long>(cp[at].y) + g * group_index_stride : ci[at];
      }
      if (op != nullptr) {
        op[row * k + i] = make_int2(__float_as_int(L[j]), static_cast<int>(id));
      } else {
        ov[row * k + i] = L[j];
        oi[row * k + i] = id;
      }
    }
  }
}

// Fills a packed candidate buffer with empty entries (-inf, -1): what a rank whose column
// shard is empty contributes to the exchange.
__global__ void fbmm_fill_empty_candidates_kernel(int2* out, long long count) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < count) out[i] = make_int2(__float_as_int(-INFINITY), -1);
}

}  // namespace fbmm

namespace {
int launch_topk_merge(cudaStream_t stream, const MergeIO& io, int groups, long long rows, int topk) {
  if (groups <= 0 || rows <= 0) return fail(FBMM_ERR_INVALID, "groups and rows must be positive");
  if (topk <= 0 || topk > 128) return fail(FBMM_ERR_INVALID, "topk must be in 1..128, got %d", topk);
  if (groups > (1 << 23)) return fail(FBMM_ERR_INVALID, "at most %d groups", 1 << 23);  // slot ids stay below 2^31
  const long long blocks = (rows + 3) / 4;
  if (blocks > 0x7fffffffll) return fail(FBMM_ERR_INVALID, "too many rows");
  const unsigned grid = static_cast<unsigned>(blocks);
  if (topk <= 64)
    fbmm::fbmm_topk_merge_kernel<2><<<grid, 128, 0, stream>>>(io.cv, io.ci, io.cp, io.group_index_stride, groups, rows,
                                                              topk, io.ov, io.oi, io.op);
  else
    fbmm::fbmm_topk_merge_kernel<4><<<grid, 128, 0, stream>>>(io.cv, io.ci, io.cp, io.group_index_stride, groups, rows,
                                                              topk, io.ov, io.oi, io.op);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}
}  // namespace

extern "C" int fbmm_topk_merge_f32(void* stream, const float* cand_values, const long long* cand_indices, int groups,
                                   long long rows, int topk, float* out_values, long long* out_indices) {
  if (cand_values == nullptr || cand_indices == nullptr || out_values == nullptr || out_indices == nullptr)
    return fail(FBMM_ERR_INVALID, "a pointer is null");
  MergeIO io{};
  io.cv = cand_values; io.ci = cand_indices; io.ov = out_values; io.oi = out_indices;
  return launch_topk_merge(static_cast<cudaStream_t>(stream), io, groups, rows, topk);
}

extern "C" int fbmm_topk_merge_packed_f32(void* stream, const void* candidates, int groups, long long rows, int topk,
                                          long long group_index_stride, float* out_values, long long* out_indices) {
  if (candidates == nullptr || out_values == nullptr || out_indices == nullptr)
    return fail(FBMM_ERR_INVALID, "a pointer is null");
  if ((reinterpret_cast<uintptr_t>(candidates) & 7u) != 0) return fail(FBMM_ERR_ALIGN, "candidates is not 8-byte aligned");
  if (group_index_stride < 0) return fail(FBMM_ERR_INVALID, "group_index_stride is negative");
  MergeIO io{};
  io.cp = static_cast<const int2*>(candidates);
  io.group_index_stride = group_index_stride;
  io.ov = out_values; io.oi = out_indices;
  return launch_topk_merge(static_cast<cudaStream_t>(stream), io, groups, rows, topk);
}

// ---------------------------------------------------------------------------------------
// k-means centroid update (the consumer of min_bmm with the l2 distance)
// ---------------------------------------------------------------------------------------
extern "C" size_t fbmm_kmeans_update_workspace_bytes(int k, int d) {
  if (k <= 0 || d <= 0) return 0;
  return align_up(static_cast<size_t>(k) * d * 4, 256) + align_up(static_cast<size_t>(k) * 4, 256);
}

extern "C" int fbmm_kmeans_update_f32(void* stream_, const float* X, long long ldx, const long long* assignment,
                                      long long n, int d, int k, float* centroids, long long ldc, float* counts_out,
                                      void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (X == nullptr || assignment == nullptr || centroids == nullptr) return fail(FBMM_ERR_INVALID, "a pointer is null");
  if (n <= 0 || d <= 0 || k <= 0) return fail(FBMM_ERR_INVALID, "n, d, k must be positive, got %lld %d %d", n, d, k);
  if (ldx < d || ldc < d) return fail(FBMM_ERR_INVALID, "a pitch is smaller than d");
  const size_t need = fbmm_kmeans_update_workspace_bytes(k, d);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(FBMM_ERR_WORKSPACE, "kmeans_update needs %zu workspace bytes, got %zu", need, workspace_bytes);
  DeviceState* st;
  int rc;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  float* sums = static_cast<float*>(workspace);
  unsigned int* counts =
      reinterpret_cast<unsigned int*>(static_cast<char*>(workspace) + align_up(static_cast<size_t>(k) * d * 4, 256));
  FBMM_CUDA(cudaMemsetAsync(workspace, 0, need, stream));
  const int threads = 256;
  const size_t part_bytes = (static_cast<size_t>(k) * d + k) * sizeof(float);
  if (part_bytes <= 96 * 1024 && n >= 65536) {
    // few clusters: per-CTA partial sums in shared memory, two CTAs per SM
    static std::mutex attr_mu;
    {
      std::lock_guard<std::mutex> g(attr_mu);
      FBMM_CUDA(cudaFuncSetAttribute(fbmm::fbmm_kmeans_accumulate_smem_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    }
    fbmm::fbmm_kmeans_accumulate_smem_kernel<<<static_cast<unsigned>(st->sms * 2), 512, part_bytes, stream>>>(
        X, ldx, assignment, n, d, k, sums, counts);
  } else {
    const long long want = (n * 32 + threads - 1) / threads;
    const long long cap = static_cast<long long>(st->sms) * 32;
    fbmm::fbmm_kmeans_accumulate_kernel<<<static_cast<unsigned>(want < cap ? want : cap), threads, 0, stream>>>(
        X, ldx, assignment, n, d, k, sums, counts);
  }
  const long long total = static_cast<long long>(k) * d;
  fbmm::fbmm_kmeans_finalize_kernel<<<static_cast<unsigned>((total + threads - 1) / threads), threads, 0, stream>>>(
      sums, counts, centroids, ldc, d, total, counts_out);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}

// ---------------------------------------------------------------------------------------
// min_bmm without caller scratch and without any allocation
// ---------------------------------------------------------------------------------------
// Some hosts that embed this library through the C ABI cannot allocate device memory at
// call time: a serving loop whose memory budget is fixed at start-up, or a plugin host that
// hands an operator its input and output buffers and nothing else and has no torch caching
// allocator to ask. cudaMalloc there would synchronise the device and may simply fail. For
// them the packed-key scratch of min_bmm (8 bytes per output row) lives in this
// file-scope device array instead of a caller workspace. Every GPU that loads the library
// holds these 2 MiB until the process exits.
#define FBMM_NOALLOC_MAX_ROWS 262144
static __device__ __align__(256) unsigned long long g_noalloc_min_keys[FBMM_NOALLOC_MAX_ROWS];

namespace {
// Device address of g_noalloc_min_keys per device. In host code the array's name is only a
// stand-in for the symbol, not a device pointer, so the address a kernel may use has to be
// asked for with cudaGetSymbolAddress while that device is current.
unsigned long long* g_noalloc_keys_addr[kMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;

int noalloc_keys_for_current_device(unsigned long long** out) {
  int dev = 0;
  FBMM_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(FBMM_ERR_INVALID, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_keys_addr[dev] == nullptr) {
    void* ptr = nullptr;
    FBMM_CUDA(cudaGetSymbolAddress(&ptr, g_noalloc_min_keys));
    if (ptr == nullptr) return fail(FBMM_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    g_noalloc_keys_addr[dev] = static_cast<unsigned long long*>(ptr);
  }
  *out = g_noalloc_keys_addr[dev];
  return FBMM_OK;
}
}  // namespace

extern "C" int fbmm_min_bmm_f32_noalloc(void* stream_, const float* A, int a_layout, long long lda, long long stride_a,
                                        const float* B, int b_layout, long long ldb, long long stride_b, float* values,
                                        long long* indices, int l, int m, int n, int k, int dim) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if (values == nullptr || indices == nullptr) return fail(FBMM_ERR_INVALID, "values or indices is null");
  RowProblem p;
  if ((rc = make_row_problem(&p, A, a_layout, lda, stride_a, B, b_layout, ldb, stride_b, l, m, n, k, dim)) != FBMM_OK) return rc;
  if ((rc = check_operand("A", dim == 2 ? p.a : p.b, k, l)) != FBMM_OK) return rc;
  if ((rc = check_operand("B", dim == 2 ? p.b : p.a, k, l)) != FBMM_OK) return rc;
  const long long rows = static_cast<long long>(l) * p.M;
  if (rows > FBMM_NOALLOC_MAX_ROWS)
    return fail(FBMM_ERR_WORKSPACE,
                "fbmm_min_bmm_f32_noalloc handles at most %d output rows per call (l * rows), got %lld; "
                "split the call or use fbmm_min_bmm_f32 with a caller workspace",
                FBMM_NOALLOC_MAX_ROWS, rows);
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  unsigned long long* keys = nullptr;
  if ((rc = noalloc_keys_for_current_device(&keys)) != FBMM_OK) return rc;
  GemmShape s = base_shape(p);
  choose_chunks(l, s.m_blocks, s.n_tiles, st->sms, kMinOverheadTiles, kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  // The array keeps the previous call's keys: every key this call will reduce into must
  // start at all-ones again.
  FBMM_CUDA(cudaMemsetAsync(keys, 0xff, static_cast<size_t>(rows) * 8, stream));
  EpiArgs e{};
  e.keys = keys;
  if ((rc = launch_gemm<kEpiMin, 1>(stream, *st, p, s, e)) != FBMM_OK) return rc;
  const int threads = 256;
  const long long blocks = (rows + threads - 1) / threads;
  fbmm_min_finalize_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(keys, values, indices, rows);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}

// ---------------------------------------------------------------------------------------
// 16-bit operands (fp16 / bf16): multiplied as they are by tcgen05.mma.kind::f16, fp32
// accumulation. Both operands k-contiguous: A stored [l][m][k], B stored [l][n][k].
// ---------------------------------------------------------------------------------------
namespace {

int check_dtype_x16(int dtype) {
  if (dtype != FBMM_F16 && dtype != FBMM_BF16)
    return fail(FBMM_ERR_INVALID, "dtype must be FBMM_F16 (1) or FBMM_BF16 (2), got %d", dtype);
  return FBMM_OK;
}

int check_operand_x16(const char* name, const Operand& op, int k, int l) {
  if (op.ptr == nullptr) return fail(FBMM_ERR_INVALID, "%s is null", name);
  if (op.ld < k) return fail(FBMM_ERR_INVALID, "%s pitch %lld smaller than k = %d", name, op.ld, k);
  if ((reinterpret_cast<uintptr_t>(op.ptr) & 15u) != 0) return fail(FBMM_ERR_ALIGN, "%s is not 16-byte aligned", name);
  if ((op.ld & 7) != 0) return fail(FBMM_ERR_ALIGN, "%s pitch %lld is not a multiple of 8 elements", name, op.ld);
  if (l > 1 && ((op.stride & 7) != 0 || op.stride < 0))
    return fail(FBMM_ERR_ALIGN, "%s batch stride %lld is not a non-negative multiple of 8 elements", name, op.stride);
  return FBMM_OK;
}

// K-major tensor map over 2-byte elements: dims (k, rows, l), box (64, box_rows, 1), i.e.
// 128 bytes per row, 128-byte swizzle. Pitches in `op` count elements.
int make_tensor_map_x16(CUtensorMap* map, const Operand& op, int k, int l, int box_rows, int dtype) {
  const TensorMapKey key{op.ptr, op.ld, l > 1 ? op.stride : 0, op.rows, k, l, box_rows, dtype == FBMM_BF16 ? 3 : 2};
  if (tensor_map_lookup(key, map)) return FBMM_OK;
  const bool one_batch = l == 1 || is_broadcast(op, l);
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(k), static_cast<cuuint64_t>(op.rows),
                        one_batch ? 1u : static_cast<cuuint64_t>(l)};
  cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint64_t pitch_bytes = static_cast<cuuint64_t>(op.ld) * 2u;
  cuuint64_t strides[2] = {pitch_bytes, one_batch ? pitch_bytes * dims[1] : static_cast<cuuint64_t>(op.stride) * 2u};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = g_encode(map, dtype == FBMM_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                              3, const_cast<float*>(op.ptr), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(FBMM_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  tensor_map_remember(key, *map);
  return FBMM_OK;
}

template <int EPI, int E, bool AR, int DT>
int launch_one_x16(const cudaLaunchConfig_t& cfg, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tem,
                   const CUtensorMap& ttm, const GemmShape& shape, const EpiArgs& epi) {
  FBMM_CUDA(cudaFuncSetAttribute(fbmm_gemm_kernel<EPI, E, AR, true, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSmemLimit)));
  FBMM_CUDA(cudaLaunchKernelEx(&cfg, fbmm_gemm_kernel<EPI, E, AR, true, DT>, ta, tb, ta, tb, tem, ttm, shape, epi));
  return FBMM_OK;
}

// The fused kernel on 16-bit operands. `p` holds the operands with pitches in elements.
template <int EPI, int E>
int launch_gemm_x16(cudaStream_t stream, const DeviceState& st, const RowProblem& p, GemmShape shape, const EpiArgs& epi,
                    int dtype) {
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tensor_map_x16(&ta, p.a, p.K, p.L, kTileM, dtype)) != FBMM_OK) return rc;
  if ((rc = make_tensor_map_x16(&tb, p.b, p.K, p.L, kTileN, dtype)) != FBMM_OK) return rc;
  const long long active = shape.num_units < st.sms ? shape.num_units : st.sms;
  const int kblocks = (p.K + 2 * kKBlock - 1) / (2 * kKBlock);  // 64 elements per k-block
  const bool a_resident = kblocks <= kMaxResidentKBlocks;
  EpiArgs epi_args = epi;
  CUtensorMap tem = ta, ttm = ta;
  if (EPI == kEpiMask && masks_fit_tma(epi, p.N)) {
    if ((rc = make_mask_maps(&tem, &ttm, epi, p.L, p.M, p.N)) != FBMM_OK) return rc;
    epi_args.mask_tma = 1;
  }
  const SmemPlan plan = make_smem_plan(a_resident, kblocks, EPI == kEpiTopk, 1u, epi_args.mask_tma != 0);
  if (plan.stages < 2) return fail(FBMM_ERR_INVALID, "internal: shared-memory plan has %u stages", plan.stages);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(active), 1, 1);
  cfg.blockDim = dim3(block_threads(EPI), 1, 1);
  cfg.dynamicSmemBytes = plan.total;
  cfg.stream = stream;
  if (dtype == FBMM_F16)
    return a_resident ? launch_one_x16<EPI, E, true, 1>(cfg, ta, tb, tem, ttm, shape, epi_args)
                      : launch_one_x16<EPI, E, false, 1>(cfg, ta, tb, tem, ttm, shape, epi_args);
  return a_resident ? launch_one_x16<EPI, E, true, 2>(cfg, ta, tb, tem, ttm, shape, epi_args)
                    : launch_one_x16<EPI, E, false, 2>(cfg, ta, tb, tem, ttm, shape, epi_args);
}

// Row-form problem of two k-contiguous 16-bit operands, checked.
int make_row_problem_x16(RowProblem* p, const void* A, long long lda, long long stride_a, const void* B, long long ldb,
                         long long stride_b, int l, int m, int n, int k, int dim) {
  int rc;
  if ((rc = make_row_problem(p, static_cast<const float*>(A), 'n', lda, stride_a, static_cast<const float*>(B), 't', ldb,
                             stride_b, l, m, n, k, dim)) != FBMM_OK)
    return rc;
  if ((rc = check_operand_x16("A", dim == 2 ? p->a : p->b, k, l)) != FBMM_OK) return rc;
  return check_operand_x16("B", dim == 2 ? p->b : p->a, k, l);
}

GemmShape base_shape_x16(const RowProblem& p) { return base_shape(p); }

// Squared norms of both 16-bit operands into `scratch` (norms_bytes); fills the epilogue arguments.
int launch_norms_x16(cudaStream_t stream, const RowProblem& p, void* scratch, EpiArgs* e, int dtype) {
  float* rn = static_cast<float*>(scratch);
  float* cn = reinterpret_cast<float*>(static_cast<char*>(scratch) + align_up(static_cast<size_t>(p.L) * p.M * 4, 256));
  const Operand* ops[2] = {&p.a, &p.b};
  float* outs[2] = {rn, cn};
  for (int i = 0; i < 2; ++i) {
    const Operand& op = *ops[i];
    const long long total = static_cast<long long>(p.L) * op.rows;
    const int threads = 256;
    const long long blocks = (total * 32 + threads - 1) / threads;
    fbmm_sqnorm_x16_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        reinterpret_cast<const uint16_t*>(op.ptr), outs[i], p.L, op.rows, p.K, op.ld, p.L > 1 ? op.stride : 0,
        dtype == FBMM_BF16 ? 1 : 0);
  }
  FBMM_CUDA(cudaGetLastError());
  e->row_norms = rn;
  e->col_norms = cn;
  return FBMM_OK;
}

}  // namespace

extern "C" int fbmm_min_bmm_x16(void* stream_, const void* A, long long lda, long long stride_a, const void* B,
                                long long ldb, long long stride_b, int dtype, float* values, long long* indices, int l,
                                int m, int n, int k, int dim, int distance, void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if ((rc = check_dtype_x16(dtype)) != FBMM_OK) return rc;
  if ((rc = check_distance(distance, false)) != FBMM_OK) return rc;
  if (values == nullptr || indices == nullptr) return fail(FBMM_ERR_INVALID, "values or indices is null");
  RowProblem p;
  if ((rc = make_row_problem_x16(&p, A, lda, stride_a, B, ldb, stride_b, l, m, n, k, dim)) != FBMM_OK) return rc;
  const size_t need = fbmm_min_bmm_workspace_bytes(l, m, n, k, dim, distance);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(FBMM_ERR_WORKSPACE, "min_bmm needs %zu workspace bytes, got %zu", need, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return fail(FBMM_ERR_ALIGN, "workspace is not 16-byte aligned");
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape_x16(p);
  choose_chunks(l, s.m_blocks, s.n_tiles, st->sms, kMinOverheadTiles, kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  const long long rows = static_cast<long long>(l) * p.M;
  unsigned long long* keys = static_cast<unsigned long long*>(workspace);
  FBMM_CUDA(cudaMemsetAsync(keys, 0xff, static_cast<size_t>(rows) * 8, stream));
  EpiArgs e{};
  e.keys = keys;
  if (distance == FBMM_DIST_L2 &&
      (rc = launch_norms_x16(stream, p, static_cast<char*>(workspace) + align_up(static_cast<size_t>(rows) * 8, 256), &e,
                             dtype)) != FBMM_OK)
    return rc;
  if ((rc = launch_gemm_x16<kEpiMin, 1>(stream, *st, p, s, e, dtype)) != FBMM_OK) return rc;
  const int threads = 256;
  fbmm_min_finalize_kernel<<<static_cast<unsigned>((rows + threads - 1) / threads), threads, 0, stream>>>(keys, values,
                                                                                                        indices, rows);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}

extern "C" int fbmm_topk_bmm_x16(void* stream_, const void* A, long long lda, long long stride_a, const void* B,
                                 long long ldb, long long stride_b, int dtype, float* values, long long* indices, int l,
                                 int m, int n, int k, int topk, int dim, int distance, long long index_offset,
                                 void* workspace, size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if ((rc = check_dtype_x16(dtype)) != FBMM_OK) return rc;
  if ((rc = check_distance(distance, false)) != FBMM_OK) return rc;
  if (topk <= 0 || topk > 128) return fail(FBMM_ERR_INVALID, "topk must be in 1..128, got %d", topk);
  if (values == nullptr || indices == nullptr) return fail(FBMM_ERR_INVALID, "values or indices is null");
  RowProblem p;
  if ((rc = make_row_problem_x16(&p, A, lda, stride_a, B, ldb, stride_b, l, m, n, k, dim)) != FBMM_OK) return rc;
  if (static_cast<long long>(p.N) + index_offset > 0x7ffffffell || index_offset < 0)
    return fail(FBMM_ERR_INVALID, "column indices (offset %lld + %d columns) must stay below 2^31 - 1", index_offset, p.N);
  const size_t need = fbmm_topk_bmm_workspace_bytes(l, m, n, k, topk, dim, distance);
  if (workspace == nullptr || workspace_bytes < need)
    return fail(FBMM_ERR_WORKSPACE, "topk_bmm needs %zu workspace bytes, got %zu", need, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(FBMM_ERR_ALIGN, "workspace is not 256-byte aligned");
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape_x16(p);
  const TopkLayout lay = topk_layout(l, p.M, p.N, k, topk, distance, st->sms, false);
  s.n_chunks = lay.n_chunks;
  s.tiles_per_chunk = lay.tiles_per_chunk;
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  const long long rows = static_cast<long long>(l) * p.M;
  char* ws = static_cast<char*>(workspace);
  EpiArgs e{};
  e.k = topk;
  e.index_offset = index_offset;
  if (s.n_chunks > 1) {
    e.topk_values = reinterpret_cast<float*>(ws);
    e.topk_indices = reinterpret_cast<long long*>(ws + lay.lists_values_bytes);
    e.topk_chunk_rows = rows;
  } else {
    e.topk_values = values;
    e.topk_indices = indices;
    e.topk_chunk_rows = 0;
  }
  if (distance == FBMM_DIST_L2 && (rc = launch_norms_x16(stream, p, ws + lay.norms_off, &e, dtype)) != FBMM_OK) return rc;
  e.topk_scratch = reinterpret_cast<float*>(ws + lay.scratch_off);
  if (topk <= 32) rc = launch_gemm_x16<kEpiTopk, 1>(stream, *st, p, s, e, dtype);
  else if (topk <= 64) rc = launch_gemm_x16<kEpiTopk, 2>(stream, *st, p, s, e, dtype);
  else rc = launch_gemm_x16<kEpiTopk, 4>(stream, *st, p, s, e, dtype);
  if (rc != FBMM_OK) return rc;
  if (s.n_chunks > 1)
    return fbmm_topk_merge_f32(stream_, e.topk_values, e.topk_indices, s.n_chunks, rows, topk, values, indices);
  return FBMM_OK;
}

extern "C" int fbmm_bmm_x16(void* stream_, const void* A, long long lda, long long stride_a, const void* B,
                            long long ldb, long long stride_b, int dtype, void* C, long long ldc, long long stride_c,
                            int l, int m, int n, int k) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if ((rc = check_dtype_x16(dtype)) != FBMM_OK) return rc;
  if (C == nullptr) return fail(FBMM_ERR_INVALID, "C is null");
  if (ldc < n) return fail(FBMM_ERR_INVALID, "ldc %lld smaller than n = %d", ldc, n);
  if ((reinterpret_cast<uintptr_t>(C) & 1u) != 0) return fail(FBMM_ERR_ALIGN, "C is not 2-byte aligned");
  RowProblem p;
  if ((rc = make_row_problem_x16(&p, A, lda, stride_a, B, ldb, stride_b, l, m, n, k, 2)) != FBMM_OK) return rc;
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape_x16(p);
  choose_chunks(l, s.m_blocks, s.n_tiles, st->sms, kStoreOverheadTiles, kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  EpiArgs e{};
  e.C = static_cast<float*>(C);  // elements are 2 bytes wide; ldc and stride_c count elements
  e.ldc = ldc;
  e.stride_c = stride_c;
  return launch_gemm_x16<kEpiStore, 1>(stream, *st, p, s, e, dtype);
}

extern "C" int fbmm_mbmm_x16(void* stream_, const void* A, long long lda, long long stride_a, const void* B,
                             long long ldb, long long stride_b, int dtype, void* C, long long ldc, long long stride_c,
                             const unsigned char* block_mask, const unsigned char* thread_mask,
                             const unsigned char* element_mask, int share_mask, int l, int m, int n, int k) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  int rc;
  if ((rc = check_dims(l, m, n, k)) != FBMM_OK) return rc;
  if ((rc = check_dtype_x16(dtype)) != FBMM_OK) return rc;
  if (C == nullptr) return fail(FBMM_ERR_INVALID, "C is null");
  if (ldc < n) return fail(FBMM_ERR_INVALID, "ldc %lld smaller than n = %d", ldc, n);
  if ((reinterpret_cast<uintptr_t>(C) & 1u) != 0) return fail(FBMM_ERR_ALIGN, "C is not 2-byte aligned");
  if (block_mask == nullptr || thread_mask == nullptr || element_mask == nullptr)
    return fail(FBMM_ERR_INVALID, "a mask pointer is null");
  RowProblem p;
  if ((rc = make_row_problem_x16(&p, A, lda, stride_a, B, ldb, stride_b, l, m, n, k, 2)) != FBMM_OK) return rc;
  DeviceState* st;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  GemmShape s = base_shape_x16(p);
  choose_chunks(l, s.m_blocks, s.n_tiles, st->sms, kStoreOverheadTiles, kMaxChunks, &s.n_chunks, &s.tiles_per_chunk);
  s.num_units = static_cast<long long>(l) * s.m_blocks * s.n_chunks;
  EpiArgs e{};
  e.C = static_cast<float*>(C);  // elements are 2 bytes wide; ldc and stride_c count elements
  e.ldc = ldc;
  e.stride_c = stride_c;
  e.block_mask = block_mask; e.thread_mask = thread_mask; e.element_mask = element_mask;
  e.bm_cols = (n + 127) / 128;
  e.tm_cols = (n + 7) / 8;
  e.bm_stride = share_mask ? 0 : static_cast<long long>((m + 127) / 128) * e.bm_cols;
  e.tm_stride = share_mask ? 0 : static_cast<long long>((m + 7) / 8) * e.tm_cols;
  e.em_stride = share_mask ? 0 : static_cast<long long>(m) * n;
  return launch_gemm_x16<kEpiMask, 1>(stream, *st, p, s, e, dtype);
}

// ---------------------------------------------------------------------------------------
// Column-sharded top-k behind the C ABI: local top-k -> one NCCL all-gather of packed
// candidates -> merge. NCCL is reached through dlopen, so the library has no link-time
// dependency on it and a process that never shards never loads it. If the process already
// holds a libnccl.so.2 (a PyTorch process does), the dynamic loader hands back that copy,
// so communicators made by the host's own NCCL calls and by fbmm_comm_init_rank agree.
// ---------------------------------------------------------------------------------------
#include <dlfcn.h>

namespace {

struct NcclUniqueId { char internal[128]; };  // ncclUniqueId: 128 opaque bytes
typedef int (*NcclGetUniqueIdFn)(NcclUniqueId*);
typedef int (*NcclCommInitRankFn)(void**, int, NcclUniqueId, int);
typedef int (*NcclCommDestroyFn)(void*);
typedef int (*NcclAllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*NcclAllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*NcclGetErrorStringFn)(int);
constexpr int kNcclInt32 = 2, kNcclInt64 = 4, kNcclMax = 2;  // ncclDataType_t / ncclRedOp_t values

struct NcclApi {
  void* handle = nullptr;
  NcclGetUniqueIdFn get_unique_id = nullptr;
  NcclCommInitRankFn comm_init_rank = nullptr;
  NcclCommDestroyFn comm_destroy = nullptr;
  NcclAllGatherFn all_gather = nullptr;
  NcclAllReduceFn all_reduce = nullptr;
  NcclGetErrorStringFn error_string = nullptr;
};
std::mutex g_nccl_mu;
NcclApi g_nccl;

int nccl_api(NcclApi** out) {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle == nullptr) {
    const char* name = getenv("FBMM_NCCL_LIB");
    if (name == nullptr || name[0] == '\0') name = "libnccl.so.2";
    void* h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (h == nullptr) return fail(FBMM_ERR_COMM, "cannot load %s: %s", name, dlerror());
    NcclApi api;
    api.get_unique_id = reinterpret_cast<NcclGetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
    api.comm_init_rank = reinterpret_cast<NcclCommInitRankFn>(dlsym(h, "ncclCommInitRank"));
    api.comm_destroy = reinterpret_cast<NcclCommDestroyFn>(dlsym(h, "ncclCommDestroy"));
    api.all_gather = reinterpret_cast<NcclAllGatherFn>(dlsym(h, "ncclAllGather"));
    api.all_reduce = reinterpret_cast<NcclAllReduceFn>(dlsym(h, "ncclAllReduce"));
    api.error_string = reinterpret_cast<NcclGetErrorStringFn>(dlsym(h, "ncclGetErrorString"));
    if (!api.get_unique_id || !api.comm_init_rank || !api.comm_destroy || !api.all_gather || !api.all_reduce ||
        !api.error_string) {
      dlclose(h);
      return fail(FBMM_ERR_COMM, "%s lacks an NCCL entry point this library needs", name);
    }
    api.handle = h;
    g_nccl = api;
  }
  *out = &g_nccl;
  return FBMM_OK;
}

#define FBMM_NCCL(api, call)                                                                         \
  do {                                                                                               \
    const int r_ = (call);                                                                           \
    if (r_ != 0) return fail(FBMM_ERR_COMM, "%s: %s", #call, (api)->error_string(r_));               \
  } while (0)

struct ShardedLayout {
  size_t send_off, recv_off, status_off, local_off, total;
};
ShardedLayout sharded_layout(int world, int m, int topk, size_t local_bytes) {
  ShardedLayout lay;
  const size_t list = align_up(static_cast<size_t>(m) * topk * 8, 256);
  lay.send_off = 0;
  lay.recv_off = list;
  lay.status_off = lay.recv_off + (world > 1 ? static_cast<size_t>(world) * list : 0);
  lay.local_off = lay.status_off + 256;
  lay.total = lay.local_off + align_up(local_bytes, 256);
  return lay;
}

}  // namespace

extern "C" int fbmm_comm_get_unique_id(void* id128) {
  if (id128 == nullptr) return fail(FBMM_ERR_INVALID, "id128 is null");
  NcclApi* api;
  int rc;
  if ((rc = nccl_api(&api)) != FBMM_OK) return rc;
  FBMM_NCCL(api, api->get_unique_id(static_cast<NcclUniqueId*>(id128)));
  return FBMM_OK;
}

extern "C" int fbmm_comm_init_rank(void** comm, int world, int rank, const void* id128) {
  if (comm == nullptr || id128 == nullptr) return fail(FBMM_ERR_INVALID, "comm or id128 is null");
  if (world <= 0 || rank < 0 || rank >= world) return fail(FBMM_ERR_INVALID, "bad rank %d of %d", rank, world);
  NcclApi* api;
  int rc;
  if ((rc = nccl_api(&api)) != FBMM_OK) return rc;
  NcclUniqueId id;
  memcpy(&id, id128, sizeof(id));
  FBMM_NCCL(api, api->comm_init_rank(comm, world, id, rank));
  return FBMM_OK;
}

extern "C" int fbmm_comm_destroy(void* comm) {
  if (comm == nullptr) return FBMM_OK;
  NcclApi* api;
  int rc;
  if ((rc = nccl_api(&api)) != FBMM_OK) return rc;
  FBMM_NCCL(api, api->comm_destroy(comm));
  return FBMM_OK;
}

extern "C" size_t fbmm_topk_bmm_sharded_workspace_bytes(int world, int m, int n_local, int k, int topk, int distance,
                                                        int a_layout, long long lda, int b_layout, long long ldb) {
  if (world <= 0 || m <= 0 || k <= 0 || topk <= 0 || n_local < 0) return 0;
  size_t local = 0;
  if (n_local > 0)
    local = align_up(fbmm_topk_bmm_workspace_bytes(1, m, n_local, k, topk, 2, distance), 256) +
            fbmm_presplit_workspace_bytes(1, m, n_local, k, 2, a_layout, lda, 0, b_layout, ldb, 0);
  return sharded_layout(world, m, topk, local).total;
}

extern "C" int fbmm_topk_bmm_sharded_f32(void* stream_, void* comm, int world, int rank, const float* A, int a_layout,
                                         long long lda, const float* B_local, int b_layout, long long ldb,
                                         long long cols_per_rank, float* values, long long* indices, int m, int n_local,
                                         int k, int topk, int distance, int check_peers, void* workspace,
                                         size_t workspace_bytes) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (world <= 0 || rank < 0 || rank >= world) return fail(FBMM_ERR_INVALID, "bad rank %d of %d", rank, world);
  if (world > 1 && comm == nullptr) return fail(FBMM_ERR_INVALID, "comm is null");
  if (m <= 0 || k <= 0 || n_local < 0) return fail(FBMM_ERR_INVALID, "m, k must be positive and n_local >= 0, got %d %d %d", m, k, n_local);
  if (topk <= 0 || topk > 128) return fail(FBMM_ERR_INVALID, "topk must be in 1..128, got %d", topk);
  if (values == nullptr || indices == nullptr) return fail(FBMM_ERR_INVALID, "values or indices is null");
  if (cols_per_rank < n_local) return fail(FBMM_ERR_INVALID, "cols_per_rank %lld is smaller than n_local %d", cols_per_rank, n_local);
  if (cols_per_rank * world > 0x7ffffffell) return fail(FBMM_ERR_INVALID, "global column indices must stay below 2^31 - 1");
  // Checks that come out the same on every rank (they depend on world, m and topk only) fail
  // here, on all ranks alike. Whatever can differ from rank to rank -- the local operands,
  // the local part of the workspace -- is folded into local_rc below and, with check_peers,
  // exchanged before any rank commits to the all-gather.
  const ShardedLayout lay = sharded_layout(world, m, topk, 0);
  if (workspace == nullptr || workspace_bytes < lay.local_off)
    return fail(FBMM_ERR_WORKSPACE, "sharded topk_bmm needs at least %zu workspace bytes for the exchange buffers, got %zu",
                lay.local_off, workspace_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(FBMM_ERR_ALIGN, "workspace is not 256-byte aligned");
  NcclApi* api = nullptr;
  int rc;
  if (world > 1 && (rc = nccl_api(&api)) != FBMM_OK) return rc;
  char* ws = static_cast<char*>(workspace);
  int2* send = reinterpret_cast<int2*>(ws + lay.send_off);
  int2* recv = world > 1 ? reinterpret_cast<int2*>(ws + lay.recv_off) : send;
  int* status = reinterpret_cast<int*>(ws + lay.status_off);
  const long long entries = static_cast<long long>(m) * topk;

  // 1. this rank's candidates, written in wire format straight into the send buffer
  int local_rc = FBMM_OK;
  const size_t need = fbmm_topk_bmm_sharded_workspace_bytes(world, m, n_local, k, topk, distance, a_layout, lda, b_layout, ldb);
  if (workspace_bytes < need) {
    local_rc = fail(FBMM_ERR_WORKSPACE, "sharded topk_bmm needs %zu workspace bytes on this rank, got %zu", need, workspace_bytes);
  } else if (n_local > 0) {
    local_rc = topk_bmm_impl(stream, A, a_layout, lda, 0, B_local, b_layout, ldb, 0, nullptr, nullptr, send, 1, m, n_local,
                             k, topk, 2, distance, 0, ws + lay.local_off, workspace_bytes - lay.local_off);
  } else {
    fbmm::fbmm_fill_empty_candidates_kernel<<<static_cast<unsigned>((entries + 255) / 256), 256, 0, stream>>>(send, entries);
    if (cudaGetLastError() != cudaSuccess) local_rc = fail(FBMM_ERR_CUDA, "fill kernel launch failed");
  }
  // 2. optional agreement that every rank got this far: a rank that failed must not leave
  //    the others waiting inside the all-gather
  if (world > 1 && check_peers) {
    char saved[sizeof(g_err)];
    memcpy(saved, g_err, sizeof(saved));
    FBMM_CUDA(cudaMemsetAsync(status, local_rc == FBMM_OK ? 0 : 1, sizeof(int), stream));
    FBMM_NCCL(api, api->all_reduce(status, status, 1, kNcclInt32, kNcclMax, comm, stream));
    int any = 0;
    FBMM_CUDA(cudaMemcpyAsync(&any, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
    FBMM_CUDA(cudaStreamSynchronize(stream));
    if (local_rc != FBMM_OK) { memcpy(g_err, saved, sizeof(saved)); return local_rc; }
    if (any != 0) return fail(FBMM_ERR_PEER, "another rank failed before the candidate exchange; nothing was merged");
  } else if (local_rc != FBMM_OK) {
    return local_rc;
  }
  // 3. one all-gather of the packed lists, 4. merge with global column indices
  if (world > 1) FBMM_NCCL(api, api->all_gather(send, recv, static_cast<size_t>(entries), kNcclInt64, comm, stream));
  MergeIO io{};
  io.cp = recv;
  io.group_index_stride = cols_per_rank;
  io.ov = values; io.oi = indices;
  return launch_topk_merge(stream, io, world, m, topk);
}

// ---------------------------------------------------------------------------------------
// self-test of the bounded-wait path
// ---------------------------------------------------------------------------------------
namespace fbmm {
// One warp waits on an mbarrier that nobody ever arrives on, with a budget of `budget`
// cycles. The wait runs out, the warp leaves the way the fused kernel's roles do (shared
// abort flag, then bit 0 of the device status word) and the kernel returns normally.
__global__ void fbmm_wait_expiry_selftest_kernel(long long budget) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  (void)mbar_wait(&bar, 0, &abort_flag, budget);
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag != 0) atomicOr(&g_fbmm_status[0], 1u);
}
}  // namespace fbmm

extern "C" int fbmm_selftest_wait_expiry(void* stream) {
  DeviceState* st;
  int rc;
  if ((rc = device_state(&st)) != FBMM_OK) return rc;
  fbmm::fbmm_wait_expiry_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(200000LL);
  FBMM_CUDA(cudaGetLastError());
  return FBMM_OK;
}

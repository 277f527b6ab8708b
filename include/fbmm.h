/* fbmm.h -- C ABI of libfbmm.so, the sm_100a fused fp32 batched-matmul library.
 *
 * This is the boundary that replaces the reference's CuPy RawKernel launches
 * (custom_kernel.py:12-43 and the `cp.RawKernel(...)(grid, block, args, stream)` calls in
 * bmm.py:115-125, mbmm.py:83-97, minbmm.py:132-143, topkbmm.py:137-148): plain pointers
 * and sizes in, status code out, no torch or CuPy types.
 *
 * Conventions shared by every entry point
 *  - All pointers are device pointers on the CURRENT CUDA device; `stream` is a
 *    cudaStream_t passed as void* (0 = default stream). Calls only enqueue work.
 *  - Logical shapes are the reference's: A is [l, m, k], B is [l, k, n] (bmm.py:86-87).
 *    `a_layout` / `b_layout` are 'n' or 't', the suffix letters of the reference kernels
 *    (kernels/bmm.cu:185,94,2,277): A 'n' is stored [l][m][k], A 't' is stored [l][k][m];
 *    B 'n' is stored [l][k][n], B 't' is stored [l][n][k] (kernels/bmm_helpers.cu:263,311,
 *    275,323). `ld*` is the pitch, in elements, between consecutive stored rows and
 *    `stride_*` the distance, in elements, between consecutive batches.
 *  - TMA requirements: operand base pointers 16-byte aligned, pitches and batch strides
 *    multiples of 4 elements. Violations return FBMM_ERR_ALIGN (the Python wrappers
 *    repack such operands before calling). A batch stride of 0 with l > 1 means one matrix
 *    shared by every batch (a broadcast operand).
 *  - Non-finite values: a NaN product never wins a min (a row whose products are all NaN
 *    returns +inf and index 0) and is never listed by top-k, which also never lists -inf
 *    (such rows are padded with -inf / -1 like rows with fewer than topk entries).
 *  - The library allocates no memory. Scratch comes from the caller through
 *    `workspace` / `workspace_bytes`, sized by the matching *_workspace_bytes query.
 *  - Return value: FBMM_OK or a negative FBMM_ERR_* code; fbmm_last_error() gives the
 *    message of the calling thread's last failure. Nothing throws, aborts or traps.
 */
#ifndef FBMM_H_
#define FBMM_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FBMM_OK 0
#define FBMM_ERR_INVALID (-1)     /* bad shape, layout letter, dim, k, null pointer */
#define FBMM_ERR_ALIGN (-2)       /* pointer or pitch breaks the TMA alignment rules */
#define FBMM_ERR_WORKSPACE (-3)   /* workspace missing or too small */
#define FBMM_ERR_CUDA (-4)        /* a CUDA runtime / driver call failed */
#define FBMM_ERR_DEVICE (-5)      /* a kernel reported a bounded wait that ran out */
#define FBMM_ERR_UNSUPPORTED (-6) /* not an sm_100 device */
#define FBMM_ERR_PEER (-7)        /* sharded call: another rank reported a failure */
#define FBMM_ERR_COMM (-8)        /* NCCL could not be loaded or one of its calls failed */

/* `distance` of min_bmm / topk_bmm, the reference's accumulate functions
 * (minbmm.py:12-19, kernels/bmm_helpers.cu:20-35): inner product (madd) or squared
 * Euclidean distance sum_k (a - b)^2 (squared_l2), computed on the tensor cores as
 * |a|^2 + |b|^2 - 2 a.b. The l1 distance sum_k |a - b| (l1) has no matrix-product form: it
 * runs as a plain fp32 SIMT tile kernel with the same epilogues, outputs and workspace. */
#define FBMM_DIST_INNER 0
#define FBMM_DIST_L2 1
#define FBMM_DIST_L1 2   /* sum_k |a - b| (kernels/bmm_helpers.cu:46-52): fp32 min and top-k only, a SIMT kernel */

/* Element types of the *_x16 entry points. */
#define FBMM_F16 1
#define FBMM_BF16 2

/* Library version (major * 1000 + minor). No reference counterpart. */
int fbmm_version(void);

/* Message of the calling thread's last failed call ("" if none). Replaces the Python
 * exceptions CuPy raised on launch failure (no explicit reference line). */
const char* fbmm_last_error(void);

/* Reads and clears the device status word of the current device after synchronising
 * `stream`. FBMM_ERR_DEVICE if a kernel gave up on a wait since the last check. The
 * reference has no counterpart (its spin mutex silently proceeds unlocked,
 * kernels/topkbmm.cu:23). */
int fbmm_check(void* stream);

/* C[l,m,n] = A @ B, fp32 in, fp32 out (3xTF32 on the tensor cores).
 * Replaces bmm_nn / bmm_nt / bmm_tn / bmm_tt (kernels/bmm.cu:185,94,2,277), launched from
 * BMMCUDA.__call__ (bmm.py:68-125). C is written completely (no pre-zeroing needed). */
int fbmm_bmm_f32(void* stream,
                 const float* A, int a_layout, long long lda, long long stride_a,
                 const float* B, int b_layout, long long ldb, long long stride_b,
                 float* C, long long ldc, long long stride_c,
                 int l, int m, int n, int k);

/* Masked bmm. Replaces mbmm_nn (kernels/mbmm.cu:209-374), launched from
 * MBMMCUDA._call_nn (mbmm.py:52-98). Masks are uint8: block_mask [l, ceil(m/128),
 * ceil(n/128)] (0 = the 128x128 tile is neither loaded nor multiplied and C is 0 there,
 * kernels/mbmm.cu:251-255), thread_mask [l, ceil(m/8), ceil(n/8)] (0 = that 8x8 tile of C
 * is 0, kernels/mbmm.cu:360-363), element_mask [l, m, n] (C is multiplied by the byte,
 * kernels/mbmm.cu:111-133). With share_mask != 0 the masks have no batch axis and serve
 * every batch (mbmm.py:65-68). C is written completely, zeros included. */
int fbmm_mbmm_f32(void* stream,
                  const float* A, int a_layout, long long lda, long long stride_a,
                  const float* B, int b_layout, long long ldb, long long stride_b,
                  float* C, long long ldc, long long stride_c,
                  const unsigned char* block_mask, const unsigned char* thread_mask,
                  const unsigned char* element_mask, int share_mask,
                  int l, int m, int n, int k);

/* Masked row softmax on top of mbmm, the consumer that attention-style callers put behind the
 * masked product: P[l,m,n] = softmax over the KEPT entries of each row of scale * (A @ B),
 * 0 where an entry is masked out (masks as for fbmm_mbmm_f32, read as keep / drop: any
 * non-zero element byte keeps), and an all-zero row where nothing is kept. The scores never
 * reach global memory: a CTA owns 128 whole rows, sweeps their column tiles once for the row
 * maxima and sums and a second time (B streams past again, A stays in shared memory) for the
 * probabilities, which is all it writes. Tiles whose block-mask byte is 0 are skipped in both
 * sweeps. The reference stops at the masked product (mbmm.py:109-196, kernels/mbmm.cu:209-374);
 * its notebook's comparison expression with the softmax applied,
 * torch.softmax(torch.bmm(A, B).masked_fill(~mask, -inf) * scale, -1), is the oracle. */
int fbmm_mbmm_softmax_f32(void* stream,
                          const float* A, int a_layout, long long lda, long long stride_a,
                          const float* B, int b_layout, long long ldb, long long stride_b,
                          float* P, long long ldp, long long stride_p,
                          const unsigned char* block_mask, const unsigned char* thread_mask,
                          const unsigned char* element_mask, int share_mask, float scale,
                          int l, int m, int n, int k);

/* Row-wise (dim = 2, output [l, m]) or column-wise (dim = 1, output [l, n]) minimum and
 * argmin of A @ B without materialising the product. Replaces min_bmm_nn/nt/tn/tt
 * (kernels/minbmm.cu:348,252,156,443) with their epilogues min_dim_2 / min_dim_1
 * (kernels/minbmm.cu:86,13), launched from MinBMMCUDA.__call__ (minbmm.py:78-143).
 * `dim` counts on the 3-D product as in minbmm.py:100,116-121. Ties: lowest index.
 * values fp32, indices int64; neither needs initialising. With FBMM_DIST_L2 the reduced
 * quantity is the squared distance between row m of A and column n of B. */
size_t fbmm_min_bmm_workspace_bytes(int l, int m, int n, int k, int dim, int distance);
int fbmm_min_bmm_f32(void* stream,
                     const float* A, int a_layout, long long lda, long long stride_a,
                     const float* B, int b_layout, long long ldb, long long stride_b,
                     float* values, long long* indices,
                     int l, int m, int n, int k, int dim, int distance,
                     void* workspace, size_t workspace_bytes);

/* min_bmm for callers that cannot allocate device memory and cannot supply scratch: a
 * serving loop with a memory budget frozen at start-up, or a plugin host that passes an
 * operator only its inputs and outputs (no torch allocator, and a cudaMalloc at call time
 * would synchronise the device or fail). Arguments and results as fbmm_min_bmm_f32 without
 * the workspace and without `distance`: this entry point reduces the inner product only
 * (there is no FBMM_DIST_L2 path here, because the norms would need scratch too). The
 * 8-byte-per-row key scratch lives in a 2 MiB device array inside the library (held by
 * every GPU that loads it, until exit). It has no counterpart in the reference.
 *  - Limit: l * (m for dim 2, n for dim 1) <= 262144 output rows per call; more returns
 *    FBMM_ERR_WORKSPACE with a message naming the limit.
 *  - Calls no cudaMalloc / cudaFree or allocating library routine. The first call on a
 *    device looks the array's address up (cudaGetSymbolAddress) and sets kernel
 *    attributes; make that first call outside any stream capture.
 *  - All calls on a device share the one array: calls whose kernels overlap on the GPU
 *    (different streams) race on it. Calls on one stream are safe; each clears the keys
 *    it uses before reducing into them. */
int fbmm_min_bmm_f32_noalloc(void* stream,
                             const float* A, int a_layout, long long lda, long long stride_a,
                             const float* B, int b_layout, long long ldb, long long stride_b,
                             float* values, long long* indices,
                             int l, int m, int n, int k, int dim);

/* Optional extra scratch for fbmm_min_bmm_f32 and fbmm_topk_bmm_f32. The kernels form every
 * fp32 product from three tf32 products of (hi, lo) operand planes; normally the lo planes
 * are produced in shared memory tile by tile. When the caller's workspace has this many
 * bytes beyond the op's own need (rounded up to 256), the planes of the operands that
 * stream through shared memory (the column operand; for k > 128 the row operand too) are
 * computed once into that room instead, which pays when every tile is fetched many times.
 * A column operand of 64 MB or more that is stored with n contiguous gets both its planes
 * written there k-contiguous (so this query can exceed the operands' own size). Returns 0
 * for shapes where it would not be used (fewer than 1024 rows or columns, or storage with
 * large gaps). `dim` is the dim of the call the scratch is for: with dim = 1 the operands
 * swap roles (B supplies the rows), and so do their planes. Same answers either way. No
 * reference counterpart (its kernels multiply in fp32 on the CUDA cores,
 * kernels/bmm_helpers.cu:20-26). */
size_t fbmm_presplit_workspace_bytes(int l, int m, int n, int k, int dim,
                                     int a_layout, long long lda, long long stride_a,
                                     int b_layout, long long ldb, long long stride_b);

/* Largest-`topk` entries (descending) and their indices per row (dim = 2, output
 * [l, m, topk]) or per column (dim = 1, output [l, n, topk]) of A @ B. Replaces
 * topk_bmm_nn/nt/tn/tt (kernels/topkbmm.cu:500,403,306,597) with topk_dim_2 / topk_dim_1
 * (kernels/topkbmm.cu:249,193), launched from TopkBMMCUDA.__call__ (topkbmm.py:81-157).
 * 0 < topk <= 128 (topkbmm.py:104). Outputs are contiguous [.., topk] (the reference
 * returns [:, :, :k] views of 128-wide buffers, topkbmm.py:150-151). If fewer than topk
 * entries exist the tail is -inf / -1 (kernels/topkbmm.cu:277-278). `index_offset` is
 * added to every index written (used when B holds a column shard). The workspace is always
 * needed: it holds the running lists of the row blocks in flight (the reference keeps them
 * in the 128-wide output buffers under a spin lock, kernels/topkbmm.cu:13-47), a few KB of
 * counters, and per-chunk lists when a row block's columns are split over several CTAs. */
size_t fbmm_topk_bmm_workspace_bytes(int l, int m, int n, int k, int topk, int dim, int distance);
int fbmm_topk_bmm_f32(void* stream,
                      const float* A, int a_layout, long long lda, long long stride_a,
                      const float* B, int b_layout, long long ldb, long long stride_b,
                      float* values, long long* indices,
                      int l, int m, int n, int k, int topk, int dim, int distance,
                      long long index_offset,
                      void* workspace, size_t workspace_bytes);

/* Merges `groups` descending candidate lists per row, cand_values / cand_indices laid
 * out [groups][rows][topk] (index -1 = empty slot), into the `topk` largest per row.
 * The stand-alone analogue of the reference's `bitonic_sort` kernel
 * (kernels/bitonic_sort.cu:183-216), used after column-sharded top-k. */
int fbmm_topk_merge_f32(void* stream,
                        const float* cand_values, const long long* cand_indices,
                        int groups, long long rows, int topk,
                        float* out_values, long long* out_indices);

/* topk_bmm with the result in wire format: `candidates` receives [l, rows, topk] entries of
 * 8 bytes, { float value; int index; }, descending, empty entries (-inf, -1). Indices are
 * plain column (dim = 2) or row (dim = 1) numbers of THIS call's operands, so a rank that
 * holds a column shard of B can hand the buffer to one all-gather as it is. Workspace as
 * fbmm_topk_bmm_f32 (same query). No reference counterpart: the reference is single-GPU
 * (outputs hard-wired to cuda:0, topkbmm.py:120-126). */
int fbmm_topk_bmm_packed_f32(void* stream,
                             const float* A, int a_layout, long long lda, long long stride_a,
                             const float* B, int b_layout, long long ldb, long long stride_b,
                             void* candidates,
                             int l, int m, int n, int k, int topk, int dim, int distance,
                             void* workspace, size_t workspace_bytes);

/* Merge of `groups` packed candidate lists per row, laid out [groups][rows][topk] as an
 * all-gather of fbmm_topk_bmm_packed_f32 results leaves them; group g's indices get
 * g * group_index_stride added (the first column of shard g) and come out as int64. The
 * packed form of fbmm_topk_merge_f32 (kernels/bitonic_sort.cu:183-216 analogue). */
int fbmm_topk_merge_packed_f32(void* stream, const void* candidates, int groups, long long rows, int topk,
                               long long group_index_stride, float* out_values, long long* out_indices);

/* Column-sharded top-k for hosts that are not Python: rank `rank` of `world` holds all of A
 * [m, k] and the columns [rank * cols_per_rank, rank * cols_per_rank + n_local) of B as
 * B_local (n_local may be 0 on trailing ranks). Every rank computes its local top-k in wire
 * format into the workspace, ONE ncclAllGather exchanges the lists, and every rank merges
 * them: values / indices [m, topk] hold the global result, indices global column numbers.
 * `comm` is an ncclComm_t (as void*), either the host's own or one made by
 * fbmm_comm_init_rank; NCCL is loaded with dlopen("libnccl.so.2") (FBMM_NCCL_LIB overrides
 * the name), which resolves to the copy the process already holds if there is one.
 * With check_peers != 0 the ranks first agree (one 4-byte all-reduce and a stream
 * synchronisation) that every local step was enqueued; if one failed, that rank returns its
 * own error, the others FBMM_ERR_PEER, and nobody enters the all-gather. With 0 the call
 * stays asynchronous and a rank that fails locally leaves its peers waiting in the
 * collective until the host aborts the communicator. The reference has no multi-GPU path. */
int fbmm_comm_get_unique_id(void* id128);                                   /* rank 0: 128 bytes to hand to every rank */
int fbmm_comm_init_rank(void** comm, int world, int rank, const void* id128); /* collective over all ranks */
int fbmm_comm_destroy(void* comm);
size_t fbmm_topk_bmm_sharded_workspace_bytes(int world, int m, int n_local, int k, int topk, int distance,
                                             int a_layout, long long lda, int b_layout, long long ldb);
int fbmm_topk_bmm_sharded_f32(void* stream, void* comm, int world, int rank,
                              const float* A, int a_layout, long long lda,
                              const float* B_local, int b_layout, long long ldb, long long cols_per_rank,
                              float* values, long long* indices,
                              int m, int n_local, int k, int topk, int distance, int check_peers,
                              void* workspace, size_t workspace_bytes);

/* Exercises the bounded-wait path on purpose, harmlessly: a one-warp kernel waits ~2e5 cycles
 * on a barrier nobody arrives on, gives up, and leaves through the same status word the fused
 * kernels use, so the next fbmm_check() on that stream returns FBMM_ERR_DEVICE once and
 * FBMM_OK after. No reference counterpart (its spin mutex gives up silently,
 * kernels/topkbmm.cu:23). */
int fbmm_selftest_wait_expiry(void* stream);

/* bmm, mbmm, min_bmm and topk_bmm on fp16 / bf16 operands (dtype FBMM_F16 / FBMM_BF16); C of
 * bmm / mbmm has the operands' type (as the reference allocates it, bmm.py:106),
 * rounded to nearest from the fp32 accumulator, pitch ldc and batch stride in elements. The reference's wrappers admit torch.half (bmm.py:89, minbmm.py:98) but its kernels
 * take float* only (kernels/minbmm.cu:348-354), so half inputs never worked there; here the
 * operands go to the tensor cores as they are (tcgen05.mma.kind::f16, fp32 accumulation, no
 * three-way split). Both operands must be k-contiguous: A stored [l][m][k] with pitch lda,
 * B stored [l][n][k] with pitch ldb (pitches and batch strides in elements, multiples of 8;
 * bases 16-byte aligned). values fp32, indices int64; dim, distance, ties, padding, topk,
 * index_offset and the workspace (same queries) as for the f32 entry points. */
int fbmm_bmm_x16(void* stream, const void* A, long long lda, long long stride_a,
                 const void* B, long long ldb, long long stride_b, int dtype,
                 void* C, long long ldc, long long stride_c, int l, int m, int n, int k);
int fbmm_mbmm_x16(void* stream, const void* A, long long lda, long long stride_a,
                  const void* B, long long ldb, long long stride_b, int dtype,
                  void* C, long long ldc, long long stride_c,
                  const unsigned char* block_mask, const unsigned char* thread_mask,
                  const unsigned char* element_mask, int share_mask, int l, int m, int n, int k);
int fbmm_min_bmm_x16(void* stream, const void* A, long long lda, long long stride_a,
                     const void* B, long long ldb, long long stride_b, int dtype,
                     float* values, long long* indices, int l, int m, int n, int k, int dim, int distance,
                     void* workspace, size_t workspace_bytes);
int fbmm_topk_bmm_x16(void* stream, const void* A, long long lda, long long stride_a,
                      const void* B, long long ldb, long long stride_b, int dtype,
                      float* values, long long* indices, int l, int m, int n, int k, int topk, int dim,
                      int distance, long long index_offset, void* workspace, size_t workspace_bytes);

/* k-means centroid update, the step that consumes min_bmm with FBMM_DIST_L2 (points as A,
 * centroids as the columns of B, dim = 2: `assignment` is its index output). For every
 * centroid c that at least one point chose, centroids[c][:] becomes the mean of those
 * points; the others are left as they are. X is [n][d] with pitch ldx, centroids [k][d] with
 * pitch ldc, assignment [n] int64 (entries outside [0, k) are skipped); counts_out (or null)
 * receives the k cluster sizes as fp32. Sums are formed with floating-point atomics, so the
 * last bits depend on the order the hardware happens to take. The reference has no such
 * kernel: it stops at the assignment (minbmm.py:78-157). */
size_t fbmm_kmeans_update_workspace_bytes(int k, int d);
int fbmm_kmeans_update_f32(void* stream, const float* X, long long ldx, const long long* assignment,
                           long long n, int d, int k, float* centroids, long long ldc, float* counts_out,
                           void* workspace, size_t workspace_bytes);

#ifdef __cplusplus
}
#endif
#endif /* FBMM_H_ */

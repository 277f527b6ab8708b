/* CPU restatement, in plain C, of the arithmetic of the reference's CUDA kernels.
 * TEST INFRASTRUCTURE ONLY: nothing in the shipped package links or calls this file.
 *
 * Where oracle/ref_semantics.py restates the reference's torch TEST expressions, this
 * file restates what its kernels compute element by element:
 *   - every C[m][n] is one fp32 accumulator updated with fmaf over k = 0..K-1 in order
 *     (madd, kernels/bmm_helpers.cu:20-26, driven by thread_matmul_v3, :140-164);
 *   - min keeps the first (lowest) index under a strict '<' (kernels/minbmm.cu:119,138);
 *     the cross-CTA combine of the reference is racy (kernels/minbmm.cu:76-79), here it is
 *     the same strict '<' over ascending columns;
 *   - top-k keeps the largest values in descending order (kernels/topkbmm.cu:170-176),
 *     padding with -inf / -1 (kernels/topkbmm.cu:277-278);
 *   - mbmm zeroes a 128x128 tile whose block-mask byte is 0 (kernels/mbmm.cu:251-255),
 *     an 8x8 tile whose thread-mask byte is 0 (:360-363), and multiplies the rest by the
 *     element-mask byte (:111-133).
 * Parity status: the reference ships no golden vectors, so this restatement is pinned (a) to
 * the reference's torch test expressions (tests/test_oracle.py) and (b) to outputs of the
 * reference's own kernels, compiled from its sources by oracle/build_ref.py and run on a GPU
 * (tests/test_gpu_reference_kernels.py): bmm and mbmm outputs and min values must match this
 * file bit for bit. top-k is pinned by (a) only (the reference's top-k kernel takes a global
 * spin mutex and is not run); index choice between equal values is unpinned in the reference
 * itself (its value / index update is racy, kernels/minbmm.cu:76-79).
 *
 * Matrices are dense row-major: A[l][m][k], B[l][k][n].
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

static float dot_fma(const float* a, const float* b, int K, long long ldb) {
  float acc = 0.0f;
  for (int k = 0; k < K; ++k) acc = fmaf(a[k], b[(long long)k * ldb], acc);
  return acc;
}

/* squared_l2 (kernels/bmm_helpers.cu:28-35): dif = a - b; c = fmaf(dif, dif, c). */
static float dist_l2(const float* a, const float* b, int K, long long ldb) {
  float acc = 0.0f;
  for (int k = 0; k < K; ++k) {
    const float dif = a[k] - b[(long long)k * ldb];
    acc = fmaf(dif, dif, acc);
  }
  return acc;
}

/* l1 (kernels/bmm_helpers.cu:46-52): c += fabsf(a - b). */
static float dist_l1(const float* a, const float* b, int K, long long ldb) {
  float acc = 0.0f;
  for (int k = 0; k < K; ++k) acc += fabsf(a[k] - b[(long long)k * ldb]);
  return acc;
}

/* dist: 0 = inner product (madd), 1 = squared_l2, 2 = l1 (minbmm.py:12-19). */
static float entry(const float* a, const float* b, int K, long long ldb, int dist) {
  return dist == 1 ? dist_l2(a, b, K, ldb) : (dist == 2 ? dist_l1(a, b, K, ldb) : dot_fma(a, b, K, ldb));
}

void oracle_bmm(const float* A, const float* B, float* C, int L, int M, int N, int K) {
  for (int l = 0; l < L; ++l)
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n)
        C[((long long)l * M + m) * N + n] =
            dot_fma(A + ((long long)l * M + m) * K, B + (long long)l * K * N + n, K, N);
}

void oracle_mbmm(const float* A, const float* B, float* C, const uint8_t* block_mask, const uint8_t* thread_mask,
                 const uint8_t* element_mask, int share_mask, int L, int M, int N, int K) {
  const int bm_cols = (N + 127) / 128, tm_cols = (N + 7) / 8;
  const long long bm_sz = (long long)((M + 127) / 128) * bm_cols, tm_sz = (long long)((M + 7) / 8) * tm_cols;
  for (int l = 0; l < L; ++l) {
    const uint8_t* bm = block_mask + (share_mask ? 0 : l * bm_sz);
    const uint8_t* tm = thread_mask + (share_mask ? 0 : l * tm_sz);
    const uint8_t* em = element_mask + (share_mask ? 0 : (long long)l * M * N);
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        float c = 0.0f;
        if (bm[(m / 128) * bm_cols + n / 128] != 0 && tm[(m / 8) * tm_cols + n / 8] != 0)
          c = dot_fma(A + ((long long)l * M + m) * K, B + (long long)l * K * N + n, K, N) *
              (float)em[(long long)m * N + n];
        C[((long long)l * M + m) * N + n] = c;
      }
  }
}

/* dim == 2: one result per row m (min over n); dim == 1: one result per column n. */
void oracle_min_bmm(const float* A, const float* B, float* values, long long* indices, int L, int M, int N, int K,
                    int dim, int dist) {
  for (int l = 0; l < L; ++l) {
    const int R = dim == 2 ? M : N, S = dim == 2 ? N : M;
    for (int r = 0; r < R; ++r) {
      float best = INFINITY;
      long long best_i = 0;
      for (int s = 0; s < S; ++s) {
        const int m = dim == 2 ? r : s, n = dim == 2 ? s : r;
        const float c = entry(A + ((long long)l * M + m) * K, B + (long long)l * K * N + n, K, N, dist);
        if (c < best) { best = c; best_i = s; }
      }
      values[(long long)l * R + r] = best;
      indices[(long long)l * R + r] = best_i;
    }
  }
}

/* Output [l][R][topk], descending; ties keep the lower index first. */
void oracle_topk_bmm(const float* A, const float* B, float* values, long long* indices, int L, int M, int N, int K,
                     int topk, int dim, int dist) {
  for (int l = 0; l < L; ++l) {
    const int R = dim == 2 ? M : N, S = dim == 2 ? N : M;
    for (int r = 0; r < R; ++r) {
      float* v = values + ((long long)l * R + r) * topk;
      long long* ix = indices + ((long long)l * R + r) * topk;
      int cnt = 0;
      for (int s = 0; s < S; ++s) {
        const int m = dim == 2 ? r : s, n = dim == 2 ? s : r;
        const float c = entry(A + ((long long)l * M + m) * K, B + (long long)l * K * N + n, K, N, dist);
        int pos = cnt;
        while (pos > 0 && v[pos - 1] < c) --pos;      /* strict: earlier index stays ahead on ties */
        if (pos >= topk) continue;
        const int last = cnt < topk ? cnt : topk - 1;
        for (int j = last; j > pos; --j) { v[j] = v[j - 1]; ix[j] = ix[j - 1]; }
        v[pos] = c; ix[pos] = s;
        if (cnt < topk) ++cnt;
      }
      for (int j = cnt; j < topk; ++j) { v[j] = -INFINITY; ix[j] = -1; }
    }
  }
}

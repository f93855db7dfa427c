/*
 * CPU oracle for the SparseTIR sparse-operator hot path.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the
 * smoke check and the benchmark's CPU-baseline leg may load it.  The product
 * library never links or calls anything in this file.
 *
 * Every function restates, in plain serial C, an algorithm of the reference
 * (uwsampl/SparseTIR).  The citation above each function names the reference
 * file and lines it follows.  Floating point is accumulated in fp32 in the
 * same order as the reference's lowered loop nests (ascending stored position
 * inside a row), which is what the reference's `llvm` target would execute.
 *
 * Pinning status
 *   - column_part_hyb : pinned.  The reference's own test derives the same
 *     arrays independently with scipy
 *     (tests/python/sparsetir/test_format_conversion_routine.py:28-127); the
 *     test-suite restates that derivation and requires equality.
 *   - condense        : pinned the same way (same file, :130-165, g = 1).
 *   - csf_to_ell3d    : parity unpinned (the reference test asserts nothing,
 *     same file :182-225).
 *   - edge_to_row     : pinned by the lowered golden loop
 *     (tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:530-549),
 *     which this file follows statement by statement, and by numpy
 *     searchsorted in the test-suite.
 *   - csr_reduce / sparse_softmax / csr2bsr / ellmm : follow the lowered code; checked against
 *     numpy in the test-suite; parity unpinned (the reference stores no vectors for them).
 *   - csrmm / ell_spmm / sddmm / bsrmm / rgms / rgms_ell3d / tcspmm : parity unpinned.  The
 *     reference stores no numeric vectors for them and cannot be built or
 *     imported on this machine; the test-suite bounds their error against an
 *     independent fp64 scipy/numpy computation instead.
 *
 * The *_omp variants are the same loops with the outermost independent loop
 * spread over host threads; they exist for the timed CPU baseline.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ util */

typedef struct {
  int32_t* p;
  size_t n, cap;
} ivec;

static void ivec_push(ivec* v, int32_t x) {
  if (v->n == v->cap) {
    v->cap = v->cap ? v->cap * 2 : 64;
    v->p = (int32_t*)realloc(v->p, v->cap * sizeof(int32_t));
  }
  v->p[v->n++] = x;
}

static int upper_bound_int(const int32_t* a, int n, int key) {
  /* first index whose element is > key, as std::upper_bound */
  int lo = 0, hi = n;
  while (lo < hi) {
    int mid = lo + (hi - lo) / 2;
    if (a[mid] > key) hi = mid; else lo = mid + 1;
  }
  return lo;
}

/* torchrun exports OMP_NUM_THREADS=1 to its workers: the timed CPU legs ask for the cores explicitly */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* ------------------------------------------------------ column_part_hyb */
/*
 * Follows src/sparse/format.cc:46-168 (ColumnPartHyb).
 *   partition_size = ceil(num_cols / num_col_parts)           (:49)
 *   degree(row, part) = stored entries of row inside part      (:64-72, :91)
 *   bucket = upper_bound(buckets, degree-1), clamped to last   (:92-96)
 *   entries appended in CSR order; a partly filled ELL row is padded with
 *   col 0 / mask 0 when a different row arrives (:99-109) or at the end
 *   (:133-139); a row longer than the last bucket continues in a new ELL
 *   row that repeats the row id (:110-116).
 * The reference keeps the degrees in an unordered_multiset; a dense counter
 * table gives the same counts.
 */
typedef struct {
  int parts, nb;
  int32_t* buckets;
  ivec* rows; /* [parts*nb] */
  ivec* cols;
  ivec* mask;
  ivec* pos;  /* CSR position of each slot, -1 for padding (not in the reference output;
                 it is what the reference's rewrite_A copy blocks index by,
                 src/tir/transforms/sparse_format_decompose.cc:242-268) */
} hyb_t;

ORACLE_API void* oracle_hyb_create(int num_rows, int num_cols, const int32_t* indptr,
                                   const int32_t* indices, int num_col_parts,
                                   const int32_t* buckets, int num_bkts) {
  int partition_size = (num_cols + num_col_parts - 1) / num_col_parts;
  hyb_t* h = (hyb_t*)calloc(1, sizeof(hyb_t));
  h->parts = num_col_parts;
  h->nb = num_bkts;
  h->buckets = (int32_t*)malloc(sizeof(int32_t) * num_bkts);
  memcpy(h->buckets, buckets, sizeof(int32_t) * num_bkts);
  size_t k = (size_t)num_col_parts * num_bkts;
  h->rows = (ivec*)calloc(k, sizeof(ivec));
  h->cols = (ivec*)calloc(k, sizeof(ivec));
  h->mask = (ivec*)calloc(k, sizeof(ivec));
  h->pos = (ivec*)calloc(k, sizeof(ivec));

  int32_t* degree = (int32_t*)calloc((size_t)num_col_parts * (size_t)(num_rows > 0 ? num_rows : 1),
                                     sizeof(int32_t));
  for (int i = 0; i < num_rows; ++i)
    for (int j = indptr[i]; j < indptr[i + 1]; ++j)
      degree[(size_t)(indices[j] / partition_size) * num_rows + i]++;

  for (int i = 0; i < num_rows; ++i) {
    for (int j = indptr[i]; j < indptr[i + 1]; ++j) {
      int row_id = i, col_id = indices[j];
      int part_id = col_id / partition_size;
      int deg = degree[(size_t)part_id * num_rows + row_id];
      int bucket_id = upper_bound_int(buckets, num_bkts, deg - 1);
      if (bucket_id == num_bkts) bucket_id--;
      int bucket_size = buckets[bucket_id];
      size_t q = (size_t)part_id * num_bkts + bucket_id;
      int create_new = 0;
      int remainder = (int)(h->cols[q].n % (size_t)bucket_size);
      if (remainder != 0) {
        if (row_id != h->rows[q].p[h->rows[q].n - 1]) {
          for (int t = remainder; t < bucket_size; ++t) {
            ivec_push(&h->cols[q], 0);
            ivec_push(&h->mask[q], 0);
            ivec_push(&h->pos[q], -1);
          }
          create_new = 1;
        }
      } else {
        create_new = 1;
      }
      if (create_new) ivec_push(&h->rows[q], row_id);
      ivec_push(&h->cols[q], col_id);
      ivec_push(&h->mask[q], 1);
      ivec_push(&h->pos[q], j);
    }
  }
  for (size_t q = 0; q < k; ++q) {
    int bucket_size = buckets[q % num_bkts];
    int remainder = (int)(h->cols[q].n % (size_t)bucket_size);
    if (remainder != 0)
      for (int t = remainder; t < bucket_size; ++t) {
        ivec_push(&h->cols[q], 0);
        ivec_push(&h->mask[q], 0);
        ivec_push(&h->pos[q], -1);
      }
  }
  free(degree);
  return h;
}

ORACLE_API int oracle_hyb_nrows(void* hv, int part, int bucket) {
  hyb_t* h = (hyb_t*)hv;
  return (int)h->rows[(size_t)part * h->nb + bucket].n;
}

ORACLE_API void oracle_hyb_copy(void* hv, int part, int bucket, int32_t* rows, int32_t* cols,
                                int32_t* mask, int32_t* pos) {
  hyb_t* h = (hyb_t*)hv;
  size_t q = (size_t)part * h->nb + bucket;
  if (rows && h->rows[q].n) memcpy(rows, h->rows[q].p, h->rows[q].n * sizeof(int32_t));
  if (cols && h->cols[q].n) memcpy(cols, h->cols[q].p, h->cols[q].n * sizeof(int32_t));
  if (mask && h->mask[q].n) memcpy(mask, h->mask[q].p, h->mask[q].n * sizeof(int32_t));
  if (pos && h->pos[q].n) memcpy(pos, h->pos[q].p, h->pos[q].n * sizeof(int32_t));
}

ORACLE_API void oracle_hyb_free(void* hv) {
  hyb_t* h = (hyb_t*)hv;
  size_t k = (size_t)h->parts * h->nb;
  for (size_t q = 0; q < k; ++q) {
    free(h->rows[q].p); free(h->cols[q].p); free(h->mask[q].p); free(h->pos[q].p);
  }
  free(h->rows); free(h->cols); free(h->mask); free(h->pos); free(h->buckets); free(h);
}

/* --------------------------------------------------------------- condense */
/*
 * Follows src/sparse/format.cc:353-429 (ConDense).  For every tile of t rows
 * the distinct columns are visited in ascending order (the reference walks a
 * std::multimap keyed by column); every g of them open a new group whose
 * unused slots keep column 0 / mask 0.
 * Returns the number of groups; call with tile_indices == NULL to size.
 */
static int cmp_pair(const void* a, const void* b) {
  const int32_t* x = (const int32_t*)a; const int32_t* y = (const int32_t*)b;
  if (x[0] != y[0]) return x[0] < y[0] ? -1 : 1;
  return 0;
}

ORACLE_API int oracle_condense(int n, const int32_t* indptr, const int32_t* indices, int t, int g,
                               int32_t* group_indptr, int32_t* tile_indices, int32_t* mask) {
  int num_tiles = (n + t - 1) / t;
  int nnz_groups = 0;
  if (group_indptr) group_indptr[0] = 0;
  for (int tile = 0; tile < num_tiles; ++tile) {
    int r0 = tile * t, r1 = r0 + t < n ? r0 + t : n;
    int cnt = indptr[r1] - indptr[r0];
    int32_t* pairs = (int32_t*)malloc(sizeof(int32_t) * 2 * (size_t)(cnt > 0 ? cnt : 1));
    int k = 0;
    for (int i = r0; i < r1; ++i)
      for (int j = indptr[i]; j < indptr[i + 1]; ++j) { pairs[2 * k] = indices[j]; pairs[2 * k + 1] = i; ++k; }
    /* only the column order matters: rows of one column set independent mask cells */
    qsort(pairs, (size_t)cnt, 2 * sizeof(int32_t), cmp_pair);
    int tile_counter = 0;
    for (int a = 0; a < cnt;) {
      int col = pairs[2 * a];
      int b = a;
      while (b < cnt && pairs[2 * b] == col) ++b;
      tile_counter++;
      if (tile_counter == 1) {
        nnz_groups++;
        if (tile_indices) {
          for (int s = 0; s < g; ++s) tile_indices[(size_t)(nnz_groups - 1) * g + s] = 0;
          for (int s = 0; s < t * g; ++s) mask[(size_t)(nnz_groups - 1) * t * g + s] = 0;
        }
      }
      if (tile_indices) {
        tile_indices[(size_t)(nnz_groups - 1) * g + (tile_counter - 1)] = col;
        for (int e = a; e < b; ++e) {
          int row_local = pairs[2 * e + 1] - r0;
          mask[(size_t)(nnz_groups - 1) * t * g + (size_t)row_local * g + (tile_counter - 1)] = 1;
        }
      }
      if (tile_counter == g) tile_counter = 0;
      a = b;
    }
    if (group_indptr) group_indptr[tile + 1] = nnz_groups;
    free(pairs);
  }
  return nnz_groups;
}

/* ----------------------------------------------------------- csf_to_ell3d */
/*
 * Follows src/sparse/format.cc:180-343 (CSFToELL3D).  Per relation and per
 * column bucket the rows are laid out exactly like column_part_hyb lays out
 * one partition (:239-275); then, per bucket, the relations are concatenated
 * and each relation's block is padded to whole groups of nnz_rows_bkt rows,
 * repeating the last row id and adding col 0 / mask 0 (:282-314).
 * Note the reference pads row ids with `back()` of the running vector, which
 * for a relation with no rows in the bucket is the previous relation's last
 * row id; the remainder is 0 in that case so nothing is appended.
 */
typedef struct {
  int nb;
  ivec* indptr; ivec* rows; ivec* cols; ivec* mask;
} ell3d_t;

ORACLE_API void* oracle_ell3d_create(int num_rels, const int32_t* indptr0, const int32_t* indices0,
                                     const int32_t* indptr1, const int32_t* indices1,
                                     const int32_t* nnz_rows_bkt, const int32_t* nnz_cols_bkt,
                                     int num_buckets) {
  size_t k = (size_t)num_buckets * (size_t)(num_rels > 0 ? num_rels : 1);
  ivec* rows = (ivec*)calloc(k, sizeof(ivec));
  ivec* cols = (ivec*)calloc(k, sizeof(ivec));
  ivec* mask = (ivec*)calloc(k, sizeof(ivec));
  for (int rel = 0; rel < num_rels; ++rel) {
    for (int i = indptr0[rel]; i < indptr0[rel + 1]; ++i) {
      int row = indices0[i];
      int num_cols_i = indptr1[i + 1] - indptr1[i];
      int bucket_id = upper_bound_int(nnz_cols_bkt, num_buckets, num_cols_i - 1);
      if (bucket_id == num_buckets) bucket_id--;
      int cbs = nnz_cols_bkt[bucket_id];
      size_t q = (size_t)bucket_id * num_rels + rel;
      for (int j = indptr1[i]; j < indptr1[i + 1]; ++j) {
        int col = indices1[j];
        int remainder = (int)(cols[q].n % (size_t)cbs);
        int create_new = 0;
        if (remainder != 0) {
          if (row != rows[q].p[rows[q].n - 1]) {
            for (int t = remainder; t < cbs; ++t) { ivec_push(&cols[q], 0); ivec_push(&mask[q], 0); }
            create_new = 1;
          }
        } else {
          create_new = 1;
        }
        if (create_new) ivec_push(&rows[q], row);
        ivec_push(&cols[q], col);
        ivec_push(&mask[q], 1);
      }
    }
  }
  ell3d_t* h = (ell3d_t*)calloc(1, sizeof(ell3d_t));
  h->nb = num_buckets;
  h->indptr = (ivec*)calloc(num_buckets, sizeof(ivec));
  h->rows = (ivec*)calloc(num_buckets, sizeof(ivec));
  h->cols = (ivec*)calloc(num_buckets, sizeof(ivec));
  h->mask = (ivec*)calloc(num_buckets, sizeof(ivec));
  for (int b = 0; b < num_buckets; ++b) {
    int rbs = nnz_rows_bkt[b], cbs = nnz_cols_bkt[b];
    ivec_push(&h->indptr[b], 0);
    for (int rel = 0; rel < num_rels; ++rel) {
      size_t q = (size_t)b * num_rels + rel;
      for (size_t s = 0; s < rows[q].n; ++s) ivec_push(&h->rows[b], rows[q].p[s]);
      for (size_t s = 0; s < cols[q].n; ++s) ivec_push(&h->cols[b], cols[q].p[s]);
      for (size_t s = 0; s < mask[q].n; ++s) ivec_push(&h->mask[b], mask[q].p[s]);
      int rr = (int)(h->rows[b].n % (size_t)rbs);
      if (rr != 0) {
        int32_t last = h->rows[b].p[h->rows[b].n - 1];
        for (int t = rr; t < rbs; ++t) ivec_push(&h->rows[b], last);
      }
      int rc = (int)(h->cols[b].n % ((size_t)rbs * cbs));
      if (rc != 0)
        for (int t = rc; t < rbs * cbs; ++t) { ivec_push(&h->cols[b], 0); ivec_push(&h->mask[b], 0); }
      ivec_push(&h->indptr[b], (int32_t)(h->rows[b].n / (size_t)rbs));
    }
  }
  for (size_t q = 0; q < k; ++q) { free(rows[q].p); free(cols[q].p); free(mask[q].p); }
  free(rows); free(cols); free(mask);
  return h;
}

ORACLE_API int oracle_ell3d_ngroups(void* hv, int bucket, int rows_per_group) {
  ell3d_t* h = (ell3d_t*)hv;
  return (int)(h->rows[bucket].n / (size_t)rows_per_group);
}

ORACLE_API void oracle_ell3d_copy(void* hv, int bucket, int32_t* indptr, int32_t* rows,
                                  int32_t* cols, int32_t* mask) {
  ell3d_t* h = (ell3d_t*)hv;
  if (indptr) memcpy(indptr, h->indptr[bucket].p, h->indptr[bucket].n * sizeof(int32_t));
  if (rows && h->rows[bucket].n) memcpy(rows, h->rows[bucket].p, h->rows[bucket].n * sizeof(int32_t));
  if (cols && h->cols[bucket].n) memcpy(cols, h->cols[bucket].p, h->cols[bucket].n * sizeof(int32_t));
  if (mask && h->mask[bucket].n) memcpy(mask, h->mask[bucket].p, h->mask[bucket].n * sizeof(int32_t));
}

ORACLE_API void oracle_ell3d_free(void* hv) {
  ell3d_t* h = (ell3d_t*)hv;
  for (int b = 0; b < h->nb; ++b) {
    free(h->indptr[b].p); free(h->rows[b].p); free(h->cols[b].p); free(h->mask[b].p);
  }
  free(h->indptr); free(h->rows); free(h->cols); free(h->mask); free(h);
}

/* ------------------------------------------------------------------ csrmm */
/*
 * Follows tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:22-68.
 * C[i,k] is initialised at the first reduction step (T.init, :64-65), so a row
 * with no stored entry is left untouched: callers pass a zero-filled C
 * (examples/spmm/bench_spmm_naive.py:127).
 */
static void csrmm_rows(const float* a, const float* b, float* c, const int32_t* indptr,
                       const int32_t* indices, int r0, int r1, int feat) {
  for (int i = r0; i < r1; ++i) {
    int len = indptr[i + 1] - indptr[i];
    for (int j = 0; j < len; ++j) {
      int p = j + indptr[i];
      float av = a[p];
      const float* brow = b + (size_t)indices[p] * feat;
      float* crow = c + (size_t)i * feat;
      if (j == 0) for (int k = 0; k < feat; ++k) crow[k] = 0.0f;
      for (int k = 0; k < feat; ++k) crow[k] = crow[k] + av * brow[k];
    }
  }
}

ORACLE_API void oracle_csrmm(const float* a, const float* b, float* c, const int32_t* indptr,
                             const int32_t* indices, int m, int n, int feat, int nnz) {
  (void)n; (void)nnz;
  csrmm_rows(a, b, c, indptr, indices, 0, m, feat);
}

ORACLE_API void oracle_csrmm_omp(const float* a, const float* b, float* c, const int32_t* indptr,
                                 const int32_t* indices, int m, int n, int feat, int nnz) {
  (void)n; (void)nnz;
#pragma omp parallel for schedule(dynamic, 256)
  for (int i = 0; i < m; ++i) csrmm_rows(a, b, c, indptr, indices, i, i + 1, feat);
}

/* --------------------------------------------------------------- ell spmm */
/*
 * One (partition, bucket) term of the decomposed hyb SpMM: for ELL row r and
 * slot s, C[rows[r], :] += W[r,s] * B[cols[r,s], :].  Argument meaning follows
 * examples/spmm/bench_spmm.py:207-222; the loop is the ELL compute of
 * tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:252-288 with
 * blk = 1 and a row-index indirection.  C is accumulated into (the reference
 * zero-fills it once, bench_spmm.py:206).
 */
ORACLE_API void oracle_ell_spmm(const float* w, const int32_t* rows, const int32_t* cols,
                                int nrows, int width, const float* b, float* c, int feat) {
  for (int r = 0; r < nrows; ++r) {
    float* crow = c + (size_t)rows[r] * feat;
    for (int s = 0; s < width; ++s) {
      float wv = w[(size_t)r * width + s];
      const float* brow = b + (size_t)cols[(size_t)r * width + s] * feat;
      for (int k = 0; k < feat; ++k) crow[k] = crow[k] + wv * brow[k];
    }
  }
}

/* ------------------------------------------------------------ edge_to_row */
/*
 * Follows the binary-search block of
 * tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:530-549
 * statement by statement: row(p) = upper_bound(indptr, p) - 1.
 */
ORACLE_API void oracle_edge_to_row(const int32_t* indptr, int m, int nnz, int32_t* mid_out) {
  for (int vj = 0; vj < nnz; ++vj) {
    int low = 0, high = m + 1;
    int mid = low + (high - low) / 2;
    while (low < high) {
      if (indptr[mid] > vj) high = mid; else low = mid + 1;
      mid = low + (high - low) / 2;
    }
    mid_out[vj] = mid - 1;
  }
}

/* ------------------------------------------------------------------ sddmm */
/*
 * Follows tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:458-507:
 * C[p] = sum_k A[row(p),k] * B[indices[p],k], k ascending.  `scale` is an
 * optional per-edge factor applied after the dot product (not part of the
 * reference operator, which is dgl's u_dot_v; pass NULL for the reference
 * semantics).
 */
static void sddmm_rows(const float* a, const float* b, float* c, const int32_t* indptr,
                       const int32_t* indices, const float* scale, int r0, int r1, int feat) {
  for (int i = r0; i < r1; ++i) {
    const float* arow = a + (size_t)i * feat;
    for (int p = indptr[i]; p < indptr[i + 1]; ++p) {
      const float* brow = b + (size_t)indices[p] * feat;
      float acc = 0.0f;
      for (int k = 0; k < feat; ++k) acc = acc + arow[k] * brow[k];
      c[p] = scale ? scale[p] * acc : acc;
    }
  }
}

ORACLE_API void oracle_sddmm(const float* a, const float* b, float* c, const int32_t* indptr,
                             const int32_t* indices, const float* scale, int m, int n, int feat,
                             int nnz) {
  (void)n; (void)nnz;
  sddmm_rows(a, b, c, indptr, indices, scale, 0, m, feat);
}

ORACLE_API void oracle_sddmm_omp(const float* a, const float* b, float* c, const int32_t* indptr,
                                 const int32_t* indices, const float* scale, int m, int n,
                                 int feat, int nnz) {
  (void)n; (void)nnz;
#pragma omp parallel for schedule(dynamic, 64)
  for (int i = 0; i < m; ++i) sddmm_rows(a, b, c, indptr, indices, scale, i, i + 1, feat);
}

/* ------------------------------------------------------------------ bsrmm */
/*
 * Follows tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:192-249
 * with fp16 operands widened to fp32 and fp32 accumulation/output:
 * C[i*blk+bi, f] = sum_{bj} sum_{j in row i} A[p,bi,bj] * B[indices[p]*blk+bj, f]
 * (bj is the outer reduction loop, the stored block j the inner one, as in the
 * lowered nest).  C elements are initialised to 0 (T.init, :226-227), so an
 * empty block-row yields zeros.
 */
static void bsrmm_rows(const _Float16* a, const _Float16* b, float* c, const int32_t* indptr,
                       const int32_t* indices, int r0, int r1, int blk, int feat) {
  for (int i = r0; i < r1; ++i)
    for (int bi = 0; bi < blk; ++bi) {
      float* crow = c + ((size_t)i * blk + bi) * feat;
      for (int f = 0; f < feat; ++f) crow[f] = 0.0f;
      for (int bj = 0; bj < blk; ++bj)
        for (int p = indptr[i]; p < indptr[i + 1]; ++p) {
          float av = (float)a[(size_t)p * blk * blk + (size_t)bi * blk + bj];
          const _Float16* brow = b + ((size_t)indices[p] * blk + bj) * feat;
          for (int f = 0; f < feat; ++f) crow[f] = crow[f] + av * (float)brow[f];
        }
    }
}

ORACLE_API void oracle_bsrmm_f16(const uint16_t* a, const uint16_t* b, float* c,
                                 const int32_t* indptr, const int32_t* indices, int nb, int mb,
                                 int nnzb, int blk, int feat) {
  (void)mb; (void)nnzb;
  bsrmm_rows((const _Float16*)a, (const _Float16*)b, c, indptr, indices, 0, nb, blk, feat);
}

ORACLE_API void oracle_bsrmm_f16_omp(const uint16_t* a, const uint16_t* b, float* c,
                                     const int32_t* indptr, const int32_t* indices, int nb, int mb,
                                     int nnzb, int blk, int feat) {
  (void)mb; (void)nnzb;
#pragma omp parallel for schedule(dynamic, 1)
  for (int i = 0; i < nb; ++i)
    bsrmm_rows((const _Float16*)a, (const _Float16*)b, c, indptr, indices, i, i + 1, blk, feat);
}

/* ------------------------------------------------------------------- rgms */
/*
 * Follows tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:902-995
 * (rgcn_hetero_forward): for fo, r, i, j, fi:
 *   Y[I[i], fo] += A[p] * W[r, fo, fi] * X[J[p], fi]       (product grouped
 *   left to right as written at :985-994)
 * The scripted T.init would reset Y per (r, i); the runnable examples instead
 * zero Y once and accumulate over relations
 * (examples/rgms/rgcn/bench_rgcn_composable.py:48-73,212), which is what this
 * function does: it ACCUMULATES into the caller's Y.
 */
static void rgms_range(const float* a, const float* w, const float* x, float* y,
                       const int32_t* indptr_i, const int32_t* indices_i, const int32_t* indptr_j,
                       const int32_t* indices_j, int num_rels, int feat, int fo0, int fo1) {
  for (int fo = fo0; fo < fo1; ++fo)
    for (int r = 0; r < num_rels; ++r) {
      const float* wrow = w + ((size_t)r * feat + fo) * feat;
      for (int i = indptr_i[r]; i < indptr_i[r + 1]; ++i) {
        float* yp = y + (size_t)indices_i[i] * feat + fo;
        for (int p = indptr_j[i]; p < indptr_j[i + 1]; ++p) {
          const float* xrow = x + (size_t)indices_j[p] * feat;
          float av = a[p];
          float acc = *yp;
          for (int fi = 0; fi < feat; ++fi) acc = acc + av * wrow[fi] * xrow[fi];
          *yp = acc;
        }
      }
    }
}

ORACLE_API void oracle_rgms(const float* a, const float* w, const float* x, float* y,
                            const int32_t* indptr_i, const int32_t* indices_i,
                            const int32_t* indptr_j, const int32_t* indices_j, int m, int n,
                            int num_rels, int feat, int nnz_i, int nnz_j) {
  (void)m; (void)n; (void)nnz_i; (void)nnz_j;
  rgms_range(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, feat, 0, feat);
}

/* fo is an independent (spatial) axis of the lowered nest, so threads split it */
ORACLE_API void oracle_rgms_omp(const float* a, const float* w, const float* x, float* y,
                                const int32_t* indptr_i, const int32_t* indices_i,
                                const int32_t* indptr_j, const int32_t* indices_j, int m, int n,
                                int num_rels, int feat, int nnz_i, int nnz_j) {
  (void)m; (void)n; (void)nnz_i; (void)nnz_j;
#pragma omp parallel for schedule(dynamic, 1)
  for (int fo = 0; fo < feat; ++fo)
    rgms_range(a, w, x, y, indptr_i, indices_i, indptr_j, indices_j, num_rels, feat, fo, fo + 1);
}

/* ------------------------------------------------------------ rgms on ELL3D */
/*
 * One bucket of the decomposed RGMS of examples/rgms/rgcn/bench_rgcn_composable.py:
 * the rgcn_hetero_forward nest (tests/python/sparsetir/sparse_tir_scripts.py:468-499) rewritten
 * to the axes (R, IO, II, J) of the ell3d buffer (examples/rgms/rgcn/utils.py:90-108) with R and
 * IO fused into one loop over groups whose relation comes from the `mid` array
 * (bench_rgcn_composable.py:40-45, :176-178):
 *   for group g, row slot ii, output feature fo, column slot j, input feature fi:
 *     Y[rows[g,ii], fo] += A[g,ii,j] * W[mid[g], fo, fi] * X[cols[g,ii,j], fi]
 * Y is accumulated into (zero-filled by the caller, :209), loop order as scheduled there
 * (io, ii, fo, j, fi).  Padding slots carry A = 0 and column 0.
 */
ORACLE_API void oracle_rgms_ell3d_bucket(const float* a, const float* w, const float* x, float* y,
                                         const int32_t* rows, const int32_t* cols,
                                         const int32_t* mid, int num_groups, int rows_per_group,
                                         int cols_per_row, int feat) {
  for (int g = 0; g < num_groups; ++g) {
    const float* wr = w + (size_t)mid[g] * feat * feat;
    for (int ii = 0; ii < rows_per_group; ++ii) {
      size_t q = (size_t)g * rows_per_group + ii;
      float* yr = y + (size_t)rows[q] * feat;
      for (int fo = 0; fo < feat; ++fo) {
        float acc = yr[fo];
        for (int j = 0; j < cols_per_row; ++j) {
          float av = a[q * cols_per_row + j];
          const float* xr = x + (size_t)cols[q * cols_per_row + j] * feat;
          for (int fi = 0; fi < feat; ++fi) acc += av * wr[(size_t)fo * feat + fi] * xr[fi];
        }
        yr[fo] = acc;
      }
    }
  }
}

/* ----------------------------------------------------------------- tcspmm */
/*
 * Condensed ("TC-GNN") SpMM of examples/spmm/bench_tc_spmm.py:537-565 (tcspmm):
 *   for row tile io, group jo in [indptr[io], indptr[io+1]), row ii < t, slot ji < g, feature f:
 *     C[io, ii, f] += A[jo, ii, ji] * B[indices[jo, ji], f]        (init 0 per output element)
 * A is the condensed mask/value array [groups, t, g], `indices` the g source rows of every
 * group (ConDense, src/sparse/format.cc:353-429; unused slots hold row 0 with A = 0).
 * fp16 operands; the products are accumulated in fp32 here (the reference's wmma fragments
 * accumulate in fp16) and the fp32 sums are returned.
 */
ORACLE_API void oracle_tcspmm_f16(const uint16_t* a, const uint16_t* b, float* c,
                                  const int32_t* indptr, const int32_t* indices, int mb, int t,
                                  int g, int feat) {
  const _Float16* ah = (const _Float16*)a;
  const _Float16* bh = (const _Float16*)b;
#pragma omp parallel for schedule(dynamic, 16)
  for (int io = 0; io < mb; ++io)
    for (int ii = 0; ii < t; ++ii) {
      float* cr = c + ((size_t)io * t + ii) * feat;
      for (int f = 0; f < feat; ++f) cr[f] = 0.f;
      for (int jo = indptr[io]; jo < indptr[io + 1]; ++jo)
        for (int ji = 0; ji < g; ++ji) {
          float av = (float)ah[((size_t)jo * t + ii) * g + ji];
          if (av == 0.f) continue; /* adding 0 * x changes nothing for finite x */
          const _Float16* br = bh + (size_t)indices[(size_t)jo * g + ji] * feat;
          for (int f = 0; f < feat; ++f) cr[f] += av * (float)br[f];
        }
    }
}

/* --------------------------------------- csr_reduce / segment_reduce, sparse_softmax, csr2bsr, ellmm */
/*
 * B[i] = sum_j A[i, j] over the stored entries of row i, init 0
 * (tests/python/sparsetir/sparse_tir_scripts.py:74-110: segment_reduce and csr_reduce; the
 * column indices take no part in the arithmetic).
 */
ORACLE_API void oracle_csr_reduce(const float* a, float* b, const int32_t* indptr, int n) {
  for (int i = 0; i < n; ++i) {
    float s = 0.f;
    for (int p = indptr[i]; p < indptr[i + 1]; ++p) s += a[p];
    b[i] = s;
  }
}

/*
 * sparse_softmax, tests/python/sparsetir/sparse_tir_scripts.py:503-528, lowered
 * sparse_tir_lowered_buffer_scripts.py:997-1046, statement by statement:
 *   TMP[i]  = max_j A[i,j]            (init: lowest float)
 *   TMP1[i] = sum_j exp(A[i,j] - TMP[i])
 *   B[i,j]  = exp(A[i,j]) / TMP1[i]   (the numerator is NOT shifted by the maximum there)
 */
#include <float.h>
#include <math.h>
ORACLE_API void oracle_sparse_softmax(const float* a, float* b, const int32_t* indptr, int n) {
  for (int i = 0; i < n; ++i) {
    float mx = -FLT_MAX, sum = 0.f;
    for (int p = indptr[i]; p < indptr[i + 1]; ++p) mx = a[p] > mx ? a[p] : mx;
    for (int p = indptr[i]; p < indptr[i + 1]; ++p) sum += expf(a[p] - mx);
    for (int p = indptr[i]; p < indptr[i + 1]; ++p) b[p] = expf(a[p]) / sum;
  }
}

/*
 * csr2bsr, sparse_tir_scripts.py:532-557, lowered sparse_tir_lowered_buffer_scripts.py:1049-1135:
 * every stored entry (i, j) is written to block (i / blk, j / blk), element (i % blk, j % blk);
 * the block's position in its block row is the lower bound of j / blk in indices_out.
 * Elements of B that no entry maps to are left as they are.
 */
ORACLE_API void oracle_csr2bsr(const float* a, float* b, const int32_t* indptr_in,
                               const int32_t* indices_in, const int32_t* indptr_out,
                               const int32_t* indices_out, int m_in, int blk) {
  for (int i = 0; i < m_in; ++i)
    for (int p = indptr_in[i]; p < indptr_in[i + 1]; ++p) {
      int bo = indptr_out[i / blk];
      int low = 0, high = indptr_out[i / blk + 1] - bo;
      int key = indices_in[p] / blk;
      while (low < high) {
        int mid = low + (high - low) / 2;
        if (indices_out[mid + bo] < key) low = mid + 1; else high = mid;
      }
      b[((size_t)(low + bo) * blk + i % blk) * blk + indices_in[p] % blk] = a[p];
    }
}

/*
 * Block-ELL SpMM `ellmm`, sparse_tir_scripts.py:150-181, lowered
 * sparse_tir_lowered_buffer_scripts.py:252-288:
 *   C[i, bi, f] = sum_{j < col} sum_bj A[i, j, bi, bj] * B[indices[i, j], bj, f]   (init 0)
 */
ORACLE_API void oracle_ellmm(const float* a, const float* b, float* c, const int32_t* indices,
                             int nb, int col, int blk, int feat) {
  for (int i = 0; i < nb; ++i)
    for (int bi = 0; bi < blk; ++bi) {
      float* cr = c + ((size_t)i * blk + bi) * feat;
      for (int f = 0; f < feat; ++f) cr[f] = 0.f;
      for (int j = 0; j < col; ++j) {
        const float* ab = a + (((size_t)i * col + j) * blk + bi) * blk;
        const float* bb = b + (size_t)indices[(size_t)i * col + j] * blk * feat;
        for (int bj = 0; bj < blk; ++bj)
          for (int f = 0; f < feat; ++f) cr[f] += ab[bj] * bb[(size_t)bj * feat + f];
      }
    }
}

/* ----------------------------------------------------------------- fusedmm */
/*
 * Sparse attention `fusedmm` of examples/flash_graph_attention/fusedmm.py:37-96, stage by stage:
 *   score[i,j] = sum_f Q[i,f] K[j,f]                      over the stored positions (i, j)
 *   temp[i]  = max_j score[i,j];  temp1[i] = sum_j exp(score[i,j] - temp[i])
 *   softmax[i,j] = exp(score[i,j]) / temp1[i]             (numerator not shifted, as written there)
 *   O[i,f] = sum_j softmax[i,j] V[j,f]                    (init 0)
 */
ORACLE_API void oracle_fusedmm(const float* q, const float* k, const float* v, float* o,
                               const int32_t* indptr, const int32_t* indices, int m, int feat) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int i = 0; i < m; ++i) {
    int p0 = indptr[i], p1 = indptr[i + 1];
    float* orow = o + (size_t)i * feat;
    for (int f = 0; f < feat; ++f) orow[f] = 0.f;
    if (p1 == p0) continue;
    float* score = (float*)malloc(sizeof(float) * (size_t)(p1 - p0));
    float mx = -FLT_MAX, sum = 0.f;
    for (int p = p0; p < p1; ++p) {
      const float* kr = k + (size_t)indices[p] * feat;
      float s = 0.f;
      for (int f = 0; f < feat; ++f) s += q[(size_t)i * feat + f] * kr[f];
      score[p - p0] = s;
      mx = s > mx ? s : mx;
    }
    for (int p = p0; p < p1; ++p) sum += expf(score[p - p0] - mx);
    for (int p = p0; p < p1; ++p) {
      float w = expf(score[p - p0]) / sum;
      const float* vr = v + (size_t)indices[p] * feat;
      for (int f = 0; f < feat; ++f) orow[f] += w * vr[f];
    }
    free(score);
  }
}

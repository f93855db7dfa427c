// Host-side format conversion: column partitioning + ELL bucketing (hyb), TC-GNN style
// condensing, and 3-level CSF -> ELL3D.  Outputs are bit-exact with the reference routines in
// src/sparse/format.cc, but built differently: instead of appending entry by entry to growing
// vectors, every row's place in its (partition, bucket) array is computed from prefix sums of
// per-row ELL-row counts, so the arrays are allocated once and filled by several threads.
//
// Why the prefix-sum layout equals the reference's append order (format.cc:86-120,133-139):
// the reference visits rows in ascending order; inside one (partition, bucket) array all
// entries of a row are contiguous, a row always starts a fresh ELL row (a partly filled ELL
// row is padded as soon as a different row arrives, :99-109, or at the end, :133-139) and a
// row longer than the bucket width continues in further ELL rows that repeat its id
// (:110-116).  Hence row i occupies ceil(deg/width) consecutive, fully padded ELL rows that
// start right after those of all smaller row ids in the same array.
#include <algorithm>
#include <cstring>
#include <numeric>
#include <thread>
#include <vector>

#include "common.h"

using sptir::fail;

struct SparsetirHyb {
  int parts = 0, nbk = 0;
  std::vector<int32_t> widths;
  // per (part, bucket)
  std::vector<std::vector<int32_t>> rows, cols, mask, pos;
};

namespace {

int resolve_threads(int requested, long long work) {
  int hw = requested > 0 ? requested : static_cast<int>(std::thread::hardware_concurrency());
  if (hw < 1) hw = 1;
  long long by_work = work / 65536 + 1;  // no point in threads for tiny inputs
  return static_cast<int>(std::min<long long>(hw, by_work));
}

template <typename F>
void parallel_chunks(int nthreads, int n, F&& fn) {
  if (nthreads <= 1 || n == 0) {
    fn(0, 0, n);
    return;
  }
  std::vector<std::thread> pool;
  int chunk = (n + nthreads - 1) / nthreads;
  for (int t = 0; t < nthreads; ++t) {
    int lo = std::min(n, t * chunk), hi = std::min(n, lo + chunk);
    pool.emplace_back([&, t, lo, hi] { fn(t, lo, hi); });
  }
  for (auto& th : pool) th.join();
}

// smallest bucket whose width is >= degree, else the last one (format.cc:92-96)
inline int bucket_of(const int32_t* widths, int nbk, int degree) {
  int b = static_cast<int>(std::upper_bound(widths, widths + nbk, degree - 1) - widths);
  return b == nbk ? nbk - 1 : b;
}

}  // namespace

extern "C" {

SparsetirHyb* sparsetir_column_part_hyb(int num_rows, int num_cols, const int32_t* indptr,
                                        const int32_t* indices, int num_col_parts,
                                        const int32_t* buckets, int num_buckets,
                                        int num_threads) {
  if (num_rows < 0 || num_cols < 0 || num_col_parts < 1 || num_buckets < 1 || !indptr ||
      !buckets) {
    fail("sparsetir_column_part_hyb: invalid argument");
    return nullptr;
  }
  for (int b = 0; b < num_buckets; ++b)
    if (buckets[b] < 1 || (b > 0 && buckets[b] <= buckets[b - 1])) {
      fail("sparsetir_column_part_hyb: bucket widths must be positive and ascending");
      return nullptr;
    }
  const int P = num_col_parts, B = num_buckets;
  const int part_size = std::max(1, (num_cols + P - 1) / P);
  const int nnz = num_rows > 0 ? indptr[num_rows] : 0;
  for (int i = 0; i < num_rows; ++i)
    if (indptr[i + 1] < indptr[i]) {
      fail("sparsetir_column_part_hyb: indptr is not monotone at row %d", i);
      return nullptr;
    }
  const int T = resolve_threads(num_threads, (long long)nnz + num_rows);

  // Pass 1: per row and partition, the degree; from it the bucket and the number of ELL rows.
  // ell_start[(p*B+b)][i] = ELL rows that rows < i occupy in array (p, b)   (exclusive scan)
  std::vector<int32_t> degree(static_cast<size_t>(P) * num_rows, 0);
  std::vector<int> bad(T, 0);
  parallel_chunks(T, num_rows, [&](int t, int lo, int hi) {
    for (int i = lo; i < hi; ++i)
      for (int j = indptr[i]; j < indptr[i + 1]; ++j) {
        int c = indices[j];
        if (c < 0 || c >= num_cols) { bad[t] = 1; continue; }
        ++degree[static_cast<size_t>(c / part_size) * num_rows + i];
      }
  });
  if (std::accumulate(bad.begin(), bad.end(), 0) != 0) {
    fail("sparsetir_column_part_hyb: a column index is outside [0, num_cols)");
    return nullptr;
  }

  // per-thread-chunk counts, then scan over chunks, then per-row offsets inside each chunk
  const size_t Q = static_cast<size_t>(P) * B;
  std::vector<std::vector<int64_t>> chunk_count(T, std::vector<int64_t>(Q, 0));
  parallel_chunks(T, num_rows, [&](int t, int lo, int hi) {
    auto& cnt = chunk_count[t];
    for (int p = 0; p < P; ++p)
      for (int i = lo; i < hi; ++i) {
        int d = degree[static_cast<size_t>(p) * num_rows + i];
        if (d == 0) continue;
        int b = bucket_of(buckets, B, d);
        cnt[static_cast<size_t>(p) * B + b] += (d + buckets[b] - 1) / buckets[b];
      }
  });
  std::vector<std::vector<int64_t>> chunk_base(T, std::vector<int64_t>(Q, 0));
  std::vector<int64_t> total(Q, 0);
  for (size_t q = 0; q < Q; ++q)
    for (int t = 0; t < T; ++t) {
      chunk_base[t][q] = total[q];
      total[q] += chunk_count[t][q];
    }

  auto* h = new SparsetirHyb();
  h->parts = P;
  h->nbk = B;
  h->widths.assign(buckets, buckets + B);
  h->rows.resize(Q); h->cols.resize(Q); h->mask.resize(Q); h->pos.resize(Q);
  for (size_t q = 0; q < Q; ++q) {
    int64_t slots = total[q] * buckets[q % B];
    if (total[q] > INT32_MAX || slots > INT32_MAX) {
      delete h;
      fail("sparsetir_column_part_hyb: bucket %zu exceeds the int32 index space", q);
      return nullptr;
    }
    h->rows[q].assign(static_cast<size_t>(total[q]), 0);
    h->cols[q].assign(static_cast<size_t>(slots), 0);   // padding: column 0
    h->mask[q].assign(static_cast<size_t>(slots), 0);   // padding: mask 0
    h->pos[q].assign(static_cast<size_t>(slots), -1);   // padding: no CSR position
  }

  // Pass 2: fill.  Each thread owns a contiguous row range and hence a contiguous, disjoint
  // range of ELL rows in every array.
  parallel_chunks(T, num_rows, [&](int t, int lo, int hi) {
    std::vector<int64_t> cursor = chunk_base[t];  // next free ELL row per array
    std::vector<int64_t> fill(P);                 // next free slot of the current row, per partition
    for (int i = lo; i < hi; ++i) {
      for (int p = 0; p < P; ++p) {
        int d = degree[static_cast<size_t>(p) * num_rows + i];
        if (d == 0) { fill[p] = -1; continue; }
        int b = bucket_of(buckets, B, d);
        size_t q = static_cast<size_t>(p) * B + b;
        int width = buckets[b];
        int nell = (d + width - 1) / width;
        for (int e = 0; e < nell; ++e) h->rows[q][static_cast<size_t>(cursor[q] + e)] = i;
        fill[p] = cursor[q] * width;
        cursor[q] += nell;
      }
      for (int j = indptr[i]; j < indptr[i + 1]; ++j) {
        int c = indices[j];
        int p = c / part_size;
        int d = degree[static_cast<size_t>(p) * num_rows + i];
        size_t q = static_cast<size_t>(p) * B + bucket_of(buckets, B, d);
        size_t s = static_cast<size_t>(fill[p]++);
        h->cols[q][s] = c;
        h->mask[q][s] = 1;
        h->pos[q][s] = j;
      }
    }
  });
  return h;
}

int64_t sparsetir_hyb_num_rows(const SparsetirHyb* h, int part, int bucket) {
  if (!h || part < 0 || part >= h->parts || bucket < 0 || bucket >= h->nbk) {
    fail("sparsetir_hyb_num_rows: bad handle or index");
    return -1;
  }
  return static_cast<int64_t>(h->rows[static_cast<size_t>(part) * h->nbk + bucket].size());
}

int sparsetir_hyb_copy_bucket(const SparsetirHyb* h, int part, int bucket, int32_t* row_indices,
                              int32_t* col_indices, int32_t* mask, int32_t* csr_pos,
                              const float* csr_data, float* values) {
  if (!h || part < 0 || part >= h->parts || bucket < 0 || bucket >= h->nbk)
    return fail("sparsetir_hyb_copy_bucket: bad handle or index");
  size_t q = static_cast<size_t>(part) * h->nbk + bucket;
  auto copy = [](int32_t* dst, const std::vector<int32_t>& src) {
    if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(int32_t));
  };
  copy(row_indices, h->rows[q]);
  copy(col_indices, h->cols[q]);
  copy(mask, h->mask[q]);
  copy(csr_pos, h->pos[q]);
  if (values) {
    if (!csr_data) return fail("sparsetir_hyb_copy_bucket: values requested without csr_data");
    const auto& pos = h->pos[q];
    for (size_t s = 0; s < pos.size(); ++s) values[s] = pos[s] >= 0 ? csr_data[pos[s]] : 0.0f;
  }
  return 0;
}

void sparsetir_hyb_free(SparsetirHyb* h) { delete h; }

// ---------------------------------------------------------------------------- condense
// Reference: src/sparse/format.cc:353-429.  The reference inserts (col, row) pairs of a tile
// into a std::multimap and walks the distinct columns in ascending order; here the tile's
// pairs are sorted by column instead.  Tiles are independent, so group counts are computed per
// tile first (pass 1) and groups are written at their prefix-sum offsets (pass 2).
int64_t sparsetir_condense(int num_rows, const int32_t* indptr, const int32_t* indices, int t, int g,
                           int32_t* group_indptr, int32_t* tile_indices, int32_t* mask) {
  if (num_rows < 0 || t < 1 || g < 1 || !indptr) return fail("sparsetir_condense: invalid argument");
  const int num_tiles = (num_rows + t - 1) / t;
  std::vector<int64_t> offs(static_cast<size_t>(num_tiles) + 1, 0);
  const int T = resolve_threads(0, num_rows > 0 ? indptr[num_rows] : 0);

  auto distinct_cols = [&](int tile, std::vector<std::pair<int32_t, int32_t>>& buf) {
    int r0 = tile * t, r1 = std::min(num_rows, r0 + t);
    buf.clear();
    for (int i = r0; i < r1; ++i)
      for (int j = indptr[i]; j < indptr[i + 1]; ++j) buf.emplace_back(indices[j], i - r0);
    std::sort(buf.begin(), buf.end());
  };

  parallel_chunks(T, num_tiles, [&](int, int lo, int hi) {
    std::vector<std::pair<int32_t, int32_t>> buf;
    for (int tile = lo; tile < hi; ++tile) {
      distinct_cols(tile, buf);
      int64_t uniq = 0;
      for (size_t k = 0; k < buf.size(); ++k)
        if (k == 0 || buf[k].first != buf[k - 1].first) ++uniq;
      offs[tile + 1] = (uniq + g - 1) / g;
    }
  });
  for (int tile = 0; tile < num_tiles; ++tile) offs[tile + 1] += offs[tile];
  const int64_t groups = offs[num_tiles];
  if (groups > INT32_MAX) return fail("sparsetir_condense: too many groups");
  if (group_indptr)
    for (int tile = 0; tile <= num_tiles; ++tile) group_indptr[tile] = static_cast<int32_t>(offs[tile]);
  if (!tile_indices && !mask) return groups;
  if (!tile_indices || !mask) return fail("sparsetir_condense: tile_indices and mask go together");

  parallel_chunks(T, num_tiles, [&](int, int lo, int hi) {
    std::vector<std::pair<int32_t, int32_t>> buf;
    for (int tile = lo; tile < hi; ++tile) {
      distinct_cols(tile, buf);
      int64_t g0 = offs[tile], g1 = offs[tile + 1];
      std::fill(tile_indices + g0 * g, tile_indices + g1 * g, 0);
      std::fill(mask + g0 * t * g, mask + g1 * t * g, 0);
      int64_t u = -1;
      for (size_t k = 0; k < buf.size(); ++k) {
        if (k == 0 || buf[k].first != buf[k - 1].first) {
          ++u;
          tile_indices[g0 * g + u] = buf[k].first;
        }
        int64_t grp = g0 + u / g, slot = u % g;
        mask[grp * t * g + static_cast<int64_t>(buf[k].second) * g + slot] = 1;
      }
    }
  });
  return groups;
}

}  // extern "C"

// ------------------------------------------------------------------------ csf_to_ell3d
// Reference: src/sparse/format.cc:180-343.  Per relation and column bucket the rows are laid
// out as in the hyb routine (one partition); then for every bucket the relations' blocks are
// concatenated, each block padded to whole groups of `rows_b` ELL rows: row ids by repeating
// the last id, columns and mask by zeros (:299-313).
struct SparsetirEll3d {
  int nbk = 0, num_rels = 0;
  std::vector<int32_t> rows_b, cols_b;
  std::vector<std::vector<int32_t>> indptr, rows, cols, mask;
};

extern "C" {

SparsetirEll3d* sparsetir_csf_to_ell3d(int num_rels, const int32_t* ip0, const int32_t* ix0,
                                       const int32_t* ip1, const int32_t* ix1,
                                       const int32_t* nnz_rows_bkt, const int32_t* nnz_cols_bkt,
                                       int num_buckets) {
  if (num_rels < 0 || num_buckets < 1 || !ip0 || !ip1 || !nnz_rows_bkt || !nnz_cols_bkt) {
    fail("sparsetir_csf_to_ell3d: invalid argument");
    return nullptr;
  }
  for (int b = 0; b < num_buckets; ++b)
    if (nnz_rows_bkt[b] < 1 || nnz_cols_bkt[b] < 1 ||
        (b > 0 && nnz_cols_bkt[b] <= nnz_cols_bkt[b - 1])) {
      fail("sparsetir_csf_to_ell3d: The given nnz_cols_bkt should be ascending.");
      return nullptr;
    }
  const int B = num_buckets;
  auto* h = new SparsetirEll3d();
  h->nbk = B;
  h->num_rels = num_rels;
  h->rows_b.assign(nnz_rows_bkt, nnz_rows_bkt + B);
  h->cols_b.assign(nnz_cols_bkt, nnz_cols_bkt + B);
  h->indptr.assign(B, std::vector<int32_t>(1, 0));
  h->rows.resize(B); h->cols.resize(B); h->mask.resize(B);

  // ELL rows each (bucket, relation) block needs, in groups after padding
  std::vector<int64_t> ell_rows(static_cast<size_t>(B) * std::max(1, num_rels), 0);
  for (int r = 0; r < num_rels; ++r)
    for (int i = ip0[r]; i < ip0[r + 1]; ++i) {
      int d = ip1[i + 1] - ip1[i];
      if (d <= 0) continue;  // a row without entries emits nothing (:250 loop body never runs)
      int b = bucket_of(nnz_cols_bkt, B, d);
      ell_rows[static_cast<size_t>(b) * num_rels + r] += (d + nnz_cols_bkt[b] - 1) / nnz_cols_bkt[b];
    }
  // group-aligned start of every block
  std::vector<int64_t> start(static_cast<size_t>(B) * std::max(1, num_rels), 0);
  for (int b = 0; b < B; ++b) {
    int64_t cur = 0;
    for (int r = 0; r < num_rels; ++r) {
      start[static_cast<size_t>(b) * num_rels + r] = cur;
      int64_t n = ell_rows[static_cast<size_t>(b) * num_rels + r];
      cur += (n + nnz_rows_bkt[b] - 1) / nnz_rows_bkt[b] * nnz_rows_bkt[b];
      h->indptr[b].push_back(static_cast<int32_t>(cur / nnz_rows_bkt[b]));
    }
    if (cur * nnz_cols_bkt[b] > INT32_MAX) {
      delete h;
      fail("sparsetir_csf_to_ell3d: bucket %d exceeds the int32 index space", b);
      return nullptr;
    }
    h->rows[b].assign(static_cast<size_t>(cur), 0);
    h->cols[b].assign(static_cast<size_t>(cur) * nnz_cols_bkt[b], 0);
    h->mask[b].assign(static_cast<size_t>(cur) * nnz_cols_bkt[b], 0);
  }
  // fill; relations are independent
  const int T = resolve_threads(0, num_rels > 0 ? ip1[ip0[num_rels]] : 0);
  parallel_chunks(T, num_rels, [&](int, int lo, int hi) {
    std::vector<int64_t> cursor(B);
    for (int r = lo; r < hi; ++r) {
      for (int b = 0; b < B; ++b) cursor[b] = start[static_cast<size_t>(b) * num_rels + r];
      for (int i = ip0[r]; i < ip0[r + 1]; ++i) {
        int d = ip1[i + 1] - ip1[i];
        if (d <= 0) continue;
        int b = bucket_of(nnz_cols_bkt, B, d);
        int width = nnz_cols_bkt[b];
        int nell = (d + width - 1) / width;
        for (int e = 0; e < nell; ++e) h->rows[b][static_cast<size_t>(cursor[b] + e)] = ix0[i];
        size_t s = static_cast<size_t>(cursor[b]) * width;
        for (int j = ip1[i]; j < ip1[i + 1]; ++j, ++s) {
          h->cols[b][s] = ix1[j];
          h->mask[b][s] = 1;
        }
        cursor[b] += nell;
      }
      // pad the block's row ids up to a whole group with the last id (:299-305)
      for (int b = 0; b < B; ++b) {
        int64_t n = ell_rows[static_cast<size_t>(b) * num_rels + r];
        if (n == 0) continue;
        int64_t end = start[static_cast<size_t>(b) * num_rels + r] +
                      (n + nnz_rows_bkt[b] - 1) / nnz_rows_bkt[b] * nnz_rows_bkt[b];
        int32_t last = h->rows[b][static_cast<size_t>(cursor[b] - 1)];
        for (int64_t e = cursor[b]; e < end; ++e) h->rows[b][static_cast<size_t>(e)] = last;
      }
    }
  });
  return h;
}

int64_t sparsetir_ell3d_num_groups(const SparsetirEll3d* h, int bucket) {
  if (!h || bucket < 0 || bucket >= h->nbk) {
    fail("sparsetir_ell3d_num_groups: bad handle or index");
    return -1;
  }
  return static_cast<int64_t>(h->rows[bucket].size()) / h->rows_b[bucket];
}

int sparsetir_ell3d_copy_bucket(const SparsetirEll3d* h, int bucket, int32_t* indptr,
                                int32_t* row_indices, int32_t* col_indices, int32_t* mask) {
  if (!h || bucket < 0 || bucket >= h->nbk)
    return fail("sparsetir_ell3d_copy_bucket: bad handle or index");
  auto copy = [](int32_t* dst, const std::vector<int32_t>& src) {
    if (dst && !src.empty()) std::memcpy(dst, src.data(), src.size() * sizeof(int32_t));
  };
  copy(indptr, h->indptr[bucket]);
  copy(row_indices, h->rows[bucket]);
  copy(col_indices, h->cols[bucket]);
  copy(mask, h->mask[bucket]);
  return 0;
}

void sparsetir_ell3d_free(SparsetirEll3d* h) { delete h; }

// ----------------------------------------------------------------------- row partition
int sparsetir_row_partition(int num_rows, const int32_t* indptr, int num_shards, int64_t* cuts) {
  if (num_rows < 0 || num_shards < 1 || !indptr || !cuts)
    return fail("sparsetir_row_partition: invalid argument");
  const int64_t nnz = num_rows > 0 ? indptr[num_rows] : 0;
  cuts[0] = 0;
  for (int k = 1; k < num_shards; ++k) {
    int64_t target = nnz * k / num_shards;
    // first row boundary whose prefix is >= target, never before the previous cut
    const int32_t* it = std::lower_bound(indptr, indptr + num_rows + 1, target,
                                         [](int32_t v, int64_t tgt) { return v < tgt; });
    int64_t row = it - indptr;
    if (nnz == 0) row = static_cast<int64_t>(num_rows) * k / num_shards;
    cuts[k] = std::min<int64_t>(std::max(row, cuts[k - 1]), num_rows);
  }
  cuts[num_shards] = num_rows;
  return 0;
}

}  // extern "C"

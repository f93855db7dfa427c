/*
 * sparsetir_b200 — C ABI of the B200 (sm_100a) sparse-operator library.
 *
 * The library replaces the functions SparseTIR *builds* for its sparse operators (CSR SpMM,
 * hyb/ELL SpMM, SDDMM, BSR SpMM, RGMS) and its host-side format conversion routines.  A
 * built SparseTIR operator is a DSO symbol of type TVMBackendPackedCFunc
 * (reference: include/tvm/runtime/c_backend_api.h:49-51) that LibraryModule wraps into a
 * PackedFunc (src/runtime/library_module.cc:74-86).  Every `sparsetir_*` operator symbol below
 * has exactly that type and takes the arguments of the reference function it stands in for,
 * in the reference's order.  Plain-pointer `*_raw` twins take device pointers and sizes.
 *
 * Conventions shared by all operator entry points (they are those of the host stub the
 * reference generates, src/tir/transforms/make_packed_api.cc:138-305 and
 * src/tir/transforms/arg_binder.cc:152-282):
 *   - array arguments are DLTensor* (type code kTVMDLTensorHandle, kTVMNDArrayHandle or
 *     kTVMOpaqueHandle); every buffer is flat and compact (strides NULL or compact,
 *     byte_offset 0); all arrays live on the same CUDA device;
 *   - integer scalars arrive as kTVMArgInt in v_int64;
 *   - all tensors are borrowed for the duration of the call; outputs are caller-allocated;
 *   - the call is asynchronous on the stream registered with sparsetir_set_stream for that
 *     device (default: the legacy default stream); no synchronisation inside;
 *   - returns 0, or -1 after recording a message readable with sparsetir_get_last_error
 *     (reference: TVMAPISetLastError / TVMGetLastError, src/runtime/c_runtime_api.cc:371-386).
 * There is no CPU fallback: a non-CUDA tensor is an error.
 */
#ifndef SPARSETIR_B200_H_
#define SPARSETIR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define SPARSETIR_API
#else
#define SPARSETIR_API __attribute__((visibility("default")))
#endif

/* ---- DLPack tensor (layout identical in DLPack 0.x and 1.x) -------------------------- */
#ifndef DLPACK_DLPACK_H_
typedef enum { kDLCPU = 1, kDLCUDA = 2, kDLCUDAHost = 3 } SpDLDeviceType;
typedef struct { int32_t device_type; int32_t device_id; } DLDevice;
typedef enum { kDLInt = 0U, kDLUInt = 1U, kDLFloat = 2U } SpDLDataTypeCode;
typedef struct { uint8_t code; uint8_t bits; uint16_t lanes; } DLDataType;
typedef struct {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
} DLTensor;
#endif

/* ---- TVM PackedFunc calling convention (include/tvm/runtime/c_runtime_api.h:110-151) -- */
#ifndef TVM_RUNTIME_C_RUNTIME_API_H_
typedef enum {
  kTVMArgInt = 0U,
  kTVMArgFloat = 2U,
  kTVMOpaqueHandle = 3U,
  kTVMNullptr = 4U,
  kTVMDLTensorHandle = 7U,
  kTVMNDArrayHandle = 13U
} SpTVMArgTypeCode;
typedef union {
  int64_t v_int64;
  double v_float64;
  void* v_handle;
  const char* v_str;
  DLDataType v_type;
  DLDevice v_device;
} TVMValue;
#endif

#define SPARSETIR_PACKED_ARGS                                                              \
  TVMValue *args, int *type_codes, int num_args, TVMValue *out_ret_value, int *out_ret_tcode, \
      void *resource_handle

/* ---- runtime glue -------------------------------------------------------------------- */

/* Message of the last failed call on this thread (TVMGetLastError,
 * include/tvm/runtime/c_runtime_api.h:195). */
SPARSETIR_API const char* sparsetir_get_last_error(void);

/* Stream used by later packed calls of the CALLING THREAD for `device_id` (TVMSetStream,
 * include/tvm/runtime/c_runtime_api.h:496; the reference keeps it in the thread-local
 * CUDAThreadEntry, src/runtime/cuda/cuda_device_api.cc:209-211, read at launch time,
 * src/runtime/cuda/cuda_module.cc:170).  `stream` is a cudaStream_t; NULL selects the legacy
 * default stream.  A thread that never called sparsetir_set_stream for a device uses the
 * process-wide default set with sparsetir_set_default_stream (initially the legacy default
 * stream).  sparsetir_get_stream returns what the calling thread's next packed call would use.
 * The `*_raw` entry points take their stream as an argument and ignore both. */
SPARSETIR_API int sparsetir_set_stream(int device_id, void* stream);
SPARSETIR_API int sparsetir_set_default_stream(int device_id, void* stream);
SPARSETIR_API void* sparsetir_get_stream(int device_id);

/* Scratch memory (no counterpart in the reference, whose generated functions allocate through
 * TVMBackendAllocWorkspace, include/tvm/runtime/c_backend_api.h:84).  Some operators keep an
 * intermediate in device memory owned by the library: one grow-only buffer (and one small buffer
 * of counters) per (device, stream), allocated by the first call that needs it and enlarged by a
 * call that needs more — cudaMalloc / cudaFree inside that call, which synchronise the device and
 * fail while the stream is being captured into a CUDA graph.  A caller that wants neither reserves
 * the buffers up front: after sparsetir_reserve_workspace(device, stream, s, c) no call on that
 * stream that needs at most s scratch bytes and c counter bytes allocates, synchronises or frees.
 * The *_workspace queries give the sizes an operator call needs (upper bounds). */
SPARSETIR_API int sparsetir_reserve_workspace(int device_id, void* stream, size_t scratch_bytes,
                                              size_t counter_bytes);

/* Deep checks of the index arrays (no counterpart in the reference, whose host stub checks
 * shapes, dtypes and devices only, src/tir/transforms/arg_binder.cc:152-282).  When switched on —
 * sparsetir_set_validate(1), or SPARSETIR_VALIDATE=1 in the environment when the library is first
 * used — every operator call first verifies on the device that its row pointers start at 0, never
 * decrease and end at the number of stored entries, and that every column / row id lies inside its
 * range; a violation makes the call return -1 with a message naming the array and the position,
 * before any kernel that would follow the bad index runs.  Costs a pass over the index arrays and
 * a stream synchronisation per call; not usable while the stream is being captured. */
SPARSETIR_API int sparsetir_set_validate(int on);

/* Sending half of an all-gather of row shards over NVLink (no counterpart in the reference, whose
 * operators run on one device).  Copies `bytes` bytes (a multiple of 4) at `src`, in the memory of
 * GPU `device_id`, to each of the `n_peers` addresses in `peer_dst`: peer-mapped device pointers
 * (CUDA IPC, cuMemMap or a symmetric-memory allocation) at which the other GPUs expect this GPU's
 * block.  One kernel on `stream` reads the block once and stores it to every peer; it waits on
 * nothing.  A GPU's buffer is complete once every peer's call has finished: order that between the
 * ranks (a stream-ordered barrier such as a one-element all-reduce).  Returns 0, or -1 with the
 * error string set. */
#define SPARSETIR_MAX_PEERS 15
SPARSETIR_API int sparsetir_peer_scatter(int device_id, void* stream, const void* src, size_t bytes,
                                         int n_peers, void* const* peer_dst);

/* Library version and the compute capability the kernels were compiled for (100). */
SPARSETIR_API int sparsetir_version(void);
SPARSETIR_API int sparsetir_sm_arch(void);

/* Health check of the tensor-core kernels (no counterpart in the reference): every wait on a
 * hardware barrier inside them is bounded, and a wait that runs out is counted instead of
 * hanging the GPU.  Synchronises `device_id` and stores the count since the library was loaded
 * (0 in a healthy run). */
SPARSETIR_API int sparsetir_tc_timeouts(int device_id, unsigned int* count);

/* ---- operators (TVMBackendPackedCFunc symbols) ---------------------------------------- */

/* CSR SpMM, fp32.  C[i,:] = sum_{p in row i} A[p] * B[indices[p],:]; rows without entries are
 * written as zeros.
 * args: (a f32[nnz], b f32[n*feat], c f32[m*feat], indptr i32[m+1], indices i32[nnz]
 *        [, m, n, feat_size, nnz])  — the trailing four integers may be omitted when
 *        m >= 1 (feat_size is then len(c)/m).
 * Replaces the function built from `csrmm`
 * (tests/python/sparsetir/sparse_tir_scripts.py:22-44; flat signature
 * tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:22-39). */
SPARSETIR_API int sparsetir_csrmm(SPARSETIR_PACKED_ARGS);

/* Decomposed hyb (column-partitioned, ELL-bucketed) SpMM, fp32, one launch for all buckets.
 * For every bucket q, ELL row r, slot s: C[rows_q[r],:] += W_q[r,s] * B[cols_q[r,s],:].
 * args: (b f32[n*feat], c f32[m*feat], {w_q f32[nrows_q*width_q], rows_q i32[nrows_q],
 *        cols_q i32[nrows_q*width_q]} x K, feat_size [, flags])
 * The bucket width is len(cols_q)/len(rows_q); buckets with no rows are accepted.
 * Without SPARSETIR_HYB_ALL_ATOMIC every output row that occurs in a bucket is WRITTEN by exactly
 * one writer (pieces of wide and split rows are added in a fixed order first), so results are
 * bit-identical from call to call and C needs no clearing between calls; rows that occur in no
 * bucket are left as the caller filled them (zero, examples/spmm/bench_spmm.py:206).  A row id
 * may repeat only in consecutive ELL rows of the widest bucket, as ColumnPartHyb emits split rows
 * (src/sparse/format.cc:110-116); any other repetition needs SPARSETIR_HYB_ALL_ATOMIC.
 * flags (bit field, default 0):
 *   SPARSETIR_HYB_ZERO_C       the call zero-fills all of C first;
 *   SPARSETIR_HYB_REARM        with ALL_ATOMIC: the call zero-fills C first, so that repeated
 *                              calls stay correct; without ALL_ATOMIC nothing needs re-arming
 *                              (the fallback kernels for odd shapes clear the rows they add to);
 *   SPARSETIR_HYB_ALL_ATOMIC   every contribution is added atomically into C, which the caller
 *                              has zero-filled (needed when the same row occurs in several
 *                              buckets, i.e. with more than one column partition).
 * Uses library scratch memory for split rows (see sparsetir_reserve_workspace).
 * Replaces the function built by examples/spmm/bench_spmm.py:116-199 (argument list :207-222). */
SPARSETIR_API int sparsetir_hyb_spmm(SPARSETIR_PACKED_ARGS);
/* The same operator for one shard of a row-sharded A whose output every GPU wants whole: each
 * finished row of C is stored on this GPU and, by the same kernel, at the same offset of every
 * peer's copy of C — the sending half of the all-gather rides on the SpMM's own stores over NVLink
 * instead of following it as a copy (no counterpart in the reference, which has one device).
 * args: as sparsetir_hyb_spmm with feat_size AND flags given, then one integer per peer: the
 *       peer-mapped address (CUDA IPC, cuMemMap, symmetric memory) at which that peer keeps this
 *       call's c, aligned like c.  1 to SPARSETIR_MAX_PEERS peers.
 * Needs the one-writer kernel: 16-byte aligned b and c, feat_size a multiple of 32, bucket widths
 * 1, 2, 4 or multiples of 8, flags without ZERO_C and ALL_ATOMIC; otherwise -1, and the caller
 * runs sparsetir_hyb_spmm followed by sparsetir_peer_scatter.  The kernel waits on nothing; a
 * GPU's copy is complete when every peer's call has finished (order that between the ranks). */
SPARSETIR_API int sparsetir_hyb_spmm_peers(SPARSETIR_PACKED_ARGS);
#define SPARSETIR_HYB_ZERO_C 1
#define SPARSETIR_HYB_REARM 2
#define SPARSETIR_HYB_ALL_ATOMIC 4
#define SPARSETIR_HYB_MAX_BUCKETS 64

/* SDDMM, fp32.  C[p] = sum_k A[row(p),k] * B[indices[p],k].
 * args: (a f32[m*feat], b f32[n*feat], c f32[nnz], indptr i32[m+1], indices i32[nnz]
 *        [, m, n, feat_size, nnz] [, scale f32[nnz]])
 * A trailing tensor argument, when present, is a per-edge factor multiplied into the result
 * (not part of the reference operator).
 * Replaces the functions built from `sddmm` / `fused_sddmm`
 * (tests/python/sparsetir/sparse_tir_scripts.py:268-318; flat signature
 * tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:458-475). */
SPARSETIR_API int sparsetir_sddmm(SPARSETIR_PACKED_ARGS);
/* SDDMM for one shard of a row-sharded graph whose per-position result every GPU wants whole:
 * every finished c[p] is also stored at the same offset of each peer's copy of c, by the kernel
 * that computes it (see sparsetir_hyb_spmm_peers).
 * args: (a, b, c, indptr, indices, peer_c_0 ... peer_c_{P-1} [, scale]): the five tensors of
 *       sparsetir_sddmm (sizes inferred from their lengths), then one integer per peer: the
 *       peer-mapped address of that peer's copy of this call's c (4-byte aligned), 1 to
 *       SPARSETIR_MAX_PEERS of them; then the optional per-position factor.
 * Needs feat_size a multiple of 32 and 32-byte aligned a and b; otherwise -1, and the caller runs
 * sparsetir_sddmm followed by sparsetir_peer_scatter. */
SPARSETIR_API int sparsetir_sddmm_peers(SPARSETIR_PACKED_ARGS);

/* Edge -> row lookup, the preprocess kernel of fused SDDMM:
 * mid[p] = upper_bound(indptr, p) - 1.
 * args: (indptr i32[m+1], mid i32[nnz])
 * Replaces the binary-search block emitted by LowerSparseIter
 * (src/tir/transforms/lower_sparse_iter.cc:768-783; golden
 * tests/python/sparsetir/sparse_tir_lowered_buffer_scripts.py:530-549). */
SPARSETIR_API int sparsetir_sddmm_edge_to_row(SPARSETIR_PACKED_ARGS);

/* BSR SpMM, fp16 blocks and dense operand, fp32 accumulation and output.
 * C[i*blk+bi, f] = sum_{p in block-row i} sum_bj A[p,bi,bj] * B[indices[p]*blk+bj, f].
 * args: (a f16[nnzb*blk*blk], b f16[mb*blk*feat], c f32[nb*blk*feat], indptr i32[nb+1],
 *        indices i32[nnzb], nb, mb, nnzb, blk, feat_size)
 * (nb = block rows of A and C, mb = block rows of B, the reference's naming.)
 * Replaces the function built from `bsrmm`
 * (tests/python/sparsetir/sparse_tir_scripts.py:114-146; call examples/blocksparse/bsr_spmm.py:432). */
SPARSETIR_API int sparsetir_bsrmm(SPARSETIR_PACKED_ARGS);

/* RGMS (relational gather-matmul-scatter), fp32.
 * Y[I[i], fo] += sum_{p in CSF row i of relation r} A[p] * sum_fi W[r,fo,fi] * X[J[p],fi],
 * accumulated over all relations into the caller's Y (zero-filled by the caller, as
 * examples/rgms/rgcn/bench_rgcn_non_composable.py:88-90 does).
 * args: (a f32[nnz_j], w f32[R*feat*feat], x f32[n*feat], y f32[m*feat], indptr_i i32[R+1],
 *        indices_i i32[nnz_i], indptr_j i32[nnz_i+1], indices_j i32[nnz_j]
 *        [, m, n, num_rels, feat_size, nnz_i, nnz_j])  — feat_size is inferred from
 *        len(w) = R*feat^2 when the scalars are omitted.
 * Replaces the function built from `rgcn_hetero_forward`
 * (tests/python/sparsetir/sparse_tir_scripts.py:468-499; call
 * examples/rgms/rgcn/bench_rgcn_non_composable.py:108). */
SPARSETIR_API int sparsetir_rgms(SPARSETIR_PACKED_ARGS);

/* Row sums of a CSR matrix: b[i] = sum of the stored entries of row i.
 * args: (a f32[nnz], b f32[n], indptr i32[n+1] [, indices i32[nnz]] [, n [, m], nnz]).  Replaces the
 * functions built from `segment_reduce` and `csr_reduce`
 * (tests/python/sparsetir/sparse_tir_scripts.py:74-110). */
SPARSETIR_API int sparsetir_csr_reduce(SPARSETIR_PACKED_ARGS);

/* Row-wise softmax over the stored entries, exactly as the reference defines it:
 *   b[i,j] = exp(a[i,j]) / sum_j exp(a[i,j] - max_j a[i,j])
 * (the numerator is not shifted by the row maximum: tests/python/sparsetir/sparse_tir_scripts.py:503-528).
 * args: (a f32[nnz], b f32[nnz], indptr i32[n+1], indices i32[nnz] [, n, nnz]). */
SPARSETIR_API int sparsetir_sparse_softmax(SPARSETIR_PACKED_ARGS);

/* Scatter of the entries of a CSR matrix into the blocks of a BSR matrix with a given block
 * structure; elements no entry maps to are left untouched.
 * args: (a f32[nnz_in], b f32[nnz_out*blk*blk], indptr_in, indices_in, indptr_out, indices_out,
 *        [m_in, n_in, m_out, n_out, nnz_in, nnz_out,] blk_size)
 * (`csr2bsr`, tests/python/sparsetir/sparse_tir_scripts.py:532-557). */
SPARSETIR_API int sparsetir_csr2bsr(SPARSETIR_PACKED_ARGS);

/* Block-ELL SpMM, fp32: c[i,bi,f] = sum_{j<col} sum_bj a[i,j,bi,bj] * b[indices[i,j],bj,f].
 * args: (a f32[nb*col*blk*blk], b f32[mb*blk*feat], c f32[nb*blk*feat], indices i32[nb*col],
 *        nb, mb, feat_size, col, blk)   (`ellmm`, tests/python/sparsetir/sparse_tir_scripts.py:150-181). */
SPARSETIR_API int sparsetir_ellmm(SPARSETIR_PACKED_ARGS);

/* Sparse attention over the stored positions of a CSR pattern, fp32, one pass:
 *   o[i,:] = sum_j P[i,j] v[j,:],  P[i,j] = exp(<q[i,:],k[j,:]>) / sum_j exp(<q[i,:],k[j,:]> - row max)
 * (SDDMM, the reference's sparse softmax and SpMM as one function).
 * args: (q f32[m*feat], k f32[n*feat], v f32[n*feat], o f32[m*feat], indptr i32[m+1],
 *        indices i32[nnz] [, m, n, nnz, feat_size]).  Replaces the function built from `fusedmm`
 * (examples/flash_graph_attention/fusedmm.py:37-96). */
SPARSETIR_API int sparsetir_fusedmm(SPARSETIR_PACKED_ARGS);

/* Condensed tensor-core SpMM ("tcspmm"), fp16 operands, fp32 accumulation:
 *   C[io*t + ii, f] = sum_{jo in [indptr[io], indptr[io+1])} sum_{ji < g} A[jo,ii,ji] * B[indices[jo*g+ji], f]
 * args: (a f16[nnzb*t*g], b f16[nb*g*feat], c f16 or f32 [mb*t*feat], indptr i32[mb+1],
 *        indices i32[nnzb*g], mb, nb, nnzb, feat_size, tile_size, group_size)
 * with (indptr, indices, a) as ConDense returns them (group_indptr, tile_indices, mask).  Replaces
 * the function built from `tcspmm` (examples/spmm/bench_tc_spmm.py:537-565, call :641-648). */
SPARSETIR_API int sparsetir_tcspmm(SPARSETIR_PACKED_ARGS);

/* RGMS over the decomposed ELL3D format, fp32: for every bucket b, group g, row slot ii,
 * column slot j:  Y[rows_b[g,ii], fo] += A_b[g,ii,j] * sum_fi W[mid_b[g],fo,fi] * X[cols_b[g,ii,j],fi].
 * args: (w f32[R*feat*feat], x f32[n*feat], y f32[m*feat],
 *        {a f32[G_b*rows_b*cols_b], rows i32[G_b*rows_b], cols i32[G_b*rows_b*cols_b]} x K,
 *        {mid i32[G_b]} x K, feat_size) — the argument list of the function built in
 * examples/rgms/rgcn/bench_rgcn_composable.py:196-208 (buckets from CSFToELL3D, `mid` = relation
 * of every group, :40-45), plus feat_size.  Accumulates into the caller's zero-filled y. */
SPARSETIR_API int sparsetir_rgms_ell3d(SPARSETIR_PACKED_ARGS);

/* The same over half-precision operands with rectangular weights:
 *   Y[rows_b[g,ii], fo] += A_b[g,ii,j] * sum_fi X[cols_b[g,ii,j], fi] * W[mid_b[g], fi, fo]
 * args: (w f16[R*feat_in*feat_out], x f16[n*feat_in], y f16 or f32 [m*feat_out],
 *        {a f16[G_b*rows_b*cols_b], rows i32[G_b*rows_b], cols i32[G_b*rows_b*cols_b]} x K,
 *        {mid i32[G_b]} x K, feat_in, feat_out) — the argument list of the function built by
 * rgcn_tensorcore (examples/rgms/rgcn/bench_rgcn_tensorcore.py:842-852; computation :564-609),
 * which the sparse convolution driver calls with one relation per kernel offset and buckets = [1]
 * (examples/rgms/sparse_conv/sparse_conv.py:93-125), plus the two feature sizes.  Products are
 * accumulated in fp32; accumulates into the caller's zero-filled y. */
SPARSETIR_API int sparsetir_rgms_ell3d_f16(SPARSETIR_PACKED_ARGS);

/* ---- operators, plain-pointer form (device pointers; stream is a cudaStream_t) -------- */
SPARSETIR_API int sparsetir_csrmm_raw(const float* a, const float* b, float* c,
                                      const int32_t* indptr, const int32_t* indices, int m, int n,
                                      int feat, int nnz, int device_id, void* stream);

typedef struct {
  const float* w;      /* [nrows*width] */
  const int32_t* rows; /* [nrows] */
  const int32_t* cols; /* [nrows*width] */
  int32_t nrows;
  int32_t width;
} SparsetirEllBucket;
SPARSETIR_API int sparsetir_hyb_spmm_raw(const float* b, float* c, const SparsetirEllBucket* buckets,
                                         int num_buckets, int m, int n, int feat, int flags,
                                         int device_id, void* stream);
/* sparsetir_hyb_spmm_peers without the packed layer: peer_c[k] is peer k's copy of c. */
SPARSETIR_API int sparsetir_hyb_spmm_peers_raw(const float* b, float* c,
                                               const SparsetirEllBucket* buckets, int num_buckets,
                                               int m, int n, int feat, int flags, int n_peers,
                                               void* const* peer_c, int device_id, void* stream);
/* Scratch and counter bytes sparsetir_hyb_spmm(_raw) uses for this bucket table and feature size
 * (non-zero only when the widest bucket may hold rows split into several ELL rows). */
SPARSETIR_API int sparsetir_hyb_spmm_workspace(const SparsetirEllBucket* buckets, int num_buckets,
                                               int feat, size_t* scratch_bytes,
                                               size_t* counter_bytes);
/* The feature tile the main hyb kernel uses for 16/32-byte aligned operands with n rows of b:
 * `lanes` lanes of `lane_floats` floats each (the kernel is hyb_spmm_lean_kernel<lanes, lane_floats>,
 * launched with feat / (lanes * lane_floats) tiles in grid.y).  For tools that match a launch with
 * a profile. */
SPARSETIR_API int sparsetir_hyb_spmm_tile(int n, int feat, int* lanes, int* lane_floats);
SPARSETIR_API int sparsetir_sddmm_raw(const float* a, const float* b, float* c,
                                      const int32_t* indptr, const int32_t* indices,
                                      const float* scale, int m, int n, int feat, int nnz,
                                      int device_id, void* stream);
SPARSETIR_API int sparsetir_sddmm_peers_raw(const float* a, const float* b, float* c,
                                            const int32_t* indptr, const int32_t* indices,
                                            const float* scale, int m, int n, int feat, int nnz,
                                            int n_peers, void* const* peer_c, int device_id,
                                            void* stream);
SPARSETIR_API int sparsetir_sddmm_edge_to_row_raw(const int32_t* indptr, int32_t* mid, int m,
                                                  int nnz, int device_id, void* stream);
SPARSETIR_API int sparsetir_bsrmm_raw(const void* a_f16, const void* b_f16, float* c,
                                      const int32_t* indptr, const int32_t* indices, int nb,
                                      int mb, int nnzb, int blk, int feat, int device_id,
                                      void* stream);
/* Scratch bytes sparsetir_rgms(_raw) uses (see sparsetir_reserve_workspace; no counters). */
SPARSETIR_API int sparsetir_rgms_workspace(int feat, int nnz_i, size_t* scratch_bytes);
SPARSETIR_API int sparsetir_rgms_raw(const float* a, const float* w, const float* x, float* y,
                                     const int32_t* indptr_i, const int32_t* indices_i,
                                     const int32_t* indptr_j, const int32_t* indices_j, int m,
                                     int n, int num_rels, int feat, int nnz_i, int nnz_j,
                                     int device_id, void* stream);

SPARSETIR_API int sparsetir_csr_reduce_raw(const float* a, float* b, const int32_t* indptr, int n,
                                           int nnz, int device_id, void* stream);
SPARSETIR_API int sparsetir_sparse_softmax_raw(const float* a, float* b, const int32_t* indptr, int n,
                                               int nnz, int device_id, void* stream);
SPARSETIR_API int sparsetir_csr2bsr_raw(const float* a, float* b, const int32_t* indptr_in,
                                        const int32_t* indices_in, const int32_t* indptr_out,
                                        const int32_t* indices_out, int m_in, int nnz_in, int blk,
                                        int device_id, void* stream);
SPARSETIR_API int sparsetir_ellmm_raw(const float* a, const float* b, float* c, const int32_t* indices,
                                      int nb, int mb, int feat, int col, int blk, int device_id,
                                      void* stream);
SPARSETIR_API int sparsetir_fusedmm_raw(const float* q, const float* k, const float* v, float* o,
                                        const int32_t* indptr, const int32_t* indices, int m, int n,
                                        int nnz, int feat, int device_id, void* stream);
SPARSETIR_API int sparsetir_tcspmm_raw(const void* a_f16, const void* b_f16, void* c, int c_is_f16,
                                       const int32_t* indptr, const int32_t* indices, int mb, int nb,
                                       int nnzb, int feat, int tile_size, int group_size,
                                       int device_id, void* stream);

/* RGMS over ELL3D buckets (the decomposed form of examples/rgms/rgcn/bench_rgcn_composable.py:
 * per bucket the arrays CSFToELL3D returns plus the relation id of every group, :40-45).
 * a/cols are [num_groups*rows_per_group*cols_per_row], rows [num_groups*rows_per_group],
 * mid [num_groups] ascending.  Accumulates into y. */
typedef struct {
  const float* a;
  const int32_t* rows;
  const int32_t* cols;
  const int32_t* mid;
  int32_t num_groups;
  int32_t rows_per_group;
  int32_t cols_per_row;
} SparsetirEll3dBucket;
SPARSETIR_API int sparsetir_rgms_ell3d_raw(const float* w, const float* x, float* y,
                                           const SparsetirEll3dBucket* buckets, int num_buckets,
                                           int m, int n, int num_rels, int feat, int device_id,
                                           void* stream);

/* Half-precision operands, rectangular weights w[num_rels][feat_in][feat_out]; y is fp16 when
 * y_is_f16 is non-zero, fp32 otherwise.  `a` points to fp16 values. */
typedef struct {
  const void* a;
  const int32_t* rows;
  const int32_t* cols;
  const int32_t* mid;
  int32_t num_groups;
  int32_t rows_per_group;
  int32_t cols_per_row;
} SparsetirEll3dBucketH;
SPARSETIR_API int sparsetir_rgms_ell3d_f16_raw(const void* w, const void* x, void* y, int y_is_f16,
                                               const SparsetirEll3dBucketH* buckets, int num_buckets,
                                               int m, int n, int num_rels, int feat_in, int feat_out,
                                               int device_id, void* stream);

/* RGMS that never allocates device memory.  No counterpart in the reference: it exists for
 * hosts that may not call the CUDA allocator when they need the operator (loops that forbid
 * allocation after start-up; processes whose device memory belongs to another pool).
 * Same arguments and result as sparsetir_rgms_raw, but the intermediate of the two-launch form
 * lives in a fixed 32 MiB array inside the library instead of an allocated scratch buffer:
 *   - feat must be 64 and nnz_i at most 131072; anything else is refused with an error;
 *   - all calls on one device share that array: calls that overlap on the GPU race, order them;
 *   - the first call on a device fetches the array's address, which is also when the 32 MiB are
 *     taken on that device: make it at start-up, while memory is free, and before any stream
 *     capture. */
SPARSETIR_API int sparsetir_rgms_noalloc(const float* a, const float* w, const float* x, float* y,
                                         const int32_t* indptr_i, const int32_t* indices_i,
                                         const int32_t* indptr_j, const int32_t* indices_j, int m,
                                         int n, int num_rels, int feat, int nnz_i, int nnz_j,
                                         int device_id, void* stream);

/* ---- host-side format conversion (CPU int32 arrays) ----------------------------------- */

/* Column partitioning + ELL bucketing of a CSR matrix, bit-exact with ColumnPartHyb
 * (src/sparse/format.cc:46-168; Python wrapper python/tvm/sparse/format.py:89-116).
 * The reference returns Array<Array<Array<NDArray>>>; without TVM's object system the result
 * is an opaque handle that is queried per (partition, bucket) and then freed.
 *   indptr i32[num_rows+1], indices i32[nnz]  host memory
 *   buckets: ascending ELL widths;  num_threads <= 0 selects the hardware concurrency.
 * Returns NULL after recording an error. */
typedef struct SparsetirHyb SparsetirHyb;
SPARSETIR_API SparsetirHyb* sparsetir_column_part_hyb(int num_rows, int num_cols,
                                                      const int32_t* indptr,
                                                      const int32_t* indices, int num_col_parts,
                                                      const int32_t* buckets, int num_buckets,
                                                      int num_threads);
/* number of ELL rows of bucket (part, bucket) */
SPARSETIR_API int64_t sparsetir_hyb_num_rows(const SparsetirHyb* h, int part, int bucket);
/* Copies the bucket's arrays into caller buffers (any may be NULL):
 * row_indices i32[nrows], col_indices i32[nrows*width], mask i32[nrows*width] are the
 * reference's three outputs (format.cc:146-149); csr_pos i32[nrows*width] is the CSR position
 * each slot came from (-1 for padding) — the gather index of the reference's rewrite_A copy
 * blocks (src/tir/transforms/sparse_format_decompose.cc:242-268); values f32[nrows*width] is
 * csr_data[csr_pos] (0 for padding) when csr_data is non-NULL. */
SPARSETIR_API int sparsetir_hyb_copy_bucket(const SparsetirHyb* h, int part, int bucket,
                                            int32_t* row_indices, int32_t* col_indices,
                                            int32_t* mask, int32_t* csr_pos,
                                            const float* csr_data, float* values);
SPARSETIR_API void sparsetir_hyb_free(SparsetirHyb* h);

/* TC-GNN style condensing, bit-exact with ConDense (src/sparse/format.cc:353-429; wrapper
 * python/tvm/sparse/format.py:119-139).  Two-call pattern: with tile_indices == NULL only the
 * number of groups is returned; group_indptr i32[ceil(n/t)+1], tile_indices i32[groups*g],
 * mask i32[groups*t*g].  Returns the number of groups, or -1 on error. */
SPARSETIR_API int64_t sparsetir_condense(int num_rows, const int32_t* indptr, const int32_t* indices,
                                         int t, int g, int32_t* group_indptr,
                                         int32_t* tile_indices, int32_t* mask);

/* 3-level CSF -> per-bucket ELL3D, bit-exact with CSFToELL3D (src/sparse/format.cc:180-343;
 * wrapper python/tvm/sparse/format.py:142-170).  Opaque handle like column_part_hyb. */
typedef struct SparsetirEll3d SparsetirEll3d;
SPARSETIR_API SparsetirEll3d* sparsetir_csf_to_ell3d(int num_rels, const int32_t* csf_indptr_0,
                                                     const int32_t* csf_indices_0,
                                                     const int32_t* csf_indptr_1,
                                                     const int32_t* csf_indices_1,
                                                     const int32_t* nnz_rows_bkt,
                                                     const int32_t* nnz_cols_bkt, int num_buckets);
SPARSETIR_API int64_t sparsetir_ell3d_num_groups(const SparsetirEll3d* h, int bucket);
/* indptr i32[num_rels+1], row_indices i32[groups*rows_b], col_indices / mask
 * i32[groups*rows_b*cols_b] */
SPARSETIR_API int sparsetir_ell3d_copy_bucket(const SparsetirEll3d* h, int bucket, int32_t* indptr,
                                              int32_t* row_indices, int32_t* col_indices,
                                              int32_t* mask);
SPARSETIR_API void sparsetir_ell3d_free(SparsetirEll3d* h);

/* ---- multi-GPU row partitioning (no counterpart in the reference, which is single-GPU) - */

/* nnz-balanced contiguous row cuts: cuts[k] = first row of shard k (cuts[0] = 0,
 * cuts[num_shards] = num_rows), chosen so that indptr[cuts[k]] is the first row boundary at or
 * after k*nnz/num_shards.  cuts i64[num_shards+1]. */
SPARSETIR_API int sparsetir_row_partition(int num_rows, const int32_t* indptr, int num_shards,
                                          int64_t* cuts);

#ifdef __cplusplus
}
#endif
#endif /* SPARSETIR_B200_H_ */

/*
 * annc_b200 -- C ABI of the B200 (sm_100a) implementation of the custom operators
 * that ANNC's XLA and TF-Grappler passes route to.
 *
 * Three groups of entry points:
 *
 *  (1) The reference's own symbols, same names and signatures, so that graphs
 *      rewritten by annc-opt / the ANNC passes dispatch here unchanged:
 *      the XLA custom-call targets (`void f(void* out, const void** in)`), the
 *      XLA:CPU runtime symbols of the kernel selector and the softmax.  They
 *      are declared at the end of this file; the C++-mangled aliases that the
 *      reference's MLIR lowering calls are defined in the library as well.
 *  (2) Plain-C twins of the TensorFlow fused ops (`annc_KPFused...`): inputs as
 *      `annc_tensor` views, outputs obtained through an allocation callback that
 *      plays the role of OpKernelContext::allocate_output, status + message in
 *      place of OP_REQUIRES.
 *  (3) Device-pointer entry points (`*_dev`, `annc_gemm_run`): no staging, no
 *      allocation, explicit stream.  The roofline figures are measured on these.
 *
 * Pointer rule for groups (1) and (2): every data pointer may be host memory or
 * device memory.  Device buffers are used in place on the calling thread's stream
 * (annc_set_stream).  A host operand gets a device mirror keyed by (pointer, bytes, device)
 * that persists between calls (the reference's callers keep their buffers: XLA buffer
 * assignment, TF variables), results are copied back before the call returns.  An upload is
 * skipped when a sampled fingerprint of the host contents (one 8-byte word per 4 KiB page, at
 * most 16384 pages, plus the first and last 64 bytes) equals the one taken when the mirror was
 * last filled: weights and tables upload once, and an output that comes back unchanged as an
 * input of the next call is not uploaded at all.  The fingerprint is a sample, not a proof: a
 * caller that rewrites part of a buffer in place between two calls, leaving every sampled word
 * as it was, must select mode 0 or 1 with annc_set_operand_cache.  One thread keeps one stream,
 * or synchronises before changing it (calls made with device pointers only do not wait for
 * the stream; a later call on another stream is ordered after them by an event).  There is no
 * CPU fallback anywhere: without a CUDA device every compute entry point fails with
 * ANNC_ERR_CUDA.
 *
 * Reference citations are paths inside the ANNC project.
 */
#ifndef ANNC_B200_H_
#define ANNC_B200_H_

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- status */

enum {
  ANNC_OK = 0,
  ANNC_ERR_INVALID_ARGUMENT = 3, /* tensorflow errors::InvalidArgument */
  ANNC_ERR_INTERNAL = 13,        /* tensorflow errors::Internal        */
  ANNC_ERR_CUDA = 100,           /* CUDA runtime/driver failure        */
  ANNC_ERR_TIMEOUT = 101,        /* a bounded device-side wait ran out */
  ANNC_ERR_UNSUPPORTED = 102
};

/* Message of the last failing call on this thread (the reference's OP_REQUIRES
 * text where there is one).  Valid until the next call on the same thread. */
const char* annc_last_error(void);

/* Version string "annc_b200 <semver> sm_100a". */
const char* annc_version(void);

/* Stream used by the calling thread for groups (1) and (2); NULL = default stream. */
void annc_set_stream(void* cuda_stream);
void* annc_get_stream(void);

/* Uploads `bytes` at host pointer `ptr` now and pins the mirror: later calls that receive
 * (`ptr`, `bytes`) use the device copy without looking at the host contents again, and the
 * mirror is never evicted (XLA constants / parameters and TF variables keep their address for
 * the lifetime of the executable).  annc_unregister_constant drops it. */
int annc_register_constant(const void* ptr, size_t bytes);
int annc_unregister_constant(const void* ptr);

/* Which host operands may reuse their mirror's contents: 0 = none (every call uploads),
 * 1 = operands in weight / table positions only (rhs and addend of the dots, embedding tables),
 * 2 = every operand (default).  max_bytes (0 = keep) caps the device memory the mirrors may
 * take (24 GiB by default); the least recently used ones are freed beyond it. */
int annc_set_operand_cache(int mode, size_t max_bytes);
/* Bytes copied host-to-device and device-to-host by the calls of this process so far, and
 * host-to-device bytes that were not copied because the mirror already held them. */
void annc_staging_counters(uint64_t* h2d_bytes, uint64_t* d2h_bytes, uint64_t* h2d_skipped_bytes);

/* Frees the calling thread's scratch arena and every mirror (synchronises the device). */
void annc_release_device_memory(void);

/* ---------------------------------------------------------------- gating
 * ANNC_FLAGS parser, same grammar, defaults and group expansion as
 * annc/service/cpu/annc_flags.cc:10-131. */

/* Parsed once from the environment, like annc::get_annc_flags(). */
int annc_flags_is_enabled(const char* name);
/* Parses `flags` (may be NULL = unset) afresh and answers for `name`. */
int annc_flags_is_enabled_in(const char* flags, const char* name);

/* Custom-call registry, the counterpart of REGISTER_ALL_GEMM_KERNELS
 * (annc/service/cpu/kdnn_rewriter.h:148-155, install/tensorflow.patch:187-198):
 * all seven targets are registered when flag `annc-pass` is on.  Returns the
 * function address or NULL. */
void* annc_lookup_custom_call(const char* target_name);
/* Which target a `dot` (optionally followed by add, add+maximum) is rewritten to
 * under the current flags, following the benefit order of
 * annc/service/cpu/gemm_rewriter.cc:116-134; NULL when none applies.
 * pattern: 0 = dot, 1 = dot+add, 2 = dot+add+maximum, 3 = batch dot;
 * rhs_is_parameter selects the layout_matmul matcher (gemm_rewriter.cc:13-56). */
const char* annc_select_gemm_target(int pattern, int rhs_is_parameter);

/* KERNEL_MAP_FILE of the kernel selector (README_kernel_selector.md:20-62; parser and lookup
 * of annc/service/cpu/xla/kernel_selector_ops_rewriter.cc:50-263): lines
 * `[gemm](m,n,k) -> symbol` with numbers, `*` and ranges `a:b` / `a:*`; kernels gemv (2 sizes),
 * gemm (3), batch3d (4), batch4d (5), argmax (3).  Load replaces the current table (path NULL =
 * the KERNEL_MAP_FILE variable); bad_lines (may be NULL) counts the lines the reference would
 * report and skip.  Lookup returns the symbol of the first matching entry in the reference's
 * order (valid until the thread's next lookup) or NULL; resolve returns that symbol's address
 * in this library (NULL if it is not one of ours). */
int annc_kernel_map_load(const char* path, int* bad_lines);
int annc_kernel_map_load_text(const char* text, int* bad_lines);
int annc_kernel_map_size(void);
void annc_kernel_map_clear(void);
const char* annc_kernel_map_lookup(const char* kernel, const int* sizes, int num_sizes);
void* annc_kernel_map_resolve(const char* kernel, const int* sizes, int num_sizes);

/* ---------------------------------------------------------------- tensors */

enum { ANNC_F32 = 1, ANNC_I32 = 3, ANNC_I64 = 9, ANNC_BOOL = 10, ANNC_U64 = 23 };

typedef struct annc_tensor {
  void* data;      /* host or device */
  int32_t dtype;   /* ANNC_F32 ... */
  int32_t rank;    /* 0..4 */
  int64_t dims[4];
} annc_tensor;

/* Output allocation callback (OpKernelContext::allocate_output): must return a
 * buffer of prod(dims) elements of `dtype`, host or device, or NULL to fail. */
typedef void* (*annc_alloc_fn)(void* ctx, int output_index, int32_t dtype,
                               int32_t rank, const int64_t* dims);

/* ---------------------------------------------------------------- TF fused-op twins */

/* KPFusedSparseSegmentReduce<Tidx>
 * (annc/tensorflow/kernels/embedding_fused_sparse_segment_reduce.cc:38-152).
 * data f32[rows,D]; indices i32|i64[nnz]; slice_input i64[nnz,ncols];
 * begin i32[2]; begin_1 i32[1]; combiner 0 sum / 1 mean.
 * Output 0: f32[max(seg)+1, D]; output 1: i32 scalar. */
int annc_KPFusedSparseSegmentReduce(const annc_tensor* data, const annc_tensor* indices,
                                    const annc_tensor* slice_input, const annc_tensor* begin,
                                    const annc_tensor* begin_1, int combiner,
                                    annc_alloc_fn alloc, void* ctx);

/* KPFusedSparseSegmentReduceNonzero<Tidx>
 * (annc/tensorflow/kernels/embedding_fused_sparse_segment_reduce_nonzero.cc:39-374).
 * data f32[rows] or f32[rows,D].  Outputs: 0 i32[r] shape, 1 i32[nz,r] indices,
 * 2 f32[nz] values; segments in first-appearance order. */
int annc_KPFusedSparseSegmentReduceNonzero(const annc_tensor* data, const annc_tensor* indices,
                                           const annc_tensor* slice_input,
                                           const annc_tensor* begin, int combiner,
                                           annc_alloc_fn alloc, void* ctx);

/* KPFusedGather (annc/tensorflow/kernels/embedding_fused_gather.cc:26-86).
 * Outputs: 0 i64[U] unique keys (first appearance), 1 i32[nnz] inverse map,
 * 2 f32[U,D] rows. */
int annc_KPFusedGather(const annc_tensor* data, const annc_tensor* keys,
                       const annc_tensor* begin, annc_alloc_fn alloc, void* ctx);

/* KPFusedSparseDynamicStitch
 * (annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:31-83).
 * x i64[...]; `num_tables` partition tables f32[rows_p, D].  Output 0: f32[numel(x), D]. */
int annc_KPFusedSparseDynamicStitch(const annc_tensor* x, const annc_tensor* tables,
                                    int num_tables, annc_alloc_fn alloc, void* ctx);

/* KPFusedEmbeddingWithHashBucket
 * (python/tensorflow/kernels/fused_embedding_with_hash_bucket.cc:29-77).
 * The string input is replaced by its 64-bit fingerprints (`fingerprints` u64[batch])
 * and an optional `empty` bool[batch] mask (NULL = no empty strings): the
 * string -> Fingerprint64 step (FarmHash) is outside this library.
 * `bounded` != 0 selects the KPFusedDnn/KPFusedLinear...WithHashBucket and
 * RecEmbeddingV2 behaviour (fused_dnn_embedding_with_hash_bucket.cc:32-47): buckets
 * outside the table leave zeros.  Output 0: f32[batch, D]. */
int annc_KPFusedEmbeddingWithHashBucket(const annc_tensor* fingerprints, const annc_tensor* empty,
                                        const annc_tensor* variable, int64_t num_buckets,
                                        int bounded, annc_alloc_fn alloc, void* ctx);

/* KPFusedSparseEmbedding / RecEmbeddingV1
 * (python/tensorflow/kernels/fused_sparse_embedding.cc:25-80).  Outputs: 0 i64[n,2]
 * indices, 1 i64[nv] values, 2 bool[nv] empty_row_indicator, 3 i64[2] dense_shape.
 * As in the reference, a non-empty input whose bucket is 0 contributes an index row
 * but no value, so nv can be smaller than n. */
int annc_KPFusedSparseEmbedding(const annc_tensor* fingerprints, const annc_tensor* empty,
                                int64_t num_buckets, annc_alloc_fn alloc, void* ctx);

/* KPFusedBatchMatMulAddSigmoid
 * (annc/tensorflow/kernels/fused_batchmatmul_add_sigmoid.cc:393-433).
 * lhs f32[B,m,k]; rhs f32[k,n] or f32[B,k,n]; bias rank <= 3, numpy broadcast.
 * Output 0: f32[B,m,n].  Computed in fp32 (tolerance of the reference test: 1e-5). */
int annc_KPFusedBatchMatMulAddSigmoid(const annc_tensor* lhs, const annc_tensor* rhs,
                                      const annc_tensor* bias, annc_alloc_fn alloc, void* ctx);

/* KPFusedEmbeddingPadding / KPFusedEmbeddingPaddingFast
 * (annc/tensorflow/kernels/embedding_fused_padding.cc:35-113).  origin_shape i64[2];
 * input f32[rows, D]; input_rows i32 scalar; reshape_sizes i32[2] = {-1, cols}; pack i32
 * scalar (= D).  Output 0: i32 scalar padding rows; output 1: the zero-padded input
 * reshaped to f32[-1, cols], or with `fast` only its row count as an i32 scalar. */
int annc_KPFusedEmbeddingPadding(const annc_tensor* origin_shape, const annc_tensor* input,
                                 const annc_tensor* input_rows, const annc_tensor* reshape_sizes,
                                 const annc_tensor* pack, int fast, annc_alloc_fn alloc, void* ctx);

/* KPFusedEmbeddingActionIdGather
 * (annc/tensorflow/kernels/embedding_fused_action_id_gather.cc:59-129): gather(gather(params,
 * indices1), indices2) reshaped to [pack_dim, -1] with `pack` zero columns appended.
 * indices1, indices2 i32|i64 matrices; params f32[P0, P1].  Output 0: f32[pack_dim, cols + pack]. */
int annc_KPFusedEmbeddingActionIdGather(const annc_tensor* indices1, const annc_tensor* params,
                                        const annc_tensor* indices2, const annc_tensor* pack_dim,
                                        const annc_tensor* pack, annc_alloc_fn alloc, void* ctx);

/* KPFusedSparseReshape (annc/tensorflow/kernels/embedding_fused_sparse_reshape.cc:152-190): the
 * sparse tensor with indices (i, slice_input[i, begin[1]]) and shape [rows, pack_const] reshaped
 * to new_shape i64[2] (one entry may be -1).  Outputs: 0 i64[rows, 2] indices, 1 i64[2] shape. */
int annc_KPFusedSparseReshape(const annc_tensor* slice_input, const annc_tensor* begin,
                              const annc_tensor* new_shape, const annc_tensor* pack_const,
                              annc_alloc_fn alloc, void* ctx);

/* KPFusedSparseSelect (annc/tensorflow/kernels/embedding_fused_sparse_select.cc:32-107).
 * a, b, c i32 with equal element counts; greater, equal1..3 i32 scalars.  Outputs: 0 f32[n,1] =
 * a; 1 f32[n,1] = (b == equal2 || b == equal1 || a > greater); 2 f32[n,2] = {output 1, 1}. */
int annc_KPFusedSparseSelect(const annc_tensor* a, const annc_tensor* b, const annc_tensor* c,
                             const annc_tensor* greater, const annc_tensor* equal1,
                             const annc_tensor* equal2, const annc_tensor* equal3,
                             annc_alloc_fn alloc, void* ctx);

/* sparse_embedding2 fusion (annc/service/cpu/graph_opt.cc:8-41): the reference only
 * wraps the subgraph in a loop fusion; this is that loop.
 * out[i,:] = (lo <= ids[i] < hi) ? table[ids[i],:] * 1.0f : table[dflt,:] * 0.0f.
 * ids i32|i64[n]; table f32[rows,D]; out f32[n,D] (caller-owned, host or device). */
int annc_sparse_embedding2(const annc_tensor* ids, const annc_tensor* table, int64_t lo,
                           int64_t hi, int64_t dflt, float* out);

/* ---------------------------------------------------------------- device entry points */

/* Embedding bag: hash-bucket mapping + row gather + segment sum/mean in one pass.
 *   id_kind 0: ids are i32 row numbers, 1: i64 row numbers,
 *           2: u64 fingerprints, row = id % num_buckets (uint64 arithmetic,
 *              fused_embedding_with_hash_bucket.cc:63-64).
 * slice_input i64[nnz, ncols], column `col` = segment id of each lookup
 * (embedding_fused_sparse_segment_reduce.cc:59-72); batch must be > max segment id.
 * Sorted segment ids (the order of a canonical SparseTensor) run bit-exactly in the
 * reference's summation order; unsorted ids are accepted and reduced with atomics.
 * out f32[batch, ...]: row s is written at out + s*out_stride (out_stride >= D floats).
 * workspace: annc_embed_bag_workspace_bytes(batch) bytes of device memory. */
typedef struct annc_bag_table {
  const float* table;          /* f32[rows, D]                         */
  int64_t rows;                /* table rows (bounds check)            */
  int64_t num_buckets;         /* modulus for id_kind 2                */
  const void* ids;             /* [nnz]                                */
  const int64_t* slice_input;  /* i64[nnz, ncols]                      */
  int64_t nnz;
  float* out;                  /* first output row of this table       */
  const int32_t* offsets;      /* optional i32[batch + 1] bag offsets (lookups of bag s are
                                  ids[offsets[s] .. offsets[s+1])); when set, slice_input is
                                  not read and may be NULL.  Produced by
                                  annc_embed_bag_prepass_dev, e.g. on the rank that owns the
                                  batch, so that only ids and offsets need to travel */
} annc_bag_table;

size_t annc_embed_bag_workspace_bytes(int num_tables, int64_t batch);

int annc_embed_bags_dev(const annc_bag_table* tables /* host array */, int num_tables,
                        int64_t dim, int id_kind, int64_t ncols, int32_t col, int combiner,
                        int64_t batch, int64_t out_stride, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Row-sharded variant for multi-GPU runs: the rank holds, for every table, the rows r
 * with r % shard_count == shard_rank at local row r / shard_count (the mod-partition rule
 * of annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:70-71); `rows` in
 * annc_bag_table is the local row count, num_buckets stays the global modulus.  Lookups
 * owned by other ranks are skipped, so `out` receives this rank's partial sums; with
 * combiner 1 the partial is scaled by 1/len(bag) (the full bag length), so the partials of
 * all ranks add up to the mean. */
int annc_embed_bags_sharded_dev(const annc_bag_table* tables /* host array */, int num_tables,
                                int64_t dim, int id_kind, int64_t ncols, int32_t col, int combiner,
                                int64_t batch, int64_t out_stride, int shard_count,
                                int shard_rank, void* workspace, size_t workspace_bytes,
                                void* stream);
/* Fused pooling + exchange step of a row-sharded table: annc_embed_bags_sharded_dev with
 * caller-supplied bag offsets (every table's `offsets` set, slice_input unused) that leaves
 * a bag unwritten when this rank owns none of its lookups.  Each table's `out` normally
 * points into the receive buffer of the rank that owns the samples (annc_peer_buffer_open),
 * so the partial sums cross NVLink as the kernel's own stores and nothing is sent for bags
 * this rank does not contribute to.  The owner learns which parts exist from its own ids
 * (annc_embed_bag_owner_mask_dev) and adds them with annc_sum_partials_masked_dev.
 * With shard_count 1 the ids are taken as this rank's local rows: every lookup is read and
 * bags with offsets[s] == offsets[s + 1] are the ones left unwritten.  The multi-GPU step
 * itself is annc_row_exchange_* below, which splits the lookups at their source. */
int annc_embed_bags_exchange_dev(const annc_bag_table* tables /* host array */, int num_tables,
                                 int64_t dim, int id_kind, int combiner, int64_t batch,
                                 int64_t out_stride, int shard_count, int shard_rank,
                                 void* workspace, size_t workspace_bytes, void* stream);
/* mask[t * batch + s], bit g set when bag s of table t (ids, offsets, num_buckets of
 * tables[t]) has a lookup whose row r has r % shard_count == g: the ranks that write a part
 * for this bag in annc_embed_bags_exchange_dev.  shard_count <= 32. */
int annc_embed_bag_owner_mask_dev(const annc_bag_table* tables /* host array */, int num_tables,
                                  int id_kind, int64_t batch, int shard_count, uint32_t* mask,
                                  void* stream);
/* out[r, slot, :] = sum, in ascending p, of the parts p whose bit is set in
 * mask[slot * rows + r]; part p holds f32[rows, slots, slot_width] at src + p * part_stride
 * floats; zero when no bit is set.  Parts whose bit is clear are not read.  With
 * mean_offsets (i32[slots][rows + 1], the bag offsets of the prepass) the sum is multiplied by
 * 1.0f / len(bag), the reference's mean (embedding_fused_sparse_segment_reduce.cc:112-130).
 * out is f32, or bf16 when out_bf16 != 0 (out_stride in elements of that type): the input of
 * a BF16 MLP is then produced here, without a separate cast pass. */
int annc_sum_partials_masked_dev(const float* src, const uint32_t* mask, int parts,
                                 int64_t part_stride, int64_t rows, int slots, int64_t slot_width,
                                 const int32_t* mean_offsets, void* out, int64_t out_stride,
                                 int out_bf16, void* stream);
/* The same with every part laid out f32[slots, rows, slot_width] (the receive slabs of
 * annc_row_exchange_*: a part's place follows its key = slot * rows + r).  out_slots (device
 * i32[slots], or NULL for the identity) names the slot of the output row that slot t of the
 * parts is written to: the output may hold more slots than the parts. */
int annc_sum_partials_masked_slot_major_dev(const float* src, const uint32_t* mask, int parts,
                                            int64_t part_stride, int64_t rows, int slots,
                                            int64_t slot_width, const int32_t* mean_offsets,
                                            const int32_t* out_slots, void* out, int64_t out_stride,
                                            int out_bf16, void* stream);

/* out[r, 0:width] = sum over p < parts of src[p][r, 0:width], added in ascending p (the
 * reduce step after the all-to-all of partial sums).  src part p starts at
 * src + p * part_stride floats, rows are src_stride / out_stride floats apart. */
int annc_sum_partials_dev(const float* src, int parts, int64_t part_stride, int64_t rows,
                          int64_t width, int64_t src_stride, float* out, int64_t out_stride,
                          void* stream);

/* Pitched device-to-device copy of `rows` rows of `width` floats (strides in floats); places
 * the pooled vectors received from another rank into their slots of the interaction input. */
int annc_copy_rows_dev(float* dst, int64_t dst_stride, const float* src, int64_t src_stride,
                       int64_t width, int64_t rows, void* stream);

/* Receive buffers for the fused pooling + exchange step of a row-sharded table (one process
 * per GPU, GPUs of one node).  annc_peer_buffer_create allocates `bytes` of device memory on
 * the current device and fills the 64-byte `handle64`; the owner sends the handle to its peers
 * over any host channel, and each peer maps the buffer with annc_peer_buffer_open.  The mapped
 * pointer can be used as `out` of annc_bag_table: the bag kernel then stores this rank's
 * partial sums directly into the owner's memory (ordinary 16-byte stores over NVLink; no
 * multicast), where annc_sum_partials_dev adds the parts in rank order once every rank's
 * kernel has finished (a stream-ordered barrier between the two is the caller's, e.g. a
 * one-element all-reduce).  This replaces the reference-side pattern "pool, then exchange"
 * (the mod partition of embedding_fused_sparse_dynamic_stitch.cc:70-71 across parameter
 * servers) by one kernel.  Peers close their mapping before the owner destroys the buffer. */
int annc_peer_buffer_create(size_t bytes, void** dev_ptr, void* handle64);
int annc_peer_buffer_open(const void* handle64, void** dev_ptr);
/* Asynchronous device-to-device copy on `stream`; either side may be a mapped peer buffer (the
 * owner of whole tables fetches the ids and bag offsets of its tables from every source). */
int annc_peer_copy_dev(void* dst, const void* src, size_t bytes, void* stream);
int annc_peer_buffer_close(void* dev_ptr);
int annc_peer_buffer_destroy(void* dev_ptr);

/* ---- Row-sharded embedding step for several GPUs of one node (one process per GPU) ----
 * The partitioning is the reference's mod rule (owner = row % world, local row = row / world,
 * annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:70-71), applied to the rows
 * of every table after the hash-bucket modulo.  The reference has no multi-device code: this
 * object has no counterpart there beyond that rule.  Per step each rank
 *   begin   splits the lookups of its own batch by owner rank into one record list per owner
 *           (record = local row + bag), in lookup order, written straight into the owner's
 *           memory, and publishes their lengths;
 *   pool    pools the lists it received from every rank lookup by lookup and stores every
 *           finished partial sum straight into the receive slab of the rank that owns the
 *           sample (pooling and exchange in one kernel, ordinary 16-byte stores over NVLink,
 *           no multicast, no NCCL call); a slab is laid out by bag key (table, then sample), so
 *           the stores in flight stay inside a few pages of each peer;
 *   finish  adds the parts of its own batch in rank order (deterministic; within 1e-5 relative
 *           of the unsharded sum) and applies 1/len for the mean combiner.
 * Ranks are ordered by flags in peer memory; every wait is bounded (2 s by default, then the
 * error bit ANNC_ROWX_ERR_TIMEOUT is set, the kernel returns and the rank's step completes
 * with whatever arrived).  A step allocates nothing and does not synchronise the host.
 *
 * Hot rows: a table may come with a replicated set of rows (every rank holds a copy).  A lookup
 * of such a row is pooled by the rank that owns the sample and sends nothing; with skewed ids
 * this removes most (bag, owner) pairs from the exchange.  The hot rows are stored behind the
 * shard's own rows in the same allocation.  hot_count == rows with hot_rows NULL replicates the
 * whole table.
 *
 * Set-up: every rank allocates annc_row_exchange_peer_bytes() with annc_peer_buffer_create,
 * exchanges the handles over any host channel, maps the peers' buffers (annc_peer_buffer_open)
 * and calls annc_row_exchange_create; a host-side barrier must separate the creates from the
 * first step.  begin / pool / finish may be called one after the other (annc_row_exchange_step)
 * or with other work of the same stream between them.  Sorted segment ids are required
 * (ANNC_ROWX_ERR_UNSORTED otherwise). */
typedef struct annc_row_shard_table {
  const float* shard;       /* f32[local_rows + hot_count, D], 16-byte aligned: first the rows r
                               with r % world == rank, at r / world; then the replicated hot rows
                               in ascending row order                                           */
  int64_t local_rows;
  int64_t rows;             /* rows of the whole table (the modulus for id_kind 2)              */
  const int64_t* hot_rows;  /* device i64[hot_count], strictly ascending rows of the table; NULL
                               when hot_count is 0 or equals rows (the whole table replicated)   */
  int64_t hot_count;
} annc_row_shard_table;

typedef struct annc_row_exchange_config {
  int32_t world, rank, num_tables, id_kind, combiner, reserved;
  int64_t dim, batch;                /* batch = samples of ONE rank per step                  */
  int64_t max_lookups;               /* capacity: lookups of one rank per step, all tables    */
  int64_t max_lookups_per_table;
  const annc_row_shard_table* tables; /* host array [num_tables]                              */
} annc_row_exchange_config;

typedef struct annc_row_exchange annc_row_exchange;

enum {
  ANNC_ROWX_ERR_ROW = 1, ANNC_ROWX_ERR_SEGMENT = 2, ANNC_ROWX_ERR_UNSORTED = 4,
  ANNC_ROWX_ERR_TIMEOUT = 8, ANNC_ROWX_ERR_BOUNDS = 16
};

size_t annc_row_exchange_peer_bytes(const annc_row_exchange_config* config);
int annc_row_exchange_create(const annc_row_exchange_config* config,
                             void* const* peer_buffers /* [world], [rank] = own */,
                             annc_row_exchange** out);
int annc_row_exchange_destroy(annc_row_exchange* ex);
/* inputs: host array [num_tables]; ids, slice_input and nnz of annc_bag_table are read. */
int annc_row_exchange_begin(annc_row_exchange* ex, const annc_bag_table* inputs, int64_t ncols,
                            int32_t col, void* stream);
int annc_row_exchange_pool(annc_row_exchange* ex, void* stream);
/* out: f32 (or bf16 with out_bf16) [batch, num_tables, dim] rows of out_stride elements. */
int annc_row_exchange_finish(annc_row_exchange* ex, void* out, int64_t out_stride, int out_bf16,
                             void* stream);
int annc_row_exchange_step(annc_row_exchange* ex, const annc_bag_table* inputs, int64_t ncols,
                           int32_t col, void* out, int64_t out_stride, int out_bf16, void* stream);
/* Synchronises `stream` and returns the ANNC_ROWX_ERR_* bits seen since the last clear;
 * ANNC_ERR_TIMEOUT when a wait ran out. */
int annc_row_exchange_check(annc_row_exchange* ex, void* stream, int* error_bits);
int annc_row_exchange_clear_errors(annc_row_exchange* ex, void* stream);
int annc_row_exchange_set_timeout_ms(annc_row_exchange* ex, int64_t ms);
/* Output slots: table t of the exchange is written to out[:, slots[t], :] by finish (host
 * array of num_tables ints, ascending or not; NULL restores the identity).  For a caller that
 * keeps some tables outside the exchange (small tables replicated whole and pooled by
 * annc_embed_bags_dev straight into the same output rows).  Synchronises nothing; the map is
 * read by the finish calls issued after it. */
int annc_row_exchange_set_output_slots(annc_row_exchange* ex, const int32_t* slots, void* stream);
/* Blocks of the pooling kernel per SM (a persistent grid; 0 = as many as fit, the default;
 * -n = n fewer than fit).
 * With several GPUs the kernel is bound by its NVLink stores, and one block per SM fewer leaves
 * room for kernels of other streams (the next step's split, the previous step's sum and dense
 * layers) to run under it. */
int annc_row_exchange_set_pool_ctas_per_sm(annc_row_exchange* ex, int ctas_per_sm);
/* With profiling on, every step records CUDA events between its phases; phase_ms returns the
 * last step's {split, first barrier, pool + exchange, second barrier, sum} in milliseconds. */
int annc_row_exchange_set_profiling(annc_row_exchange* ex, int on);
int annc_row_exchange_phase_ms(annc_row_exchange* ex, float* ms5);
/* Last step: records this rank pooled per source rank, and the bags of its own batch each
 * owner rank sent a part for (synchronises `stream`; a reporting aid, not for the hot loop). */
int annc_row_exchange_stats(annc_row_exchange* ex, void* stream, int64_t* records_per_source,
                            int64_t* parts_per_owner);

/* Same operation as annc_embed_bags_dev for callers that must not allocate device
 * memory and have none to lend: code running inside a framework callback where
 * cudaMalloc is forbidden or would deadlock (an allocator hook, a stream-ordered
 * region owned by somebody else), or a host that fixed its memory budget at start-up.
 * No counterpart in the reference: its CPU kernels take their scratch from the heap.
 * The bag offsets live in an 8 MiB + 512 B array inside the library image, which every
 * GPU that loads the library keeps until the process exits.
 *   - Limit: num_tables * (batch + 1) <= 2,097,152; larger requests fail with
 *     ANNC_ERR_UNSUPPORTED and a message naming the limit.  Nothing is allocated or
 *     freed, here or in any routine it calls.
 *   - The first call on each device looks the array's address up (with that device
 *     current); make that first call before starting any stream capture.
 *   - All calls on a device share the array and it keeps the last call's contents
 *     (the part that must start at zero is cleared on `stream` by each call): two calls
 *     that can overlap on the GPU (different streams, no ordering) race on it.
 *   - error_bits_dev (device int, may be NULL) receives the error word that
 *     annc_embed_bag_check would report, by an asynchronous copy on `stream`. */
int annc_embed_bags_static_dev(const annc_bag_table* tables /* host array */, int num_tables,
                               int64_t dim, int id_kind, int64_t ncols, int32_t col, int combiner,
                               int64_t batch, int64_t out_stride, int* error_bits_dev,
                               void* stream);

/* Runs only the segment prepass: fills the workspace (layout of
 * annc_embed_bag_workspace_bytes: 512-byte header, then i32 offsets[num_tables][batch + 1])
 * from column `col` of every table's slice_input.  The offsets of table t start at byte
 * 512 + 4 * t * (batch + 1) of the workspace. */
int annc_embed_bag_prepass_dev(const annc_bag_table* tables /* host array */, int num_tables,
                               int64_t ncols, int32_t col, int64_t batch, void* workspace,
                               size_t workspace_bytes, void* stream);

/* Reads the device-side error word the embedding kernels set (0 = clean,
 * bit 0 = row index outside its table, bit 1 = segment id outside [0,batch)).
 * Synchronises `stream`. */
int annc_embed_bag_check(void* workspace, void* stream, int* error_bits);

/* Measurement hooks: CUDA events made by annc_timer_create.  While a pair is set on
 * the calling thread, annc_embed_bags_dev records `start` right before and `stop`
 * right after its bag-reduce kernel (the prepass and the atomic route stay outside),
 * so a benchmark can time that kernel alone inside a longer step.  NULL, NULL clears. */
void* annc_timer_create(void);
void annc_timer_destroy(void* event);
int annc_timer_elapsed_ms(void* start, void* stop, float* ms);
void annc_embed_bag_set_timing_events(void* start, void* stop);
/* Blocks per SM of the persistent lookup-granular bag kernel for the calls of this thread
 * (0 = as many as fit, the default; n > 0 = at most n; -n = n fewer than fit).  For a caller
 * that runs annc_embed_bags_dev on one stream beside another kernel of its own on a second
 * stream and wants both resident (see annc_row_exchange_set_pool_ctas_per_sm). */
void annc_embed_bag_set_stream_ctas_per_sm(int ctas_per_sm);

/* GEMM core: C = act(alpha * op(A) * op(B) + beta * C + addend + bias), row-major. */
enum { ANNC_ACT_NONE = 0, ANNC_ACT_RELU = 1, ANNC_ACT_SIGMOID = 2 };
enum { ANNC_B_PLAIN = 0, ANNC_B_KN4 = 1 };
enum { ANNC_MATH_AUTO = 0, ANNC_MATH_FP32 = 1, ANNC_MATH_TF32 = 2, ANNC_MATH_BF16 = 3 };
/* io_flags.  The reference's operators are fp32 end to end; the BF16 route is for graphs that
 * ask for it: weights converted once (annc_bf16_weight_dev), activations produced in bf16 by
 * the previous layer's epilogue (ANNC_IO_C_BF16).  With ANNC_MATH_BF16, a and b point to bf16
 * data: A [M,K], B [N,K] (trans_b = 1), lda / ldb / stride_a / stride_b in elements.
 * ANNC_IO_SOFTMAX applies a row softmax over the n <= 256 columns after bias and activation
 * (batch_matmul followed by the XNNPACK softmax, in one kernel). */
enum { ANNC_IO_A_BF16 = 1, ANNC_IO_B_BF16 = 2, ANNC_IO_C_BF16 = 4, ANNC_IO_SOFTMAX = 8,
       ANNC_IO_PAIR = 16 /* ask for the CTA-pair kernel whatever the shape heuristic says */ };

typedef struct annc_gemm_desc {
  int32_t trans_a, trans_b;
  int64_t m, n, k;
  int64_t batch;                 /* >= 1 */
  int64_t lda, ldb, ldc, ld_addend;
  int64_t stride_a, stride_b, stride_c, stride_addend; /* per batch, in floats; 0 = shared */
  float alpha, beta;
  const float* a;
  const float* b;
  float* c;
  const float* addend;           /* [m,n] or NULL */
  const float* bias;             /* [n] or NULL   */
  int32_t activation;            /* ANNC_ACT_*    */
  int32_t b_format;              /* ANNC_B_*; KN4 = python/annc/optimize/data_pack.py layout */
  int32_t math;                  /* ANNC_MATH_*   */
  int32_t io_flags;              /* ANNC_IO_* */
  void* workspace;               /* optional device scratch, 16-byte aligned, or NULL      */
  size_t workspace_bytes;        /* with >= 4*k*n bytes a large kn4 GEMM first unpacks B   */
} annc_gemm_desc;                /* into it and then runs at the speed of the plain layout */

int annc_gemm_run(const annc_gemm_desc* desc, void* stream);
/* Synchronises `stream` and reports whether a tensor-core GEMM CTA has given up on one of
 * its bounded mbarrier waits since the library was loaded (its output is then invalid). */
int annc_gemm_check(void* stream, int* timed_out);
/* Test aid: sets (non-zero) or clears (0) that device-side word by hand, the way a CTA whose
 * wait ran out does, so that the reporting path can be exercised without a kernel giving up.
 * While it is set the tensor-core GEMM kernels return at once. */
int annc_gemm_debug_set_error_word(int value);
/* Name of the kernel family annc_gemm_run would pick: "tcgen05_pair_tf32" / "tcgen05_pair_bf16"
 * (persistent CTA-pair kernel), "tcgen05_tf32" (single-CTA tiles, also the kn4 loader),
 * "simt_fp32" (CUDA cores). */
const char* annc_gemm_kernel_name(const annc_gemm_desc* desc);

/* fp32 -> bf16 (round to nearest even), n elements. */
int annc_cast_bf16_dev(const float* src, void* dst_bf16, int64_t n, void* stream);
/* Weight for the BF16 route: fp32 B[K,N] (row pitch ldb) -> bf16 [N,K], converted once. */
int annc_bf16_weight_dev(const float* b_kn, int64_t ldb, void* b_nk_bf16, int64_t k, int64_t n,
                         void* stream);

/* Benchmark utility: fills table[i, c] (f32[local_rows, dim], dim % 4 == 0) with the value a
 * counter-based hash gives for (seed, table_id, row = first_row + i * row_step, c), uniform in
 * [-0.05, 0.05).  Used for tables too large to generate on the host (the 655 GB row-sharded
 * configuration): each rank fills its own shard (first_row = rank, row_step = ranks) and the
 * CPU oracle regenerates any row with the same integer steps (annc_b200/synth.py). */
int annc_synth_fill_rows_dev(float* table, int64_t local_rows, int64_t dim, uint64_t seed,
                             int64_t table_id, int64_t first_row, int64_t row_step, void* stream);
/* The same values for an explicit list of rows (device i64[count]): table[i, :] = row rows[i].
 * Fills the replicated hot rows of a hashed table. */
int annc_synth_fill_row_list_dev(float* table, const int64_t* rows, int64_t count, int64_t dim,
                                 uint64_t seed, int64_t table_id, void* stream);

/* kn4 <-> [K,N] conversion on the device (layout of python/annc/optimize/data_pack.py,
 * vector 12, tiles 352 x 128, python/annc/optimize/constant_folding.py:77-88). */
int annc_kn4_pack_dev(const float* b_kn, float* b_packed, int64_t k, int64_t n, void* stream);
int annc_kn4_unpack_dev(const float* b_packed, float* b_kn, int64_t k, int64_t n, void* stream);
/* Host: offset of element (k, n) inside the packed buffer. */
int64_t annc_kn4_offset(int64_t K, int64_t N, int64_t k, int64_t n);

/* Row softmax, fp32 (annc/service/cpu/xla/xnnpack_ops.cc:30-74). */
int annc_softmax_dev(const float* in, float* out, int64_t batch, int64_t channels, void* stream);
/* __pooling (annc/service/cpu/graph_opt.cc:131-176). */
int annc_pooling_dev(float* out, const int64_t* arg, const float* mul_out, int64_t m, int64_t k,
                     int64_t n, const int64_t slice_starts[3], const int64_t slice_limits[3],
                     void* stream);
/* __reduce_mean (annc/service/cpu/reduce_rewriter.cc:31-46): out[i] = sum_j |value[i*m+j]| / m. */
int annc_reduce_mean_dev(float* out, const float* value, int64_t m, int64_t n, void* stream);
/* ArgMax over the last dim, ties -> last (annc/service/cpu/xla/kernel_selector.cc:317-340). */
int annc_argmax_dev(int64_t rows, int64_t n, const float* invals, const int32_t* inidxs,
                    float init_value, int32_t init_idx, float* outvals, int32_t* outidxs,
                    void* stream);
/* y = alpha*op(A)x + beta*y (annc/service/cpu/xla/kernel_selector.cc:168-178). */
int annc_gemv_dev(int trans_a, int64_t m, int64_t n, float alpha, const float* a, const float* x,
                  float beta, float* y, void* stream);

/* DLRM dot interaction on the device: Z f32[batch, F, D] (row stride z_stride floats per
 * sample) -> out[b, :] = [ Z[b,0,:] (D values) | strict lower triangle of Z[b] Z[b]^T in
 * row-major (i,j<i) order | zero padding up to out_stride ].  This is the
 * `__batch_matmul` of Z by its transpose (annc/service/cpu/gemm_rewriter.cc:187-216)
 * followed by the triangle gather and concat that XLA fuses around it.
 * math: ANNC_MATH_FP32 = CUDA cores, exact fp32; ANNC_MATH_AUTO / TF32 = tcgen05 kernel
 * (dim 64, z_stride == features*dim), products in TF32, sums in fp32. */
int annc_dot_interaction_dev(const float* z, int64_t batch, int features, int dim,
                             int64_t z_stride, float* out, int64_t out_stride, int math,
                             void* stream);

/* ---------------------------------------------------------------- reference symbols
 * XLA custom-call targets (annc/service/cpu/kdnn_rewriter.h:140-155).  `in` holds the
 * fusion operands followed by one s64 vector [dims..., minor_to_major...] per operand
 * (annc/service/hlo_util.h:14-33). */
void __matmul(void* out, const void** in);          /* gemm_rewriter.cc:161-185 */
void __layout_matmul(void* out, const void** in);   /* gemm_rewriter.cc:136-159 */
void __batch_matmul(void* out, const void** in);    /* gemm_rewriter.cc:187-216 */
void __matmul_add(void* out, const void** in);      /* gemm_rewriter.cc:218-247 */
void __matmul_add_relu(void* out, const void** in); /* gemm_rewriter.cc:249-281 */
void __reduce_mean(void* out, const void** in);     /* reduce_rewriter.cc:31-46 */
void __pooling(void* out, void** in);               /* graph_opt.cc:131-176     */

/* XLA:CPU runtime symbols (annc/service/cpu/xla/xnnpack_ops.h:26-29,
 * annc/service/cpu/xla/kernel_selector.h:94-183).  The reference declares the
 * kernel-selector functions with C++ linkage in xla::cpu; the library exports them
 * under both the plain and the mangled names. */
void __xla_cpu_runtime_XnnPackSoftMaxND(const void* run_options_ptr, void* in, void* out,
                                        int64_t batch_size, int64_t channels);
#define ANNC_DECL_GEMM(name)                                                              \
  void __xla_cpu_runtime_KernelSelectorGEMM##name(const void* run_options_ptr, bool trA,  \
                                                  bool trB, const float* A, const float* B,\
                                                  int M, int N, int K, float alpha,        \
                                                  float beta, float* C);
#define ANNC_DECL_B3D(name)                                                                \
  void __xla_cpu_runtime_KernelSelectorBatch3D##name(const void* run_options_ptr, bool trA,\
                                                     bool trB, const float* A,             \
                                                     const float* B, int P, int M, int N,  \
                                                     int K, float* C);
#define ANNC_DECL_B4D(name)                                                                \
  void __xla_cpu_runtime_KernelSelectorBatch4D##name(const void* run_options_ptr, bool trA,\
                                                     bool trB, const float* A,             \
                                                     const float* B, int Q, int P, int M,  \
                                                     int N, int K, float* C);
#define ANNC_DECL_GEMV(name)                                                              \
  void __xla_cpu_runtime_KernelSelectorGEMV##name(const void* run_options_ptr, bool trA,  \
                                                  const float* A, const float* X, int M,  \
                                                  int N, float alpha, float beta, float* Y);
#define ANNC_DECL_ARGMAX(name)                                                            \
  void __xla_cpu_runtime_ArgMax3D##name(const void* run_options_ptr, int B, int M, int N, \
                                        float* invals, int32_t* inidxs, float init_value, \
                                        int32_t init_idx, float* outvals, int32_t* outidxs);
ANNC_DECL_GEMM(Sequential) ANNC_DECL_GEMM(Parallel) ANNC_DECL_GEMM(MLIR) ANNC_DECL_GEMM(Empty)
ANNC_DECL_B3D(Sequential) ANNC_DECL_B3D(Parallel) ANNC_DECL_B3D(MLIR) ANNC_DECL_B3D(Empty)
ANNC_DECL_B4D(Sequential) ANNC_DECL_B4D(Parallel) ANNC_DECL_B4D(MLIR) ANNC_DECL_B4D(Empty)
ANNC_DECL_GEMV() ANNC_DECL_GEMV(MLIR) ANNC_DECL_GEMV(Empty)
ANNC_DECL_ARGMAX(Parallel) ANNC_DECL_ARGMAX(Sequential) ANNC_DECL_ARGMAX(Empty)
#undef ANNC_DECL_GEMM
#undef ANNC_DECL_B3D
#undef ANNC_DECL_B4D
#undef ANNC_DECL_GEMV
#undef ANNC_DECL_ARGMAX

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* ANNC_B200_H_ */

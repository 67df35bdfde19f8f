/*
 * CPU oracle for the ANNC custom-operator hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the reference's CPU kernels, used as the checker
 * in tests/, in the smoke test and as the timed CPU baseline of bench.py.
 * The product library never links, loads or calls anything in this file.
 *
 * Every function cites the reference file:line (paths inside the ANNC
 * project) whose arithmetic, operand order and summation order it follows.
 * The NEON 4-wide loops of the reference add lane-wise, so each output
 * column sees the same sequence of scalar fp32 additions as the scalar
 * loops here.  Build with -ffp-contract=off so no FMA is formed where the
 * reference does separate multiplies and adds.
 *
 * Pinning: the E3/E4/E5/E6/G9 functions are checked against the literal
 * known-answer tensors of the reference's own unit tests
 * (the _test.cc files under annc/tensorflow/kernels) in tests/test_oracle_golden.py.
 * The GEMM custom calls, __pooling, __reduce_mean and the sequential
 * KernelSelector GEMM / batch / GEMV / ArgMax3D symbols are checked against
 * the reference's own function bodies, cut from the reference tree and
 * compiled beside this file (xla_ref_shim.cc, tests/test_oracle_xla_ref.py).
 * Softmax, the kn4 GEMM's kp_sgemm, the hash-bucket ops and sparse_embedding2
 * have no test in the reference and bodies that cannot be compiled here:
 * parity unpinned for those; they follow the cited source text.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <pthread.h>
#include <unistd.h>

#define ORACLE_OK 0
#define ORACLE_ERR_RANGE 1

/* ------------------------------------------------------------------ */
/* E3: KPFusedSparseSegmentReduce                                      */
/* annc/tensorflow/kernels/embedding_fused_sparse_segment_reduce.cc    */
/* ------------------------------------------------------------------ */

/* :64-72  batch_size = max(segment id) + 1, max starts at 0. */
int64_t oracle_segment_batch(const int64_t *slice_input, int64_t nnz,
                             int64_t ncols, int32_t col) {
  int64_t max_seg = 0;
  for (int64_t i = 0; i < nnz; ++i) {
    int64_t s = slice_input[i * ncols + col];
    if (s > max_seg) max_seg = s;
  }
  return max_seg + 1;
}

static inline int64_t load_index(const void *indices, int idx64, int64_t i) {
  return idx64 ? ((const int64_t *)indices)[i]
               : (int64_t)((const int32_t *)indices)[i];
}

/* :77 zero fill, :133-150 sum, :88-130 mean (count then multiply by
 * 1.0f/float(count)), :81-83 second output.  out is [batch, dim]. */
int oracle_sparse_segment_reduce(const float *data, int64_t dim,
                                 const void *indices, int idx64, int64_t nnz,
                                 const int64_t *slice_input, int64_t ncols,
                                 int32_t col, int32_t begin_1, int combiner,
                                 float *out, int64_t batch,
                                 int32_t *slice_out) {
  memset(out, 0, (size_t)(batch * dim) * sizeof(float));
  *slice_out = (begin_1 == 0) ? (int32_t)batch : (int32_t)dim;
  int32_t *counts = NULL;
  if (combiner == 1) counts = (int32_t *)calloc((size_t)batch, sizeof(int32_t));
  for (int64_t i = 0; i < nnz; ++i) {
    int64_t seg = slice_input[i * ncols + col];
    int64_t row = load_index(indices, idx64, i);
    if (counts) counts[seg] += 1;
    float *o = out + seg * dim;
    const float *r = data + row * dim;
    for (int64_t j = 0; j < dim; ++j) o[j] += r[j];
  }
  if (counts) {
    for (int64_t s = 0; s < batch; ++s) {
      if (counts[s] > 0) {
        const float inv = 1.0f / (float)counts[s];
        float *o = out + s * dim;
        for (int64_t j = 0; j < dim; ++j) o[j] *= inv;
      }
    }
    free(counts);
  }
  return ORACLE_OK;
}

/* ------------------------------------------------------------------ */
/* E1 + E2: hash-bucket id mapping and row gather                      */
/* python/tensorflow/kernels/fused_embedding_with_hash_bucket.cc:59-76 */
/* The string -> Fingerprint64 step is outside the contract: `hash`    */
/* holds the 64-bit fingerprints, `empty[i]` marks empty strings.      */
/* ------------------------------------------------------------------ */

/* :64,72  uint64 hash % (int64 num_buckets promoted to uint64). */
void oracle_hash_bucket(const uint64_t *hash, int64_t n, int64_t num_buckets,
                        int64_t *bucket) {
  for (int64_t i = 0; i < n; ++i)
    bucket[i] = (int64_t)(hash[i] % (uint64_t)num_buckets);
}

/* :59 memset, :60-67 dim==1 case, :69-75 memcpy of one row. */
void oracle_embedding_with_hash_bucket(const uint64_t *hash,
                                       const uint8_t *empty, int64_t batch,
                                       const float *weight, int64_t dim,
                                       int64_t num_buckets, float *out) {
  memset(out, 0, (size_t)(batch * dim) * sizeof(float));
  for (int64_t i = 0; i < batch; ++i) {
    if (empty && empty[i]) continue;
    uint64_t x = hash[i] % (uint64_t)num_buckets;
    memcpy(out + i * dim, weight + x * dim, (size_t)dim * sizeof(float));
  }
}

/* E2b: python/tensorflow/kernels/fused_dnn_embedding_with_hash_bucket.cc
 * :32-47 (same in fused_linear_embdedding_with_hash_bucket.cc:41-56 and
 * RecEmbeddingV2, install/xla/remap_subgraph.patch:287-300): the bucket
 * is converted to int64 and rows outside [0, rows) stay zero. */
void oracle_dnn_embedding_with_hash_bucket(const uint64_t *hash,
                                           const uint8_t *empty, int64_t batch,
                                           const float *weight, int64_t rows,
                                           int64_t dim, int64_t num_buckets,
                                           float *out) {
  memset(out, 0, (size_t)(batch * dim) * sizeof(float));
  for (int64_t i = 0; i < batch; ++i) {
    if (empty && empty[i]) continue;
    int64_t b = (int64_t)(hash[i] % (uint64_t)num_buckets);
    if (b >= 0 && b < rows)
      for (int64_t j = 0; j < dim; ++j) out[i * dim + j] = weight[b * dim + j];
  }
}

/* E2c: python/tensorflow/kernels/fused_sparse_embedding.cc:33-79 (same as
 * RecEmbeddingV1, install/xla/remap_subgraph.patch:216-262).  The index
 * pair is always pushed; value/empty flag only when the string is empty or
 * the bucket is > 0 (:39-42), so n_values can be smaller than n_indices.
 * The final copy loop (:74-79) runs over indices.size() and would read
 * past `value` in that case; the oracle reports the two counts and writes
 * only the entries that exist. */
void oracle_sparse_embedding(const uint64_t *hash, const uint8_t *empty,
                             int64_t n, int64_t num_buckets,
                             int64_t *indices /*[n,2]*/, int64_t *values,
                             uint8_t *empty_out, int64_t *dense_shape /*[2]*/,
                             int64_t *n_indices, int64_t *n_values) {
  int64_t ni = 0, nv = 0;
  for (int64_t i = 0; i < n; ++i) {
    indices[2 * ni] = i;
    indices[2 * ni + 1] = 0;
    ++ni;
    if (!(empty && empty[i])) {
      int64_t x = (int64_t)(hash[i] % (uint64_t)num_buckets);
      if (x > 0) {
        values[nv] = x;
        empty_out[nv] = 0;
        ++nv;
      }
    } else {
      values[nv] = 0;
      empty_out[nv] = 1;
      ++nv;
    }
  }
  dense_shape[0] = n;
  dense_shape[1] = 1;
  *n_indices = ni;
  *n_values = nv;
}

/* ------------------------------------------------------------------ */
/* E4: KPFusedSparseSegmentReduceNonzero                                */
/* annc/tensorflow/kernels/embedding_fused_sparse_segment_reduce_nonzero.cc */
/* ------------------------------------------------------------------ */

typedef struct {
  int64_t *keys;
  int64_t *vals;
  uint8_t *used;
  int64_t cap; /* power of two */
} imap_t;

static uint64_t mix64(uint64_t x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdULL;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ULL;
  x ^= x >> 33;
  return x;
}

static void imap_init(imap_t *m, int64_t n) {
  int64_t cap = 16;
  while (cap < 2 * n + 2) cap <<= 1;
  m->cap = cap;
  m->keys = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
  m->vals = (int64_t *)malloc((size_t)cap * sizeof(int64_t));
  m->used = (uint8_t *)calloc((size_t)cap, 1);
}

static void imap_free(imap_t *m) {
  free(m->keys);
  free(m->vals);
  free(m->used);
}

/* Returns the value stored for key, inserting `fresh` when absent;
 * *inserted tells which happened. */
static int64_t imap_get_or_put(imap_t *m, int64_t key, int64_t fresh,
                               int *inserted) {
  uint64_t h = mix64((uint64_t)key) & (uint64_t)(m->cap - 1);
  while (m->used[h]) {
    if (m->keys[h] == key) {
      *inserted = 0;
      return m->vals[h];
    }
    h = (h + 1) & (uint64_t)(m->cap - 1);
  }
  m->used[h] = 1;
  m->keys[h] = key;
  m->vals[h] = fresh;
  *inserted = 1;
  return fresh;
}

/* data_rank 1: :79-209; data_rank 2: :211-370.  Segments are emitted in
 * first-appearance order (:94-121, :226-268), value = sum * inv_count for
 * mean (:124-133, :273-289), entries with value != 0.0f only.
 * out_indices is [nz, data_rank] int32, out_values [nz] float.
 * Capacity needed: (number of distinct segments) * dim entries.
 * Returns the number of non-zero entries; out_shape gets batch (and dim). */
int64_t oracle_sparse_segment_reduce_nonzero(
    const float *data, int data_rank, int64_t dim, const void *indices,
    int idx64, int64_t nnz, const int64_t *slice_input, int64_t ncols,
    int32_t col, int combiner, int32_t *out_shape, int32_t *out_indices,
    float *out_values) {
  int64_t batch = oracle_segment_batch(slice_input, nnz, ncols, col);
  if (data_rank == 1) dim = 1;
  out_shape[0] = (int32_t)batch;
  if (data_rank == 2) out_shape[1] = (int32_t)dim;

  imap_t map;
  imap_init(&map, nnz);
  int64_t nseg = 0;
  int64_t *order = (int64_t *)malloc((size_t)(nnz + 1) * sizeof(int64_t));
  int32_t *counts = (int32_t *)calloc((size_t)(nnz + 1), sizeof(int32_t));
  float *sums = (float *)calloc((size_t)((nnz + 1) * dim), sizeof(float));

  for (int64_t i = 0; i < nnz; ++i) {
    int64_t seg = slice_input[i * ncols + col];
    int64_t row = load_index(indices, idx64, i);
    int ins;
    int64_t idx = imap_get_or_put(&map, seg, nseg, &ins);
    if (ins) order[nseg++] = seg;
    float *s = sums + idx * dim;
    const float *r = data + row * dim;
    for (int64_t d = 0; d < dim; ++d) s[d] += r[d];
    counts[idx]++;
  }

  int64_t nz = 0;
  for (int64_t s = 0; s < nseg; ++s) {
    float inv = 1.0f;
    if (combiner == 1)
      inv = counts[s] > 0 ? (1.0f / (float)counts[s]) : 0.0f;
    for (int64_t d = 0; d < dim; ++d) {
      /* 1-D sum mode tests the raw sum (:176-197); every other mode
       * multiplies first; with inv == 1.0f both are the same value. */
      float v = (combiner == 1 || data_rank == 2) ? sums[s * dim + d] * inv
                                                  : sums[s * dim + d];
      if (v != 0.0f) {
        out_indices[nz * data_rank] = (int32_t)order[s];
        if (data_rank == 2) out_indices[nz * 2 + 1] = (int32_t)d;
        out_values[nz] = v;
        ++nz;
      }
    }
  }
  free(order);
  free(counts);
  free(sums);
  imap_free(&map);
  return nz;
}

/* ------------------------------------------------------------------ */
/* E5: KPFusedGather  annc/tensorflow/kernels/embedding_fused_gather.cc */
/* ------------------------------------------------------------------ */

/* :50-63 unique keys of column `col` in first-appearance order and the
 * inverse map; :76-85 row copy with the `idx < rows` check.
 * Returns the number of unique keys, or -1 for "idx out of table range". */
int64_t oracle_fused_gather(const float *data, int64_t rows, int64_t dim,
                            const int64_t *keys, int64_t nnz, int64_t ncols,
                            int32_t col, int64_t *out_unique,
                            int32_t *out_indices, float *out_data) {
  imap_t map;
  imap_init(&map, nnz);
  int64_t nu = 0;
  for (int64_t i = 0; i < nnz; ++i) {
    int64_t k = keys[i * ncols + col];
    int ins;
    int64_t idx = imap_get_or_put(&map, k, nu, &ins);
    if (ins) out_unique[nu++] = k;
    out_indices[i] = (int32_t)idx;
  }
  imap_free(&map);
  for (int64_t u = 0; u < nu; ++u) {
    int64_t idx = out_unique[u];
    if (!(idx < rows)) return -1;
    memcpy(out_data + u * dim, data + idx * dim, (size_t)dim * sizeof(float));
  }
  return nu;
}

/* ------------------------------------------------------------------ */
/* E6: KPFusedSparseDynamicStitch                                      */
/* annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:66-79 */
/* ------------------------------------------------------------------ */
int oracle_sparse_dynamic_stitch(const int64_t *x, int64_t n,
                                 const float *const *tables,
                                 const int64_t *table_rows, int num_partitions,
                                 int64_t dim, float *out) {
  for (int64_t i = 0; i < n; ++i) {
    const int64_t id = x[i];
    const int64_t t = id % num_partitions;
    const int64_t r = id / num_partitions;
    if (!(r < table_rows[t])) return ORACLE_ERR_RANGE; /* "row_id out of range." */
    memcpy(out + i * dim, tables[t] + r * dim, (size_t)dim * sizeof(float));
  }
  return ORACLE_OK;
}

/* ------------------------------------------------------------------ */
/* E7: sparse_embedding2 fusion  annc/service/cpu/graph_opt.cc:8-41     */
/* out[i,:] = float(lo <= id < hi) * table[valid ? id : dflt, :]        */
/* (the subgraph as matched in bisheng-cpu/embedding_simplify.cc:31-48) */
/* ------------------------------------------------------------------ */
void oracle_sparse_embedding2(const int64_t *ids, int64_t n,
                              const float *table, int64_t dim, int64_t lo,
                              int64_t hi, int64_t dflt, float *out) {
  for (int64_t i = 0; i < n; ++i) {
    const int valid = (ids[i] >= lo) && (ids[i] < hi);
    const float m = valid ? 1.0f : 0.0f;
    const float *r = table + (valid ? ids[i] : dflt) * dim;
    for (int64_t j = 0; j < dim; ++j) out[i * dim + j] = m * r[j];
  }
}

/* ------------------------------------------------------------------ */
/* E8: __pooling  annc/service/cpu/graph_opt.cc:131-176                */
/* ------------------------------------------------------------------ */
void oracle_pooling(float *out, const int64_t *arg, const float *mul_out,
                    const int64_t *slice_starts, const int64_t *slice_limits,
                    const int64_t *arg_shape, const int64_t *mul_shape) {
  const int64_t m = arg_shape[0], k = arg_shape[1], n = mul_shape[2];
  for (int64_t i = 0; i < m; ++i) {
    float red = 0.0f; /* :149-152 count accumulated in float */
    for (int64_t j = 0; j < k; ++j) red += (float)(arg[i * k + j] > 0);
    const int in_i = i >= slice_starts[0] && i < slice_limits[0];
    for (int64_t p = 0; p < n; ++p) {
      const int in_p = p >= slice_starts[2] && p < slice_limits[2];
      float sum = 0.0f; /* :168-172 sums all k entries, masked ones are 0 */
      for (int64_t j = 0; j < k; ++j) {
        float v = 0.0f;
        if (in_i && in_p && j >= slice_starts[1] && j < slice_limits[1] &&
            arg[i * k + j] > 0)
          v = mul_out[i * k * n + j * n + p];
        sum += v;
      }
      out[i * n + p] = (red == 0.0f) ? 0.0f : sum / red;
    }
  }
}

/* ------------------------------------------------------------------ */
/* S1: __xla_cpu_runtime_XnnPackSoftMaxND                               */
/* annc/service/cpu/xla/xnnpack_ops.cc:30-74 (XNNPACK softmax_nc_f32,   */
/* not in the tree: restated as max-subtract / expf / sum / divide).    */
/* ------------------------------------------------------------------ */
void oracle_softmax(const float *in, float *out, int64_t batch,
                    int64_t channels) {
  for (int64_t b = 0; b < batch; ++b) {
    const float *x = in + b * channels;
    float *y = out + b * channels;
    float mx = x[0];
    for (int64_t c = 1; c < channels; ++c) mx = x[c] > mx ? x[c] : mx;
    float sum = 0.0f;
    for (int64_t c = 0; c < channels; ++c) {
      y[c] = expf(x[c] - mx);
      sum += y[c];
    }
    for (int64_t c = 0; c < channels; ++c) y[c] = y[c] / sum;
  }
}

/* S2: __reduce_mean  annc/service/cpu/reduce_rewriter.cc:31-46:
 * out[i] = sasum(m, value + i*m) / m, for i < n (sum of absolute values). */
void oracle_reduce_mean(float *out, const float *value, int64_t m, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    float s = 0.0f;
    for (int64_t j = 0; j < m; ++j) s += fabsf(value[i * m + j]);
    out[i] = s / (float)(int)m;
  }
}

/* G10: __xla_cpu_runtime_ArgMaxTask
 * annc/service/cpu/xla/kernel_selector.cc:317-340 (ties: last wins, >=). */
void oracle_argmax3d(int64_t rows, int64_t n, const float *invals,
                     const int32_t *inidxs, float init_value, int32_t init_idx,
                     float *outvals, int32_t *outidxs) {
  for (int64_t r = 0; r < rows; ++r) {
    float mv = init_value;
    int32_t mi = init_idx;
    for (int64_t i = 0; i < n; ++i) {
      float v = invals[r * n + i];
      if (v >= mv) {
        mv = v;
        mi = inidxs[r * n + i];
      }
    }
    outvals[r] = mv;
    outidxs[r] = mi;
  }
}

/* ------------------------------------------------------------------ */
/* GEMM family, scalar fp32.  C = alpha*op(A)*op(B) + beta*C, row-major */
/* with the leading dimensions the callers use:                         */
/* annc/service/cpu/gemm_rewriter.cc:161-281,                           */
/* annc/service/cpu/xla/kernel_selector.cc:31-43 (lda = trA ? M : K,    */
/* ldb = trB ? K : N, ldc = N).  The reference calls OpenBLAS here; the */
/* Python side of the oracle uses OpenBLAS sgemm for the large cases    */
/* and this loop for the small ones.                                    */
/* ------------------------------------------------------------------ */
void oracle_sgemm(int trA, int trB, int64_t M, int64_t N, int64_t K,
                  float alpha, const float *A, const float *B, float beta,
                  float *C) {
  const int64_t lda = trA ? M : K, ldb = trB ? K : N;
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) {
        const float a = trA ? A[k * lda + i] : A[i * lda + k];
        const float b = trB ? B[j * ldb + k] : B[k * ldb + j];
        acc += a * b;
      }
      C[i * N + j] = (beta == 0.0f) ? alpha * acc : alpha * acc + beta * C[i * N + j];
    }
  }
}

/* G8: cblas_sgemv row-major, annc/service/cpu/xla/kernel_selector.cc:168-178.
 * A is [M,N]; y has M entries (no trans) or N entries (trans). */
void oracle_sgemv(int trA, int64_t M, int64_t N, float alpha, const float *A,
                  const float *X, float beta, float *Y) {
  const int64_t ny = trA ? N : M, nx = trA ? M : N;
  for (int64_t i = 0; i < ny; ++i) {
    float acc = 0.0f;
    for (int64_t j = 0; j < nx; ++j)
      acc += (trA ? A[j * N + i] : A[i * N + j]) * X[j];
    Y[i] = (beta == 0.0f) ? alpha * acc : alpha * acc + beta * Y[i];
  }
}

/* G9: KPFusedBatchMatMulAddSigmoid, generic path
 * annc/tensorflow/kernels/fused_batchmatmul_add_sigmoid.cc:216-255 with the
 * bias broadcast of BuildBiasInfo (:197-214); sigmoid as in the
 * reference's own test oracle (fused_batchmatmul_add_sigmoid_test.cc:42).
 * bias_dims holds the bias shape right-aligned to 3 dims. */
void oracle_batch_matmul_add_sigmoid(const float *lhs, const float *rhs,
                                     const float *bias,
                                     const int64_t *bias_dims, int64_t batch,
                                     int64_t m, int64_t k, int64_t n,
                                     int rhs_batched, float *out) {
  int64_t st[3];
  st[2] = bias_dims[2] == 1 ? 0 : 1;
  st[1] = bias_dims[1] == 1 ? 0 : bias_dims[2];
  st[0] = bias_dims[0] == 1 ? 0 : bias_dims[1] * bias_dims[2];
  for (int64_t b = 0; b < batch; ++b) {
    const float *L = lhs + b * m * k;
    const float *R = rhs + (rhs_batched ? b * k * n : 0);
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j) {
        float acc = bias[b * st[0] + i * st[1] + j * st[2]];
        for (int64_t kk = 0; kk < k; ++kk) acc += L[i * k + kk] * R[kk * n + j];
        out[(b * m + i) * n + j] = 1.0f / (1.0f + expf(-acc));
      }
  }
}

/* ------------------------------------------------------------------ */
/* CPU baseline driver for the DLRM-style workload: hash-bucket mapping  */
/* (E1) followed by the segment reduce of E3 for each table.  The        */
/* reference kernel itself is single-threaded; a TF executor would run   */
/* the per-table ops concurrently, so tables are handed out to `threads` */
/* POSIX threads.  The output row of table t for sample s is             */
/* out[(s*out_slots + out_first + t)*dim].                               */
/* ------------------------------------------------------------------ */
typedef struct {
  int num_tables;
  const float *const *tables;
  const int64_t *table_rows;
  int64_t dim;
  const int64_t *const *raw_ids;
  const int64_t *const *slice_inputs;
  const int64_t *nnz;
  int64_t ncols;
  int32_t col;
  int combiner;
  int64_t batch;
  float *out;
  int64_t out_slots, out_first;
  int next; /* next table to take, guarded by mu */
  pthread_mutex_t mu;
} bags_job_t;

static void bags_one_table(const bags_job_t *J, int t) {
  const float *W = J->tables[t];
  const uint64_t rows = (uint64_t)J->table_rows[t];
  const int64_t dim = J->dim;
  int32_t *counts = (int32_t *)calloc((size_t)J->batch, sizeof(int32_t));
  for (int64_t s = 0; s < J->batch; ++s)
    memset(J->out + (s * J->out_slots + J->out_first + t) * dim, 0,
           (size_t)dim * sizeof(float));
  for (int64_t i = 0; i < J->nnz[t]; ++i) {
    const int64_t seg = J->slice_inputs[t][i * J->ncols + J->col];
    const uint64_t b = (uint64_t)J->raw_ids[t][i] % rows;
    float *o = J->out + (seg * J->out_slots + J->out_first + t) * dim;
    const float *r = W + b * dim;
    counts[seg] += 1;
    for (int64_t j = 0; j < dim; ++j) o[j] += r[j];
  }
  if (J->combiner == 1)
    for (int64_t s = 0; s < J->batch; ++s)
      if (counts[s] > 0) {
        const float inv = 1.0f / (float)counts[s];
        float *o = J->out + (s * J->out_slots + J->out_first + t) * dim;
        for (int64_t j = 0; j < dim; ++j) o[j] *= inv;
      }
  free(counts);
}

static void *bags_worker(void *arg) {
  bags_job_t *J = (bags_job_t *)arg;
  for (;;) {
    pthread_mutex_lock(&J->mu);
    int t = J->next++;
    pthread_mutex_unlock(&J->mu);
    if (t >= J->num_tables) break;
    bags_one_table(J, t);
  }
  return NULL;
}

void oracle_embed_bags_tables(int num_tables, const float *const *tables,
                              const int64_t *table_rows, int64_t dim,
                              const int64_t *const *raw_ids,
                              const int64_t *const *slice_inputs,
                              const int64_t *nnz, int64_t ncols, int32_t col,
                              int combiner, int64_t batch, float *out,
                              int64_t out_slots, int64_t out_first,
                              int threads) {
  bags_job_t J = {num_tables, tables, table_rows, dim, raw_ids, slice_inputs,
                  nnz, ncols, col, combiner, batch, out, out_slots, out_first,
                  0, PTHREAD_MUTEX_INITIALIZER};
  if (threads < 1) threads = 1;
  if (threads > num_tables) threads = num_tables;
  if (threads == 1) {
    for (int t = 0; t < num_tables; ++t) bags_one_table(&J, t);
    return;
  }
  pthread_t *th = (pthread_t *)malloc((size_t)threads * sizeof(pthread_t));
  for (int i = 0; i < threads; ++i) pthread_create(&th[i], NULL, bags_worker, &J);
  for (int i = 0; i < threads; ++i) pthread_join(th[i], NULL);
  free(th);
}

/* Number of host cores this process may run on. */
int oracle_num_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n > 0 ? (int)n : 1;
}

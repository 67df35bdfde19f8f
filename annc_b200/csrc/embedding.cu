// Host side of the embedding path: the grouped bag entry point and the plain-C
// twins of the TensorFlow fused embedding ops.  Validation order and messages
// follow the reference kernels so that its unit tests translate one to one.
#include <algorithm>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.h"
#include "embedding_kernels.cuh"

namespace annc {
namespace emb {

static inline int grid_for(long long items, int per_block, int cap = 148 * 16) {
  long long g = (items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return (int)g;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <int LANES, int VPL>
static void launch_bag(const BagParams& p, BagHeader* hdr, int* offsets, cudaStream_t s) {
  const long long groups = (long long)p.num_tables * p.batch;
  const long long groups_per_block = (256 / 32) * (32 / LANES);
  const long long blocks = (groups + groups_per_block - 1) / groups_per_block;
  if (p.shard_count > 1) bag_reduce_kernel<LANES, VPL, true><<<(unsigned)blocks, 256, 0, s>>>(p, hdr, offsets);
  else bag_reduce_kernel<LANES, VPL, false><<<(unsigned)blocks, 256, 0, s>>>(p, hdr, offsets);
}

// Blocks per SM of the persistent lookup-granular kernel (0: as many as fit, -n: n fewer), per
// calling thread: a caller that runs the kernel beside another gather-bound kernel of its own
// (the pooling kernel of the row exchange on a second stream) splits the SMs' slots between them.
static thread_local int t_stream_ctas_per_sm = 0;

template <int LANES, int VW, int VPL, int TILES, int INFLIGHT, int MINB>
static void launch_stream(const BagParams& p, BagHeader* hdr, cudaStream_t s) {
  static int per_sm[kMaxDevices] = {0};
  const int slot = device_slot();
  if (!per_sm[slot]) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, bag_stream_kernel<LANES, VW, VPL, TILES, INFLIGHT, MINB>,
                                                      256, 0) != cudaSuccess || n < 1)
      n = 2;
    per_sm[slot] = n;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, slot);
  StreamChunks sc;
  long long total = 0;
  for (int t = 0; t < p.num_tables; ++t) {
    sc.first[t] = (int)total;
    const long long n = p.t[t].nnz;
    total += n > 0 ? (n + LANES * TILES - 1) / (LANES * TILES) : (p.batch + 1023) / 1024;
  }
  sc.first[p.num_tables] = (int)total;
  // a persistent grid, no larger than the chunks there are
  const long long groups_per_block = (256 / 32) * (32 / LANES);
  const int ctas = t_stream_ctas_per_sm > 0 ? std::min(t_stream_ctas_per_sm, per_sm[slot])
                                            : std::max(1, per_sm[slot] + t_stream_ctas_per_sm);
  long long blocks = std::min<long long>((long long)sms * ctas, (total + groups_per_block - 1) / groups_per_block);
  bag_stream_kernel<LANES, VW, VPL, TILES, INFLIGHT, MINB><<<(unsigned)std::max<long long>(blocks, 1), 256, 0, s>>>(p, sc, hdr);
}

// Launches the bag kernels (+ the atomic route) for up to kMaxTables tables.
static int run_bags(const annc_bag_table* tables, int num_tables, int64_t dim, int id_kind,
                    int64_t ncols, int32_t col, int combiner, int64_t batch, int64_t out_stride,
                    BagHeader* hdr, int* offsets, cudaStream_t s, int shard_count = 1,
                    int shard_rank = 0, int skip_empty = 0) {
  BagParams p;
  memset(&p, 0, sizeof(p));
  p.shard_count = shard_count;
  p.shard_rank = shard_rank;
  p.skip_empty = skip_empty;
  p.num_tables = num_tables;
  p.id_kind = id_kind;
  p.combiner = combiner;
  p.col = col;
  p.ncols = ncols;
  p.batch = batch;
  p.dim = dim;
  p.out_stride = out_stride;
  long long max_nnz = 0;
  bool vec_ok = (dim % 4 == 0) && (out_stride % 4 == 0);
  for (int t = 0; t < num_tables; ++t) {
    if (tables[t].nnz >= (int64_t(1) << 31) - 1)
      return fail(ANNC_ERR_UNSUPPORTED, "more than 2^31-2 lookups in one table");
    if (tables[t].rows >= (int64_t(1) << 31))
      return fail(ANNC_ERR_UNSUPPORTED, "more than 2^31-1 rows in one (local) table");
    if (id_kind == 2 && tables[t].num_buckets < 1)
      return fail(ANNC_ERR_INVALID_ARGUMENT, "num_buckets must be >= 1");
    p.t[t].table = tables[t].table;
    p.t[t].ids = tables[t].ids;
    p.t[t].seg = tables[t].slice_input;
    p.t[t].out = tables[t].out;
    p.t[t].rows = (int)tables[t].rows;
    p.t[t].num_buckets = (unsigned long long)tables[t].num_buckets;
    p.t[t].magic = id_kind == 2 ? mod_magic(p.t[t].num_buckets) : 0;
    p.t[t].nnz = (int)tables[t].nnz;
    p.t[t].given_off = tables[t].offsets;
    max_nnz = std::max<long long>(max_nnz, tables[t].nnz);
    vec_ok = vec_ok && aligned16(tables[t].table) && aligned16(tables[t].out);
  }
  if (batch <= 0) return ANNC_OK;

  dim3 pre_grid(grid_for(max_nnz + 1, 256), num_tables);
  bool seg16 = ncols == 2, need_prepass = false, any_offsets = false;
  for (int t = 0; t < num_tables; ++t) {
    if (tables[t].offsets) {
      any_offsets = true;
      continue;
    }
    need_prepass = true;
    seg16 = seg16 && aligned16(tables[t].slice_input);
  }
  const int vecs = vec_ok ? (int)(dim / 4) : 0;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  timing_events(&ev0, &ev1);

  // Lookup-granular route: no prepass, one pass over ids and segment ids.  Taken when every
  // table comes with its index matrix (no caller-supplied offsets), unsharded, 16-byte rows.
  const bool stream = !any_offsets && shard_count == 1 && vecs >= 4 && batch < (1LL << 31) - 1 &&
                      (vecs == 4 || vecs == 8 || vecs == 16 || vecs == 32 || vecs == 64 || vecs == 128);
  if (stream) {
    if (ev0) cudaEventRecord(ev0, s);
    switch (vecs) {
      case 4: launch_stream<4, 4, 1, 8, 4, 5>(p, hdr, s); break;
      case 8: launch_stream<8, 4, 1, 8, 4, 5>(p, hdr, s); break;
      // dim 64 and 128: 32 bytes per lane (8 / 16 lanes per row), two row loads in flight: fewer
      // lanes repeat the per-lookup control instructions (0.70 ms against 0.79 ms with 16 lanes x
      // 16 bytes x 4 in flight on the 17.9 M lookups of the DLRM batch)
      case 16: launch_stream<8, 4, 2, 16, 2, 5>(p, hdr, s); break;
      case 32: launch_stream<16, 4, 2, 8, 2, 5>(p, hdr, s); break;
      case 64: launch_stream<32, 4, 2, 4, 4, 4>(p, hdr, s); break;
      default: launch_stream<32, 4, 4, 4, 2, 3>(p, hdr, s); break;
    }
    if (ev1) cudaEventRecord(ev1, s);
    dim3 rs_grid(148, num_tables);
    bag_stream_reset_kernel<<<rs_grid, 256, 0, s>>>(p, hdr, offsets);  // returns at once for sorted tables
    dim3 sc_grid(grid_for(max_nnz, 8, 148), num_tables);
    bag_scatter_kernel<<<sc_grid, 256, 0, s>>>(p, hdr, offsets);
    if (combiner == 1) {
      dim3 mean_grid(grid_for(batch * dim, 256, 148), num_tables);
      bag_scatter_mean_kernel<<<mean_grid, 256, 0, s>>>(p, hdr, offsets);
    }
    cudaError_t es = cudaGetLastError();
    if (es != cudaSuccess) return cuda_fail(es, "embedding bag launch");
    return ANNC_OK;
  }

  if (need_prepass) {  // tables that brought their offsets are skipped inside the kernel
    if (seg16) bag_prepass2_kernel<<<pre_grid, 256, 0, s>>>(p, hdr, offsets);
    else bag_prepass_kernel<<<pre_grid, 256, 0, s>>>(p, hdr, offsets);
  }

  if (ev0) cudaEventRecord(ev0, s);
  switch (vecs) {
    case 1: launch_bag<1, 1>(p, hdr, offsets, s); break;
    case 2: launch_bag<2, 1>(p, hdr, offsets, s); break;
    case 4: launch_bag<4, 1>(p, hdr, offsets, s); break;
    case 8: launch_bag<8, 1>(p, hdr, offsets, s); break;
    case 16: launch_bag<16, 1>(p, hdr, offsets, s); break;
    case 32: launch_bag<32, 1>(p, hdr, offsets, s); break;
    case 64: launch_bag<32, 2>(p, hdr, offsets, s); break;
    case 128: launch_bag<32, 4>(p, hdr, offsets, s); break;
    default: {
      const long long groups = (long long)num_tables * batch;
      bag_reduce_generic_kernel<<<(unsigned)((groups + 7) / 8), 256, 0, s>>>(p, hdr, offsets);
    }
  }
  if (ev1) cudaEventRecord(ev1, s);
  // Atomic route for tables whose segment ids were not sorted; the blocks return
  // at once for sorted tables.
  dim3 sc_grid(grid_for(max_nnz, 8, 148), num_tables);
  bag_scatter_kernel<<<sc_grid, 256, 0, s>>>(p, hdr, offsets);
  if (combiner == 1) {
    dim3 mean_grid(grid_for(batch * dim, 256, 148), num_tables);
    bag_scatter_mean_kernel<<<mean_grid, 256, 0, s>>>(p, hdr, offsets);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "embedding bag launch");
  return ANNC_OK;
}

// Exclusive scan of int32 on the device; *total_dev receives the sum.
// tile_scratch needs ceil(n / kScanTile) + 1 ints.
static void exclusive_scan(const int* in, long long n, int* out, int* tile_scratch,
                           int* total_dev, cudaStream_t s) {
  const long long tiles = std::max<long long>(1, (n + kScanTile - 1) / kScanTile);
  scan_tile_sums_kernel<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, n, tile_scratch);
  scan_tile_offsets_kernel<<<1, kScanThreads, 0, s>>>(tile_scratch, tiles, total_dev);
  scan_apply_kernel<<<(unsigned)tiles, kScanThreads, 0, s>>>(in, n, tile_scratch, out);
}

static size_t scan_scratch_ints(long long n) {
  return (size_t)std::max<long long>(1, (n + kScanTile - 1) / kScanTile) + 1;
}

// First-appearance unique of column `col` of src[n, ncols] (device).  Produces the
// number of unique keys (host), and optionally the unique keys, the int32 inverse
// map and an int64 copy of it.
struct UniqueResult {
  long long count = 0;
};

static int unique_first_appearance(Call& call, const int64_t* src, long long n, long long ncols,
                                   int col, long long* out_unique /*[n] or null*/,
                                   int* inverse32, long long* inverse64, UniqueResult* res) {
  cudaStream_t s = call.stream();
  long long cap = 16;
  while (cap < 2 * n + 2) cap <<= 1;
  auto* keys = static_cast<long long*>(call.scratch((cap + 1) * sizeof(long long)));
  auto* first = static_cast<int*>(call.scratch((cap + 1) * sizeof(int)));
  auto* slot_of = static_cast<int*>(call.scratch(std::max<long long>(n, 1) * sizeof(int)));
  auto* flag = static_cast<int*>(call.scratch(std::max<long long>(n, 1) * sizeof(int)));
  auto* rank = static_cast<int*>(call.scratch(std::max<long long>(n, 1) * sizeof(int)));
  auto* tiles = static_cast<int*>(call.scratch(scan_scratch_ints(n) * sizeof(int)));
  auto* total = static_cast<int*>(call.scratch(sizeof(int)));
  if (call.status() != ANNC_OK) return call.status();
  unique_init_kernel<<<grid_for(cap + 1, 256), 256, 0, s>>>(keys, first, cap);
  if (n > 0) {
    const int g = grid_for(n, 256);
    unique_insert_kernel<<<g, 256, 0, s>>>(src, n, ncols, col, keys, first, cap, slot_of);
    unique_flag_kernel<<<g, 256, 0, s>>>(slot_of, first, n, flag);
    exclusive_scan(flag, n, rank, tiles, total, s);
    unique_emit_kernel<<<g, 256, 0, s>>>(src, n, ncols, col, slot_of, flag, rank, first, out_unique);
    unique_inverse_kernel<<<g, 256, 0, s>>>(slot_of, first, n, inverse32, inverse64);
    int h = 0;
    ANNC_TRY(call.read_host(total, sizeof(int), &h));
    res->count = h;
  } else {
    res->count = 0;
  }
  return ANNC_OK;
}

static int check_err_word(Call& call, const int* err_dev, int* bits) {
  return call.read_host(err_dev, sizeof(int), bits);
}

}  // namespace emb
}  // namespace annc

using namespace annc;
using namespace annc::emb;

extern "C" {

size_t annc_embed_bag_workspace_bytes(int num_tables, int64_t batch) {
  if (num_tables < 1) num_tables = 1;
  if (batch < 0) batch = 0;
  size_t off = (size_t)num_tables * (size_t)(batch + 1) * sizeof(int);
  return kHeaderBytes + ((off + 255) & ~size_t(255));
}

void annc_embed_bag_set_stream_ctas_per_sm(int ctas_per_sm) { t_stream_ctas_per_sm = ctas_per_sm; }

int annc_embed_bags_dev(const annc_bag_table* tables, int num_tables, int64_t dim, int id_kind,
                        int64_t ncols, int32_t col, int combiner, int64_t batch,
                        int64_t out_stride, void* workspace, size_t workspace_bytes,
                        void* stream) {
  ANNC_REQUIRE(tables && num_tables >= 1, ANNC_ERR_INVALID_ARGUMENT, "no tables");
  ANNC_REQUIRE(combiner == 0 || combiner == 1, ANNC_ERR_INVALID_ARGUMENT, "combiner must be 0 or 1");
  ANNC_REQUIRE(id_kind >= 0 && id_kind <= 2, ANNC_ERR_INVALID_ARGUMENT, "id_kind must be 0, 1 or 2");
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  ANNC_REQUIRE(dim >= 1 && out_stride >= dim, ANNC_ERR_INVALID_ARGUMENT, "bad dim / out_stride");
  ANNC_REQUIRE(workspace && workspace_bytes >= annc_embed_bag_workspace_bytes(num_tables, batch),
               ANNC_ERR_INVALID_ARGUMENT, "workspace too small");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* hdr = static_cast<BagHeader*>(workspace);
  int* offsets = reinterpret_cast<int*>(static_cast<char*>(workspace) + kHeaderBytes);
  ANNC_CUDA(cudaMemsetAsync(hdr, 0, kHeaderBytes, s));
  for (int t0 = 0; t0 < num_tables; t0 += kMaxTables) {
    const int nt = std::min(kMaxTables, num_tables - t0);
    if (t0 > 0) ANNC_CUDA(cudaMemsetAsync(hdr->unsorted, 0, sizeof(hdr->unsorted), s));
    ANNC_TRY(run_bags(tables + t0, nt, dim, id_kind, ncols, col, combiner, batch, out_stride, hdr,
                      offsets + (size_t)t0 * (size_t)(batch + 1), s));
  }
  return ANNC_OK;
}

static int bags_sharded(const annc_bag_table* tables, int num_tables, int64_t dim, int id_kind,
                        int64_t ncols, int32_t col, int combiner, int64_t batch,
                        int64_t out_stride, int shard_count, int shard_rank, int skip_empty,
                        void* workspace, size_t workspace_bytes, void* stream) {
  ANNC_REQUIRE(tables && num_tables >= 1, ANNC_ERR_INVALID_ARGUMENT, "no tables");
  ANNC_REQUIRE(combiner == 0 || combiner == 1, ANNC_ERR_INVALID_ARGUMENT, "combiner must be 0 or 1");
  ANNC_REQUIRE(id_kind >= 0 && id_kind <= 2, ANNC_ERR_INVALID_ARGUMENT, "id_kind must be 0, 1 or 2");
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  ANNC_REQUIRE(dim >= 1 && out_stride >= dim, ANNC_ERR_INVALID_ARGUMENT, "bad dim / out_stride");
  ANNC_REQUIRE(shard_count >= 1 && shard_count <= 32 && shard_rank >= 0 && shard_rank < shard_count,
               ANNC_ERR_INVALID_ARGUMENT, "bad shard_count / shard_rank");
  ANNC_REQUIRE(workspace && workspace_bytes >= annc_embed_bag_workspace_bytes(num_tables, batch),
               ANNC_ERR_INVALID_ARGUMENT, "workspace too small");
  if (skip_empty)
    for (int t = 0; t < num_tables; ++t)
      ANNC_REQUIRE(tables[t].offsets, ANNC_ERR_INVALID_ARGUMENT,
                   "skipping unowned bags needs caller-supplied sorted bag offsets");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* hdr = static_cast<BagHeader*>(workspace);
  int* offsets = reinterpret_cast<int*>(static_cast<char*>(workspace) + kHeaderBytes);
  ANNC_CUDA(cudaMemsetAsync(hdr, 0, kHeaderBytes, s));
  for (int t0 = 0; t0 < num_tables; t0 += kMaxTables) {
    const int nt = std::min(kMaxTables, num_tables - t0);
    if (t0 > 0) ANNC_CUDA(cudaMemsetAsync(hdr->unsorted, 0, sizeof(hdr->unsorted), s));
    ANNC_TRY(run_bags(tables + t0, nt, dim, id_kind, ncols, col, combiner, batch, out_stride, hdr,
                      offsets + (size_t)t0 * (size_t)(batch + 1), s, shard_count, shard_rank,
                      skip_empty));
  }
  return ANNC_OK;
}

int annc_embed_bags_sharded_dev(const annc_bag_table* tables, int num_tables, int64_t dim,
                                int id_kind, int64_t ncols, int32_t col, int combiner,
                                int64_t batch, int64_t out_stride, int shard_count,
                                int shard_rank, void* workspace, size_t workspace_bytes,
                                void* stream) {
  return bags_sharded(tables, num_tables, dim, id_kind, ncols, col, combiner, batch, out_stride,
                      shard_count, shard_rank, 0, workspace, workspace_bytes, stream);
}

int annc_embed_bags_exchange_dev(const annc_bag_table* tables, int num_tables, int64_t dim,
                                 int id_kind, int combiner, int64_t batch, int64_t out_stride,
                                 int shard_count, int shard_rank, void* workspace,
                                 size_t workspace_bytes, void* stream) {
  return bags_sharded(tables, num_tables, dim, id_kind, 1, 0, combiner, batch, out_stride,
                      shard_count, shard_rank, 1, workspace, workspace_bytes, stream);
}

int annc_embed_bag_owner_mask_dev(const annc_bag_table* tables, int num_tables, int id_kind,
                                  int64_t batch, int shard_count, uint32_t* mask, void* stream) {
  ANNC_REQUIRE(tables && num_tables >= 1 && mask, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(id_kind >= 0 && id_kind <= 2, ANNC_ERR_INVALID_ARGUMENT, "id_kind must be 0, 1 or 2");
  ANNC_REQUIRE(shard_count >= 1 && shard_count <= 32, ANNC_ERR_INVALID_ARGUMENT, "bad shard_count");
  if (batch <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int t0 = 0; t0 < num_tables; t0 += kMaxTables) {
    const int nt = std::min(kMaxTables, num_tables - t0);
    BagParams p;
    memset(&p, 0, sizeof(p));
    p.num_tables = nt;
    p.id_kind = id_kind;
    p.batch = batch;
    p.shard_count = shard_count;
    for (int t = 0; t < nt; ++t) {
      const annc_bag_table& T = tables[t0 + t];
      ANNC_REQUIRE(T.offsets && (T.ids || T.nnz == 0), ANNC_ERR_INVALID_ARGUMENT,
                   "owner mask needs ids and bag offsets");
      if (id_kind == 2 && T.num_buckets < 1)
        return fail(ANNC_ERR_INVALID_ARGUMENT, "num_buckets must be >= 1");
      p.t[t].ids = T.ids;
      ANNC_REQUIRE(T.nnz < (int64_t(1) << 31) - 1, ANNC_ERR_UNSUPPORTED,
                   "more than 2^31-2 lookups in one table");
      p.t[t].num_buckets = (unsigned long long)T.num_buckets;
      p.t[t].magic = id_kind == 2 ? mod_magic(p.t[t].num_buckets) : 0;
      p.t[t].nnz = (int)T.nnz;
      p.t[t].given_off = T.offsets;
    }
    const long long groups = (long long)nt * batch;
    bag_owner_mask_kernel<<<(unsigned)((groups + 15) / 16), 256, 0, s>>>(
        p, mask + (size_t)t0 * (size_t)batch);
  }
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_embed_bag_prepass_dev(const annc_bag_table* tables, int num_tables, int64_t ncols,
                               int32_t col, int64_t batch, void* workspace, size_t workspace_bytes,
                               void* stream) {
  ANNC_REQUIRE(tables && num_tables >= 1, ANNC_ERR_INVALID_ARGUMENT, "no tables");
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  ANNC_REQUIRE(workspace && workspace_bytes >= annc_embed_bag_workspace_bytes(num_tables, batch),
               ANNC_ERR_INVALID_ARGUMENT, "workspace too small");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* hdr = static_cast<BagHeader*>(workspace);
  int* offsets = reinterpret_cast<int*>(static_cast<char*>(workspace) + kHeaderBytes);
  ANNC_CUDA(cudaMemsetAsync(hdr, 0, kHeaderBytes, s));
  if (batch <= 0) return ANNC_OK;
  for (int t0 = 0; t0 < num_tables; t0 += kMaxTables) {
    const int nt = std::min(kMaxTables, num_tables - t0);
    BagParams p;
    memset(&p, 0, sizeof(p));
    p.num_tables = nt;
    p.col = col;
    p.ncols = ncols;
    p.batch = batch;
    long long max_nnz = 0;
    bool seg16 = ncols == 2;
    for (int t = 0; t < nt; ++t) {
      ANNC_REQUIRE(tables[t0 + t].nnz < (int64_t(1) << 31) - 1, ANNC_ERR_UNSUPPORTED,
                   "more than 2^31-2 lookups in one table");
      p.t[t].seg = tables[t0 + t].slice_input;
      p.t[t].nnz = tables[t0 + t].nnz;
      max_nnz = std::max<long long>(max_nnz, tables[t0 + t].nnz);
      seg16 = seg16 && aligned16(tables[t0 + t].slice_input);
    }
    // the marks of unsorted tables are per launch; a later launch reuses the slots
    dim3 grid(grid_for(max_nnz + 1, 256), nt);
    int* off = offsets + (size_t)t0 * (size_t)(batch + 1);
    if (seg16) bag_prepass2_kernel<<<grid, 256, 0, s>>>(p, hdr, off);
    else bag_prepass_kernel<<<grid, 256, 0, s>>>(p, hdr, off);
  }
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_embed_bag_check(void* workspace, void* stream, int* error_bits) {
  ANNC_REQUIRE(workspace && error_bits, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ANNC_CUDA(cudaMemcpyAsync(error_bits, workspace, sizeof(int), cudaMemcpyDeviceToHost, s));
  ANNC_CUDA(cudaStreamSynchronize(s));
  return ANNC_OK;
}

// ---------------------------------------------------------------- bags without a workspace
// Scratch of annc_embed_bags_static_dev: lives in the library image, so every GPU
// that loads the library holds these 8 MiB + 512 B until the process exits.
constexpr size_t kStaticBagInts = size_t(2) << 20;  // offsets: num_tables * (batch + 1) ints
static __device__ __align__(256) unsigned char g_bag_scratch[kHeaderBytes + kStaticBagInts * sizeof(int)];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {nullptr};

// In host code `g_bag_scratch` is only a handle for the runtime, never a device
// address: the address is asked for once per device, with that device current.
int static_scratch(void** out) {
  int dev = -1;
  ANNC_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(ANNC_ERR_UNSUPPORTED, "device ordinal out of range");
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    ANNC_CUDA(cudaGetSymbolAddress(&p, g_bag_scratch));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return ANNC_OK;
}
}  // namespace

int annc_embed_bags_static_dev(const annc_bag_table* tables, int num_tables, int64_t dim,
                               int id_kind, int64_t ncols, int32_t col, int combiner,
                               int64_t batch, int64_t out_stride, int* error_bits_dev,
                               void* stream) {
  ANNC_REQUIRE(tables && num_tables >= 1, ANNC_ERR_INVALID_ARGUMENT, "no tables");
  ANNC_REQUIRE(combiner == 0 || combiner == 1, ANNC_ERR_INVALID_ARGUMENT, "combiner must be 0 or 1");
  ANNC_REQUIRE(id_kind >= 0 && id_kind <= 2, ANNC_ERR_INVALID_ARGUMENT, "id_kind must be 0, 1 or 2");
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  ANNC_REQUIRE(dim >= 1 && out_stride >= dim && batch >= 0, ANNC_ERR_INVALID_ARGUMENT,
               "bad dim / out_stride / batch");
  if ((size_t)num_tables * (size_t)(batch + 1) > kStaticBagInts)
    return fail(ANNC_ERR_UNSUPPORTED,
                "annc_embed_bags_static_dev: num_tables * (batch + 1) = %lld exceeds the built-in "
                "scratch of %lld entries; use annc_embed_bags_dev with a caller workspace",
                (long long)num_tables * (long long)(batch + 1), (long long)kStaticBagInts);
  void* ws = nullptr;
  ANNC_TRY(static_scratch(&ws));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  auto* hdr = static_cast<BagHeader*>(ws);
  int* offsets = reinterpret_cast<int*>(static_cast<char*>(ws) + kHeaderBytes);
  // The array keeps the previous call's contents: the header (error word, unsorted
  // marks) must start at zero.  The offsets are written before they are read: by the
  // prepass on the offsets route, and as per-bag counters cleared by the reset kernel for a
  // table whose segment ids turn out unsorted.
  ANNC_CUDA(cudaMemsetAsync(hdr, 0, kHeaderBytes, s));
  for (int t0 = 0; t0 < num_tables; t0 += kMaxTables) {
    const int nt = std::min(kMaxTables, num_tables - t0);
    if (t0 > 0) ANNC_CUDA(cudaMemsetAsync(hdr->unsorted, 0, sizeof(hdr->unsorted), s));
    ANNC_TRY(run_bags(tables + t0, nt, dim, id_kind, ncols, col, combiner, batch, out_stride, hdr,
                      offsets + (size_t)t0 * (size_t)(batch + 1), s));
  }
  if (error_bits_dev)
    ANNC_CUDA(cudaMemcpyAsync(error_bits_dev, &hdr->err_bits, sizeof(int), cudaMemcpyDeviceToDevice, s));
  return ANNC_OK;
}

// ---------------------------------------------------------------- KPFusedSparseSegmentReduce

int annc_KPFusedSparseSegmentReduce(const annc_tensor* data, const annc_tensor* indices,
                                    const annc_tensor* slice_input, const annc_tensor* begin,
                                    const annc_tensor* begin_1, int combiner,
                                    annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(combiner == 0 || combiner == 1, ANNC_ERR_INVALID_ARGUMENT, "combiner must be 0 or 1");
  ANNC_REQUIRE(data && indices && slice_input && begin && begin_1 && alloc,
               ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(data->rank == 2, ANNC_ERR_INVALID_ARGUMENT, "input must be 2-D");
  ANNC_REQUIRE(slice_input->rank == 2, ANNC_ERR_INVALID_ARGUMENT, "slice input must be 2-D");
  ANNC_REQUIRE(numel(*begin) == 2, ANNC_ERR_INVALID_ARGUMENT, "begin must have 2 elements");
  ANNC_REQUIRE(numel(*begin_1) == 1, ANNC_ERR_INVALID_ARGUMENT, "begin_1 must have 1 element");
  ANNC_REQUIRE(indices->dtype == ANNC_I32 || indices->dtype == ANNC_I64, ANNC_ERR_INVALID_ARGUMENT,
               "indices must be int32 or int64");
  Call call;
  int32_t b[2], b1;
  ANNC_TRY(call.read_host(begin->data, sizeof(b), b));
  ANNC_TRY(call.read_host(begin_1->data, sizeof(b1), &b1));
  const int64_t nnz = indices->rank >= 1 ? indices->dims[0] : 1;
  const int64_t dim = data->dims[1], ncols = slice_input->dims[1];
  const int32_t col = b[1];
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  ANNC_REQUIRE(nnz == slice_input->dims[0], ANNC_ERR_INVALID_ARGUMENT,
               "indices and slice_input.dim_zie(0) should have same size");

  cudaStream_t s = call.stream();
  const float* d_data = call.in_constant((const float*)data->data, (size_t)numel(*data));
  const void* d_idx = call.in(indices->data, (size_t)nnz * dtype_size(indices->dtype));
  const int64_t* d_seg = call.in((const int64_t*)slice_input->data, (size_t)(nnz * ncols));
  auto* d_max = static_cast<long long*>(call.scratch(sizeof(long long)));
  if (call.status() != ANNC_OK) return call.status();

  // batch = max segment id + 1 (max starts at 0), needed on the host to size output 0.
  ANNC_CUDA(cudaMemsetAsync(d_max, 0, sizeof(long long), s));
  if (nnz > 0) seg_max_kernel<<<grid_for(nnz, 256), 256, 0, s>>>(d_seg, nnz, ncols, col, d_max);
  long long max_seg = 0;
  ANNC_TRY(call.read_host(d_max, sizeof(long long), &max_seg));
  const int64_t batch = max_seg + 1;

  const int64_t dims0[2] = {batch, dim};
  float* out0 = static_cast<float*>(alloc(ctx, 0, ANNC_F32, 2, dims0));
  int32_t* out1 = static_cast<int32_t*>(alloc(ctx, 1, ANNC_I32, 0, nullptr));
  ANNC_REQUIRE(out0 && out1, ANNC_ERR_INTERNAL, "output allocation failed");
  float* d_out = call.out(out0, (size_t)(batch * dim));
  void* ws = call.scratch(annc_embed_bag_workspace_bytes(1, batch));
  if (call.status() != ANNC_OK) return call.status();

  annc_bag_table tb;
  tb.table = d_data;
  tb.rows = data->dims[0];
  tb.num_buckets = 1;
  tb.ids = d_idx;
  tb.slice_input = d_seg;
  tb.nnz = nnz;
  tb.out = d_out;
  tb.offsets = nullptr;
  auto* hdr = static_cast<BagHeader*>(ws);
  ANNC_CUDA(cudaMemsetAsync(hdr, 0, kHeaderBytes, s));
  ANNC_TRY(run_bags(&tb, 1, dim, indices->dtype == ANNC_I64 ? 1 : 0, ncols, col, combiner, batch,
                    dim, hdr, reinterpret_cast<int*>(static_cast<char*>(ws) + kHeaderBytes), s));
  // Second output: begin_1[0] == 0 ? batch : embedding size (reference :81-83).
  const int32_t slice_out = (b1 == 0) ? (int32_t)batch : (int32_t)dim;
  if (call.is_device(out1)) {
    ANNC_CUDA(cudaMemcpyAsync(out1, &slice_out, sizeof(int32_t), cudaMemcpyHostToDevice, s));
    ANNC_CUDA(cudaStreamSynchronize(s));
  } else {
    *out1 = slice_out;
  }
  int bits = 0;
  ANNC_TRY(check_err_word(call, &hdr->err_bits, &bits));
  ANNC_TRY(call.finish());
  if (bits & kErrRow) return fail(ANNC_ERR_INVALID_ARGUMENT, "indices out of range of input rows");
  if (bits & kErrSegment) return fail(ANNC_ERR_INVALID_ARGUMENT, "segment ids must be >= 0");
  return ANNC_OK;
}

// ---------------------------------------------------------------- KPFusedSparseSegmentReduceNonzero

int annc_KPFusedSparseSegmentReduceNonzero(const annc_tensor* data, const annc_tensor* indices,
                                           const annc_tensor* slice_input,
                                           const annc_tensor* begin, int combiner,
                                           annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(combiner == 0 || combiner == 1, ANNC_ERR_INVALID_ARGUMENT, "combiner must be 0 or 1");
  ANNC_REQUIRE(data && indices && slice_input && begin && alloc, ANNC_ERR_INVALID_ARGUMENT,
               "null argument");
  ANNC_REQUIRE(data->rank == 1 || data->rank == 2, ANNC_ERR_INVALID_ARGUMENT,
               "Input data must be a 1-D vector or 2-D matrix");
  ANNC_REQUIRE(slice_input->rank == 2, ANNC_ERR_INVALID_ARGUMENT, "slice input must be 2-D");
  ANNC_REQUIRE(numel(*begin) == 2, ANNC_ERR_INVALID_ARGUMENT, "begin must have 2 elements");
  ANNC_REQUIRE(indices->dtype == ANNC_I32 || indices->dtype == ANNC_I64, ANNC_ERR_INVALID_ARGUMENT,
               "indices must be int32 or int64");
  Call call;
  int32_t b[2];
  ANNC_TRY(call.read_host(begin->data, sizeof(b), b));
  const int64_t nnz = indices->rank >= 1 ? indices->dims[0] : 1;
  const int64_t ncols = slice_input->dims[1];
  const int32_t col = b[1];
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  ANNC_REQUIRE(nnz == slice_input->dims[0], ANNC_ERR_INVALID_ARGUMENT,
               "indices and slice_input.dim_size(0) should have same size");
  const int rank = data->rank;
  const int64_t dim = rank == 2 ? data->dims[1] : 1;

  cudaStream_t s = call.stream();
  const float* d_data = call.in_constant((const float*)data->data, (size_t)numel(*data));
  const void* d_idx = call.in(indices->data, (size_t)nnz * dtype_size(indices->dtype));
  const int64_t* d_seg = call.in((const int64_t*)slice_input->data, (size_t)(nnz * ncols));
  auto* d_max = static_cast<long long*>(call.scratch(sizeof(long long)));
  auto* d_order = static_cast<long long*>(call.scratch(std::max<int64_t>(nnz, 1) * sizeof(long long)));
  auto* d_inv64 = static_cast<long long*>(call.scratch(std::max<int64_t>(nnz, 1) * sizeof(long long)));
  if (call.status() != ANNC_OK) return call.status();

  ANNC_CUDA(cudaMemsetAsync(d_max, 0, sizeof(long long), s));
  if (nnz > 0) seg_max_kernel<<<grid_for(nnz, 256), 256, 0, s>>>(d_seg, nnz, ncols, col, d_max);

  // Segments in first-appearance order; every lookup gets the rank of its segment.
  UniqueResult ur;
  ANNC_TRY(unique_first_appearance(call, d_seg, nnz, ncols, col, d_order, nullptr, d_inv64, &ur));
  long long max_seg = 0;
  ANNC_TRY(call.read_host(d_max, sizeof(long long), &max_seg));
  const int64_t batch = max_seg + 1, nseg = ur.count;

  const int64_t shape_dims[1] = {rank};
  int32_t* out_shape = static_cast<int32_t*>(alloc(ctx, 0, ANNC_I32, 1, shape_dims));
  ANNC_REQUIRE(out_shape, ANNC_ERR_INTERNAL, "output allocation failed");
  int32_t shape_host[2] = {(int32_t)batch, (int32_t)dim};
  if (call.is_device(out_shape)) {
    ANNC_CUDA(cudaMemcpyAsync(out_shape, shape_host, rank * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    ANNC_CUDA(cudaStreamSynchronize(s));
  } else {
    memcpy(out_shape, shape_host, rank * sizeof(int32_t));
  }

  // Dense [nseg, dim] reduce over the ranks (non-decreasing when the segment ids are
  // sorted, so the exact route applies), then compaction of the non-zeros.
  const int64_t total = nseg * dim;
  auto* d_dense = static_cast<float*>(call.scratch(std::max<int64_t>(total, 1) * sizeof(float)));
  void* ws = call.scratch(annc_embed_bag_workspace_bytes(1, nseg));
  auto* d_flag = static_cast<int*>(call.scratch(std::max<int64_t>(total, 1) * sizeof(int)));
  auto* d_pos = static_cast<int*>(call.scratch(std::max<int64_t>(total, 1) * sizeof(int)));
  auto* d_tiles = static_cast<int*>(call.scratch(scan_scratch_ints(total) * sizeof(int)));
  auto* d_total = static_cast<int*>(call.scratch(sizeof(int)));
  if (call.status() != ANNC_OK) return call.status();
  auto* hdr = static_cast<BagHeader*>(ws);
  ANNC_CUDA(cudaMemsetAsync(hdr, 0, kHeaderBytes, s));
  int nz = 0;
  if (nseg > 0) {
    annc_bag_table tb;
    tb.table = d_data;
    tb.rows = data->dims[0];
    tb.num_buckets = 1;
    tb.ids = d_idx;
    tb.slice_input = reinterpret_cast<const int64_t*>(d_inv64);
    tb.nnz = nnz;
    tb.out = d_dense;
    tb.offsets = nullptr;
    ANNC_TRY(run_bags(&tb, 1, dim, indices->dtype == ANNC_I64 ? 1 : 0, 1, 0, combiner, nseg, dim,
                      hdr, reinterpret_cast<int*>(static_cast<char*>(ws) + kHeaderBytes), s));
    nonzero_flag_kernel<<<grid_for(total, 256), 256, 0, s>>>(d_dense, total, d_flag);
    exclusive_scan(d_flag, total, d_pos, d_tiles, d_total, s);
    ANNC_TRY(call.read_host(d_total, sizeof(int), &nz));
  }
  const int64_t idx_dims[2] = {nz, rank};
  const int64_t val_dims[1] = {nz};
  int32_t* out_idx = static_cast<int32_t*>(alloc(ctx, 1, ANNC_I32, 2, idx_dims));
  float* out_val = static_cast<float*>(alloc(ctx, 2, ANNC_F32, 1, val_dims));
  ANNC_REQUIRE((out_idx && out_val) || nz == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  if (nz > 0) {
    int32_t* d_oidx = call.out(out_idx, (size_t)nz * rank);
    float* d_oval = call.out(out_val, (size_t)nz);
    if (call.status() != ANNC_OK) return call.status();
    nonzero_emit_kernel<<<grid_for(total, 256), 256, 0, s>>>(d_dense, total, dim, rank, d_order,
                                                             d_flag, d_pos, d_oidx, d_oval);
  }
  int bits = 0;
  ANNC_TRY(check_err_word(call, &hdr->err_bits, &bits));
  ANNC_TRY(call.finish());
  if (bits & kErrRow) return fail(ANNC_ERR_INVALID_ARGUMENT, "indices out of range of input rows");
  return ANNC_OK;
}

// ---------------------------------------------------------------- KPFusedGather

int annc_KPFusedGather(const annc_tensor* data, const annc_tensor* keys, const annc_tensor* begin,
                       annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(data && keys && begin && alloc, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(keys->rank == 2, ANNC_ERR_INTERNAL, "Input key must be 2D");
  ANNC_REQUIRE(data->rank == 2, ANNC_ERR_INTERNAL, "Embedding table shape must be 2D");
  ANNC_REQUIRE(numel(*begin) == 2, ANNC_ERR_INTERNAL, "begin must be same as keys rank");
  Call call;
  int32_t b[2];
  ANNC_TRY(call.read_host(begin->data, sizeof(b), b));
  const int32_t col = b[1];
  const int64_t nnz = keys->dims[0], ncols = keys->dims[1], dim = data->dims[1];
  ANNC_REQUIRE(col < ncols, ANNC_ERR_INTERNAL, "slice cols out of keys range");
  ANNC_REQUIRE(col >= 0, ANNC_ERR_INTERNAL, "slice cols out of keys range");

  cudaStream_t s = call.stream();
  const int64_t idx_dims[1] = {nnz};
  int32_t* out_inv = static_cast<int32_t*>(alloc(ctx, 1, ANNC_I32, 1, idx_dims));
  ANNC_REQUIRE(out_inv || nnz == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  const float* d_data = call.in_constant((const float*)data->data, (size_t)numel(*data));
  const int64_t* d_keys = call.in((const int64_t*)keys->data, (size_t)(nnz * ncols));
  int32_t* d_inv = nnz > 0 ? call.out(out_inv, (size_t)nnz) : nullptr;
  auto* d_unique = static_cast<long long*>(call.scratch(std::max<int64_t>(nnz, 1) * sizeof(long long)));
  auto* d_err = static_cast<int*>(call.scratch(sizeof(int)));
  if (call.status() != ANNC_OK) return call.status();
  ANNC_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
  UniqueResult ur;
  ANNC_TRY(unique_first_appearance(call, d_keys, nnz, ncols, col, d_unique, d_inv, nullptr, &ur));
  const int64_t nu = ur.count;

  const int64_t u_dims[1] = {nu};
  const int64_t d_dims[2] = {nu, dim};
  int64_t* out_unique = static_cast<int64_t*>(alloc(ctx, 0, ANNC_I64, 1, u_dims));
  float* out_rows = static_cast<float*>(alloc(ctx, 2, ANNC_F32, 2, d_dims));
  ANNC_REQUIRE((out_unique && out_rows) || nu == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  if (nu > 0) {
    if (call.is_device(out_unique)) {
      ANNC_CUDA(cudaMemcpyAsync(out_unique, d_unique, nu * sizeof(int64_t), cudaMemcpyDeviceToDevice, s));
    } else {
      ANNC_CUDA(cudaMemcpyAsync(out_unique, d_unique, nu * sizeof(int64_t), cudaMemcpyDeviceToHost, s));
    }
    float* d_rows = call.out(out_rows, (size_t)(nu * dim));
    if (call.status() != ANNC_OK) return call.status();
    unique_rows_kernel<<<grid_for(nu, 8), 256, 0, s>>>(d_data, data->dims[0], dim, d_unique, nu,
                                                       d_rows, d_err);
  }
  int bits = 0;
  ANNC_TRY(check_err_word(call, d_err, &bits));
  ANNC_TRY(call.finish());
  if (bits & kErrRow) return fail(ANNC_ERR_INTERNAL, "idx out of table range");
  return ANNC_OK;
}

// ---------------------------------------------------------------- KPFusedSparseDynamicStitch

int annc_KPFusedSparseDynamicStitch(const annc_tensor* x, const annc_tensor* tables,
                                    int num_tables, annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(x && tables && alloc, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(num_tables > 1, ANNC_ERR_INVALID_ARGUMENT, "num partitions must > 1");
  int64_t dim = 0;
  for (int i = 0; i < num_tables; ++i) {
    ANNC_REQUIRE(tables[i].rank == 2, ANNC_ERR_INVALID_ARGUMENT, "input dims must == 2");
    if (i == 0) {
      dim = tables[i].dims[1];
    } else {
      ANNC_REQUIRE(tables[i].dims[1] == dim, ANNC_ERR_INVALID_ARGUMENT,
                   "All inputs must have same second dimension");
    }
  }
  ANNC_REQUIRE(dim > 0, ANNC_ERR_INVALID_ARGUMENT, "output_stride must > 0");
  Call call;
  cudaStream_t s = call.stream();
  const int64_t n = numel(*x);
  const int64_t out_dims[2] = {n, dim};
  float* out = static_cast<float*>(alloc(ctx, 0, ANNC_F32, 2, out_dims));
  ANNC_REQUIRE(out || n == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  std::vector<const float*> ptrs(num_tables);
  std::vector<long long> rows(num_tables);
  for (int i = 0; i < num_tables; ++i) {
    ptrs[i] = call.in_constant((const float*)tables[i].data, (size_t)numel(tables[i]));
    rows[i] = tables[i].dims[0];
  }
  auto* d_ptrs = static_cast<const float**>(call.scratch(num_tables * sizeof(float*)));
  auto* d_rows = static_cast<long long*>(call.scratch(num_tables * sizeof(long long)));
  auto* d_err = static_cast<int*>(call.scratch(sizeof(int)));
  const int64_t* d_x = call.in((const int64_t*)x->data, (size_t)n);
  float* d_out = n > 0 ? call.out(out, (size_t)(n * dim)) : nullptr;
  if (call.status() != ANNC_OK) return call.status();
  ANNC_CUDA(cudaMemcpyAsync(d_ptrs, ptrs.data(), num_tables * sizeof(float*), cudaMemcpyHostToDevice, s));
  ANNC_CUDA(cudaMemcpyAsync(d_rows, rows.data(), num_tables * sizeof(long long), cudaMemcpyHostToDevice, s));
  ANNC_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
  // The host vectors above must outlive the copies.
  ANNC_CUDA(cudaStreamSynchronize(s));
  if (n > 0) {
    StitchParams g{d_ptrs, d_rows, (const long long*)d_x, d_out, n, dim, num_tables};
    stitch_kernel<<<grid_for(n, 8), 256, 0, s>>>(g, d_err);
  }
  int bits = 0;
  ANNC_TRY(check_err_word(call, d_err, &bits));
  ANNC_TRY(call.finish());
  if (bits & kErrRow) return fail(ANNC_ERR_INVALID_ARGUMENT, "row_id out of range.");
  return ANNC_OK;
}

// ---------------------------------------------------------------- hash-bucket family

int annc_KPFusedEmbeddingWithHashBucket(const annc_tensor* fingerprints, const annc_tensor* empty,
                                        const annc_tensor* variable, int64_t num_buckets,
                                        int bounded, annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(fingerprints && variable && alloc, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(num_buckets >= 1, ANNC_ERR_INVALID_ARGUMENT, "num_buckets must be >= 1");
  ANNC_REQUIRE(variable->rank == 2, ANNC_ERR_INVALID_ARGUMENT, "variable must be 2-D");
  ANNC_REQUIRE(variable->dtype == ANNC_F32, ANNC_ERR_INVALID_ARGUMENT, "Expect float weight");
  Call call;
  cudaStream_t s = call.stream();
  const int64_t n = bounded ? numel(*fingerprints) : (fingerprints->rank >= 1 ? fingerprints->dims[0] : 1);
  const int64_t dim = variable->dims[1];
  const int64_t out_dims[2] = {n, dim};
  float* out = static_cast<float*>(alloc(ctx, 0, ANNC_F32, 2, out_dims));
  ANNC_REQUIRE(out || n * dim == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  if (n * dim == 0) return ANNC_OK;
  GatherParams g;
  memset(&g, 0, sizeof(g));
  g.table = call.in_constant((const float*)variable->data, (size_t)numel(*variable));
  g.ids = call.in(fingerprints->data, (size_t)n * 8);
  g.empty = (empty && empty->data) ? call.in((const unsigned char*)empty->data, (size_t)n) : nullptr;
  g.out = call.out(out, (size_t)(n * dim));
  g.n = n;
  g.rows = variable->dims[0];
  g.dim = dim;
  g.num_buckets = (unsigned long long)num_buckets;
  g.mode = bounded ? 1 : 0;
  auto* d_err = static_cast<int*>(call.scratch(sizeof(int)));
  if (call.status() != ANNC_OK) return call.status();
  ANNC_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
  row_gather_kernel<<<grid_for(n, 8), 256, 0, s>>>(g, d_err);
  int bits = 0;
  ANNC_TRY(check_err_word(call, d_err, &bits));
  ANNC_TRY(call.finish());
  if (bits & kErrRow)
    return fail(ANNC_ERR_INVALID_ARGUMENT, "hash bucket outside the variable (num_buckets > rows)");
  return ANNC_OK;
}

int annc_sparse_embedding2(const annc_tensor* ids, const annc_tensor* table, int64_t lo,
                           int64_t hi, int64_t dflt, float* out) {
  ANNC_REQUIRE(ids && table && out, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(table->rank == 2, ANNC_ERR_INVALID_ARGUMENT, "table must be 2-D");
  ANNC_REQUIRE(ids->dtype == ANNC_I32 || ids->dtype == ANNC_I64, ANNC_ERR_INVALID_ARGUMENT,
               "ids must be int32 or int64");
  Call call;
  cudaStream_t s = call.stream();
  const int64_t n = numel(*ids), dim = table->dims[1];
  if (n * dim == 0) return ANNC_OK;
  GatherParams g;
  memset(&g, 0, sizeof(g));
  g.table = call.in_constant((const float*)table->data, (size_t)numel(*table));
  g.ids = call.in(ids->data, (size_t)n * dtype_size(ids->dtype));
  g.out = call.out(out, (size_t)(n * dim));
  g.n = n;
  g.rows = table->dims[0];
  g.dim = dim;
  g.num_buckets = 1;
  g.lo = lo;
  g.hi = hi;
  g.dflt = dflt;
  g.mode = 2;
  g.ids64 = ids->dtype == ANNC_I64;
  auto* d_err = static_cast<int*>(call.scratch(sizeof(int)));
  if (call.status() != ANNC_OK) return call.status();
  ANNC_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
  row_gather_kernel<<<grid_for(n, 8), 256, 0, s>>>(g, d_err);
  int bits = 0;
  ANNC_TRY(check_err_word(call, d_err, &bits));
  ANNC_TRY(call.finish());
  if (bits & kErrRow) return fail(ANNC_ERR_INVALID_ARGUMENT, "gather index outside the table");
  return ANNC_OK;
}

// KPFusedSparseEmbedding: a tiny stream compaction whose output sizes are data
// dependent.  The ids are mapped on the device (uint64 modulo), the three short
// output lists are assembled on the host exactly as the reference does.
__global__ void sparse_embedding_bucket_kernel(const unsigned long long* fp, long long n,
                                               unsigned long long num_buckets, long long* bucket) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    bucket[i] = (long long)(fp[i] % num_buckets);
}

int annc_KPFusedSparseEmbedding(const annc_tensor* fingerprints, const annc_tensor* empty,
                                int64_t num_buckets, annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(fingerprints && alloc, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(num_buckets >= 1, ANNC_ERR_INVALID_ARGUMENT, "num_buckets must be >= 1");
  Call call;
  cudaStream_t s = call.stream();
  const int64_t n = numel(*fingerprints);
  std::vector<long long> bucket(std::max<int64_t>(n, 1));
  std::vector<unsigned char> emp(std::max<int64_t>(n, 1), 0);
  if (n > 0) {
    const auto* d_fp = (const unsigned long long*)call.in(fingerprints->data, (size_t)n * 8);
    auto* d_b = static_cast<long long*>(call.scratch((size_t)n * 8));
    if (call.status() != ANNC_OK) return call.status();
    sparse_embedding_bucket_kernel<<<grid_for(n, 256), 256, 0, s>>>(d_fp, n, (unsigned long long)num_buckets, d_b);
    ANNC_CUDA(cudaMemcpyAsync(bucket.data(), d_b, (size_t)n * 8, cudaMemcpyDeviceToHost, s));
    ANNC_CUDA(cudaStreamSynchronize(s));
    if (empty && empty->data) ANNC_TRY(call.read_host(empty->data, (size_t)n, emp.data()));
  }
  std::vector<int64_t> indices, values;
  std::vector<unsigned char> empty_out;
  for (int64_t i = 0; i < n; ++i) {
    indices.push_back(i);
    indices.push_back(0);
    if (!emp[i]) {
      if (bucket[i] > 0) {
        values.push_back(bucket[i]);
        empty_out.push_back(0);
      }
    } else {
      values.push_back(0);
      empty_out.push_back(1);
    }
  }
  const int64_t nv = (int64_t)values.size();
  const int64_t d0[2] = {n, 2}, d1[1] = {nv}, d3[1] = {2};
  void* o0 = alloc(ctx, 0, ANNC_I64, 2, d0);
  void* o1 = alloc(ctx, 1, ANNC_I64, 1, d1);
  void* o2 = alloc(ctx, 2, ANNC_BOOL, 1, d1);
  void* o3 = alloc(ctx, 3, ANNC_I64, 1, d3);
  ANNC_REQUIRE(o3 && (o0 || n == 0) && ((o1 && o2) || nv == 0), ANNC_ERR_INTERNAL,
               "output allocation failed");
  const int64_t shape[2] = {n, 1};
  struct Item { void* dst; const void* src; size_t bytes; };
  const Item items[4] = {{o0, indices.data(), (size_t)n * 16}, {o1, values.data(), (size_t)nv * 8},
                         {o2, empty_out.data(), (size_t)nv}, {o3, shape, 16}};
  for (const Item& it : items) {
    if (!it.bytes) continue;
    if (call.is_device(it.dst)) {
      ANNC_CUDA(cudaMemcpyAsync(it.dst, it.src, it.bytes, cudaMemcpyHostToDevice, s));
    } else {
      memcpy(it.dst, it.src, it.bytes);
    }
  }
  ANNC_CUDA(cudaStreamSynchronize(s));
  return call.finish();
}

}  // extern "C"

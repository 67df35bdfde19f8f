// Host side of the row-sharded embedding exchange: the per-rank object that owns the step
// protocol (classify, scan, scatter, flag barrier, pooling + exchange, flag barrier, masked sum)
// behind a C ABI.  The caller supplies the peer-visible buffer of every rank (allocated and
// mapped with annc_peer_buffer_*; the handles travel over any host channel) and, per step, the
// ids and index matrices of its own batch.  A step allocates nothing and makes no host
// synchronisation; ranks are ordered by flags in peer memory with bounded waits.
#include <algorithm>
#include <cstring>
#include <vector>

#include "common.h"
#include "row_exchange_kernels.cuh"

extern "C" int annc_sum_partials_masked_slot_major_dev(const float* src, const uint32_t* mask, int parts,
                                                       int64_t part_stride, int64_t rows, int slots,
                                                       int64_t slot_width, const int32_t* mean_offsets,
                                                       const int32_t* out_slots, void* out,
                                                       int64_t out_stride, int out_bf16, void* stream);
extern "C" size_t annc_embed_bag_workspace_bytes(int num_tables, int64_t batch);
extern "C" int annc_embed_bag_prepass_dev(const annc_bag_table* tables, int num_tables, int64_t ncols,
                                          int32_t col, int64_t batch, void* workspace,
                                          size_t workspace_bytes, void* stream);

namespace annc {
namespace rowx {

static size_t up256(size_t n) { return (n + 255) & ~size_t(255); }

// The peer-visible buffer of a rank.  Lists, bounds and receive slabs exist twice: a rank may
// publish the lists of step i + 1 while its peers still pool step i and while it still adds the
// parts of step i, so consecutive steps alternate between the two sets.
struct Layout {
  size_t flags, bounds, records[2], recv[2], total;
  size_t rec_bytes;    // one source's region of a record buffer
  size_t slab_floats;
};
constexpr int kFlagWordsA = 0;    // barrier "lists published"
constexpr int kFlagWordsB = 16;   // barrier "parts stored"
constexpr int kBoundsInts = 32;   // ints per set of published bounds

static Layout layout_of(int world, int num_tables, int64_t batch, int64_t dim, int64_t max_lookups) {
  Layout l;
  l.flags = 0;
  l.bounds = 256;
  const size_t rec = up256((size_t)std::max<int64_t>(max_lookups, 1) * sizeof(int2));
  l.rec_bytes = rec;
  l.records[0] = 512;
  l.records[1] = l.records[0] + (size_t)world * rec;  // one region per source
  l.slab_floats = (size_t)batch * (size_t)num_tables * (size_t)dim;
  const size_t slabs = up256((size_t)world * l.slab_floats * sizeof(float));
  l.recv[0] = l.records[1] + (size_t)world * rec;
  l.recv[1] = l.recv[0] + slabs;
  l.total = l.recv[1] + slabs;
  return l;
}

struct HotSet {
  unsigned* words = nullptr;
  unsigned* prefix = nullptr;
};

struct Exchange {
  int world = 1, rank = 0, T = 0, id_kind = 2, combiner = 0;
  int64_t dim = 0, batch = 0, max_lookups = 0;
  int blocks_x = 1;
  Layout lay;
  std::vector<char*> peer;  // every rank's buffer as seen from here
  std::vector<annc_row_shard_table> tables;
  std::vector<HotSet> hot;
  // device scratch owned by the object
  unsigned char* owner = nullptr;
  int* local = nullptr;
  int* pos = nullptr;         // counts, then positions: world * T * blocks_x + 1
  int* scan_tiles = nullptr;
  unsigned* mask[2] = {nullptr, nullptr};   // [T * batch], one per step in flight
  int* meta = nullptr;        // (first, count) per source
  int* err = nullptr;
  void* offsets_ws[2] = {nullptr, nullptr};  // bag offsets for mean pooling
  size_t offsets_ws_bytes = 0;
  long long pos_n = 0;
  long long begun = 0, pooled = 0, finished = 0;  // steps that passed each phase
  unsigned long long limit_ns = 2000000000ull;
  int pool_ctas_per_sm = 0;  // 0: as many as fit; -n: n fewer
  int* out_slots = nullptr;  // device i32[T]: output slot of every table
  std::vector<int32_t> out_slots_host;
  bool out_slots_set = false;
  bool profiling = false;
  cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
  bool ev_valid = false;
  PoolParams pool;
  BarrierParams bar;
};

static constexpr int kScanTile = emb::kScanTile;

static void exclusive_scan_inplace(int* data, long long n, int* tile_scratch, cudaStream_t s) {
  const long long tiles = std::max<long long>(1, (n + kScanTile - 1) / kScanTile);
  emb::scan_tile_sums_kernel<<<(unsigned)tiles, emb::kScanThreads, 0, s>>>(data, n, tile_scratch);
  emb::scan_tile_offsets_kernel<<<1, emb::kScanThreads, 0, s>>>(tile_scratch, tiles, tile_scratch + tiles);
  emb::scan_apply_kernel<<<(unsigned)tiles, emb::kScanThreads, 0, s>>>(data, n, tile_scratch, data);
}

template <int LANES, int VPL, int TILES, int INFLIGHT, int MINB>
static void launch_pool(const Exchange& x, cudaStream_t s) {
  static int per_sm[kMaxDevices] = {0};
  const int slot = device_slot();
  if (!per_sm[slot]) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, pool_kernel<LANES, VPL, TILES, INFLIGHT, MINB>, 256, 0) !=
            cudaSuccess || n < 1)
      n = 2;
    per_sm[slot] = n;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, slot);
  const int ctas = x.pool_ctas_per_sm > 0 ? std::min(x.pool_ctas_per_sm, per_sm[slot])
                                          : std::max(1, per_sm[slot] + x.pool_ctas_per_sm);
  pool_kernel<LANES, VPL, TILES, INFLIGHT, MINB><<<(unsigned)(sms * ctas), 256, 0, s>>>(x.pool, x.err);
}

static int run_pool(const Exchange& x, cudaStream_t s) {
  switch ((int)(x.dim / 4)) {
    case 4: launch_pool<4, 1, 8, 4, 5>(x, s); break;
    case 8: launch_pool<8, 1, 8, 4, 5>(x, s); break;
    // dim 64 and 128: half as many lanes per row as 16-byte pieces, two pieces per lane, two row
    // loads in flight (fewer lanes repeat the per-record control instructions: 0.67 ms against
    // 0.76 ms for the 17.9 M lookups of the DLRM batch)
    case 16: launch_pool<8, 2, 16, 2, 5>(x, s); break;
    case 32: launch_pool<16, 2, 8, 2, 5>(x, s); break;
    case 64: launch_pool<32, 2, 8, 4, 4>(x, s); break;
    case 128: launch_pool<32, 4, 8, 2, 3>(x, s); break;
    default: return fail(ANNC_ERR_UNSUPPORTED, "row exchange: dim must be 16, 32, 64, 128, 256 or 512");
  }
  return ANNC_OK;
}

static void destroy(Exchange* x) {
  if (!x) return;
  cudaFree(x->owner);
  cudaFree(x->local);
  cudaFree(x->pos);
  cudaFree(x->scan_tiles);
  cudaFree(x->mask[0]);
  cudaFree(x->mask[1]);
  cudaFree(x->meta);
  cudaFree(x->out_slots);
  cudaFree(x->err);
  cudaFree(x->offsets_ws[0]);
  cudaFree(x->offsets_ws[1]);
  for (auto& h : x->hot) {
    cudaFree(h.words);
    cudaFree(h.prefix);
  }
  for (auto& e : x->ev)
    if (e) cudaEventDestroy(e);
  delete x;
}

}  // namespace rowx
}  // namespace annc

using namespace annc;
using namespace annc::rowx;

extern "C" {

size_t annc_row_exchange_peer_bytes(const annc_row_exchange_config* c) {
  if (!c || c->world < 1 || c->num_tables < 1 || c->batch < 1 || c->dim < 1) return 0;
  return layout_of(c->world, c->num_tables, c->batch, c->dim, c->max_lookups).total;
}

int annc_row_exchange_create(const annc_row_exchange_config* c, void* const* peer_buffers,
                             annc_row_exchange** out) {
  ANNC_REQUIRE(c && peer_buffers && out, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null argument");
  ANNC_REQUIRE(c->world >= 1 && c->world <= kMaxWorld && c->rank >= 0 && c->rank < c->world,
               ANNC_ERR_INVALID_ARGUMENT, "row exchange: world must be 1..16 and rank inside it");
  ANNC_REQUIRE(c->num_tables >= 1 && c->num_tables <= kMaxTables, ANNC_ERR_UNSUPPORTED,
               "row exchange: 1..120 tables");
  ANNC_REQUIRE(c->batch >= 1 && c->max_lookups >= 1 && c->max_lookups_per_table >= 1 && c->tables,
               ANNC_ERR_INVALID_ARGUMENT, "row exchange: bad sizes");
  ANNC_REQUIRE(c->id_kind >= 0 && c->id_kind <= 2 && (c->combiner == 0 || c->combiner == 1),
               ANNC_ERR_INVALID_ARGUMENT, "row exchange: bad id_kind / combiner");
  ANNC_REQUIRE(c->max_lookups < (1LL << 31) - 1 && c->num_tables * c->batch < (1LL << 31) - 1,
               ANNC_ERR_UNSUPPORTED, "row exchange: more than 2^31-2 lookups or bags per step");
  ANNC_REQUIRE(c->dim % 4 == 0 && (double)c->batch * c->num_tables * (c->dim / 4) < 4294967000.0,
               ANNC_ERR_UNSUPPORTED, "row exchange: dim must be a multiple of 4 and one slab below 64 GB");
  switch ((int)(c->dim / 4)) {
    case 4: case 8: case 16: case 32: case 64: case 128: break;
    default: return fail(ANNC_ERR_UNSUPPORTED, "row exchange: dim must be 16, 32, 64, 128, 256 or 512");
  }
  auto* x = new Exchange();
  x->world = c->world;
  x->rank = c->rank;
  x->T = c->num_tables;
  x->id_kind = c->id_kind;
  x->combiner = c->combiner;
  x->dim = c->dim;
  x->batch = c->batch;
  x->max_lookups = c->max_lookups;
  x->blocks_x = (int)((c->max_lookups_per_table + kClassifyItems - 1) / kClassifyItems);
  x->lay = layout_of(c->world, c->num_tables, c->batch, c->dim, c->max_lookups);
  x->tables.assign(c->tables, c->tables + c->num_tables);
  x->hot.resize(c->num_tables);
  for (int q = 0; q < c->world; ++q) {
    if (!peer_buffers[q]) {
      destroy(x);
      return fail(ANNC_ERR_INVALID_ARGUMENT, "row exchange: null peer buffer");
    }
    x->peer.push_back(static_cast<char*>(peer_buffers[q]));
  }
  x->pos_n = (long long)x->world * x->T * x->blocks_x + 1;
  const long long scan_tiles = (x->pos_n + kScanTile - 1) / kScanTile + 2;
  cudaError_t e = cudaSuccess;
  auto alloc = [&](void** p, size_t bytes) {
    if (e == cudaSuccess) e = cudaMalloc(p, std::max<size_t>(bytes, 256));
  };
  alloc((void**)&x->owner, (size_t)c->max_lookups);
  alloc((void**)&x->local, (size_t)c->max_lookups * sizeof(int));
  alloc((void**)&x->pos, (size_t)x->pos_n * sizeof(int));
  alloc((void**)&x->scan_tiles, (size_t)scan_tiles * sizeof(int));
  alloc((void**)&x->mask[0], (size_t)x->T * (size_t)x->batch * sizeof(unsigned));
  alloc((void**)&x->mask[1], (size_t)x->T * (size_t)x->batch * sizeof(unsigned));
  alloc((void**)&x->meta, 2 * kMaxWorld * sizeof(int));
  alloc((void**)&x->out_slots, (size_t)std::max(1, x->T) * sizeof(int));
  alloc((void**)&x->err, 256);
  if (c->combiner == 1) {
    x->offsets_ws_bytes = annc_embed_bag_workspace_bytes(x->T, x->batch);
    alloc(&x->offsets_ws[0], x->offsets_ws_bytes);
    alloc(&x->offsets_ws[1], x->offsets_ws_bytes);
  }
  if (e == cudaSuccess) e = cudaMemset(x->err, 0, 256);
  for (int b = 0; b < 2 && e == cudaSuccess; ++b)
    if (x->offsets_ws[b]) e = cudaMemset(x->offsets_ws[b], 0, 512);  // header: error word, marks
  if (e == cudaSuccess) e = cudaMemset(x->pos, 0, (size_t)x->pos_n * sizeof(int));
  // this rank's flags and bounds start at zero; the caller orders create() on all ranks
  // before the first step (a host barrier), so no peer's flag can be wiped here
  if (e == cudaSuccess) e = cudaMemset(x->peer[x->rank], 0, 512);
  // hot-row sets: bitmap over the table's rows + number of set bits before each word
  for (int t = 0; t < x->T && e == cudaSuccess; ++t) {
    const annc_row_shard_table& tb = x->tables[t];
    const bool bad = tb.rows < 1 || tb.rows >= (1LL << 31) || tb.local_rows < 0 || tb.hot_count < 0 ||
                     tb.hot_count > tb.rows || (tb.local_rows + tb.hot_count > 0 && !tb.shard) ||
                     tb.local_rows + tb.hot_count >= (1LL << 31) ||
                     (reinterpret_cast<uintptr_t>(tb.shard) & 15) != 0;
    if (bad) {
      destroy(x);
      return fail(ANNC_ERR_INVALID_ARGUMENT, "row exchange: bad table description");
    }
    if (tb.hot_count == 0 || (tb.hot_count == tb.rows && !tb.hot_rows)) continue;
    if (!tb.hot_rows) {
      destroy(x);
      return fail(ANNC_ERR_INVALID_ARGUMENT, "row exchange: hot_rows missing");
    }
    const long long nwords = (tb.rows + 31) / 32;
    alloc((void**)&x->hot[t].words, (size_t)nwords * 4);
    alloc((void**)&x->hot[t].prefix, (size_t)(nwords + 1) * 4);
    int* tiles = nullptr;
    alloc((void**)&tiles, (size_t)((nwords + 1 + kScanTile - 1) / kScanTile + 2) * 4);
    if (e != cudaSuccess) break;
    cudaMemsetAsync(x->hot[t].words, 0, (size_t)nwords * 4, nullptr);
    cudaMemsetAsync(x->hot[t].prefix, 0, (size_t)(nwords + 1) * 4, nullptr);
    hot_set_bits_kernel<<<148 * 4, 256>>>(reinterpret_cast<const long long*>(tb.hot_rows), tb.hot_count, tb.rows, x->hot[t].words, x->err);
    hot_popc_kernel<<<148 * 4, 256>>>(x->hot[t].words, nwords, reinterpret_cast<int*>(x->hot[t].prefix));
    exclusive_scan_inplace(reinterpret_cast<int*>(x->hot[t].prefix), nwords + 1, tiles, nullptr);
    e = cudaDeviceSynchronize();
    cudaFree(tiles);
  }
  int bits = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&bits, x->err, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) {
    destroy(x);
    return cuda_fail(e, "row exchange: set-up");
  }
  if (bits) {
    destroy(x);
    return fail(ANNC_ERR_INVALID_ARGUMENT, "row exchange: hot_rows must be strictly ascending rows of the table");
  }
  for (auto& ev : x->ev) cudaEventCreate(&ev);
  // fixed parts of the kernel parameters
  memset(&x->pool, 0, sizeof(x->pool));
  memset(&x->bar, 0, sizeof(x->bar));
  for (int t = 0; t < x->T; ++t) {
    x->pool.tab[t] = x->tables[t].shard;
    x->pool.rows[t] = (int)(x->tables[t].local_rows + x->tables[t].hot_count);
  }
  {  // key / batch by multiplication: exact for every key below 2^31
    int lg = 0;
    while ((1LL << lg) < x->batch) ++lg;
    x->pool.batch_shift = 31 + lg;
    x->pool.batch_magic = ((1ull << x->pool.batch_shift) + (unsigned long long)x->batch - 1) /
                          (unsigned long long)x->batch;
  }
  for (int q = 0; q < x->world; ++q) {
    x->bar.flags[q] = reinterpret_cast<int*>(x->peer[q] + x->lay.flags);
    x->bar.bounds[q] = reinterpret_cast<const int*>(x->peer[q] + x->lay.bounds);
  }
  x->pool.meta = x->meta;
  x->pool.batch = (unsigned)x->batch;
  x->pool.num_tables = x->T;
  x->pool.world = x->world;
  x->pool.rank = x->rank;
  x->pool.rounds = 64;
  x->bar.world = x->world;
  x->bar.rank = x->rank;
  *out = reinterpret_cast<annc_row_exchange*>(x);
  return ANNC_OK;
}

int annc_row_exchange_destroy(annc_row_exchange* ex) {
  destroy(reinterpret_cast<Exchange*>(ex));
  return ANNC_OK;
}

int annc_row_exchange_set_timeout_ms(annc_row_exchange* ex, int64_t ms) {
  ANNC_REQUIRE(ex && ms >= 1, ANNC_ERR_INVALID_ARGUMENT, "row exchange: bad timeout");
  reinterpret_cast<Exchange*>(ex)->limit_ns = (unsigned long long)ms * 1000000ull;
  return ANNC_OK;
}

int annc_row_exchange_set_output_slots(annc_row_exchange* ex, const int32_t* slots, void* stream) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null object");
  if (!slots) {
    x->out_slots_set = false;
    return ANNC_OK;
  }
  for (int t = 0; t < x->T; ++t)
    ANNC_REQUIRE(slots[t] >= 0, ANNC_ERR_INVALID_ARGUMENT, "row exchange: negative output slot");
  // staged through an owned host copy: the caller's array need not outlive the call
  x->out_slots_host.assign(slots, slots + x->T);
  ANNC_CUDA(cudaMemcpyAsync(x->out_slots, x->out_slots_host.data(), sizeof(int32_t) * (size_t)x->T,
                            cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)));
  x->out_slots_set = true;
  return ANNC_OK;
}

int annc_row_exchange_set_pool_ctas_per_sm(annc_row_exchange* ex, int ctas_per_sm) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null object");
  x->pool_ctas_per_sm = ctas_per_sm;
  return ANNC_OK;
}

int annc_row_exchange_set_profiling(annc_row_exchange* ex, int on) {
  ANNC_REQUIRE(ex, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null object");
  reinterpret_cast<Exchange*>(ex)->profiling = on != 0;
  return ANNC_OK;
}

int annc_row_exchange_begin(annc_row_exchange* ex, const annc_bag_table* inputs, int64_t ncols,
                            int32_t col, void* stream) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x && inputs, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null argument");
  ANNC_REQUIRE(x->begun - x->finished <= 1, ANNC_ERR_INVALID_ARGUMENT,
               "row exchange: begin may run at most one step ahead of finish");
  ANNC_REQUIRE(col >= 0 && col < ncols, ANNC_ERR_INVALID_ARGUMENT, "Column index out of range");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int buf = (int)(x->begun & 1);
  ClassifyParams p;
  memset(&p, 0, sizeof(p));
  long long flat = 0;
  for (int t = 0; t < x->T; ++t) {
    const annc_bag_table& in = inputs[t];
    ANNC_REQUIRE(in.nnz >= 0 && (in.nnz == 0 || (in.ids && in.slice_input)), ANNC_ERR_INVALID_ARGUMENT,
                 "row exchange: ids and slice_input are needed for every table");
    ANNC_REQUIRE(in.nnz <= (int64_t)x->blocks_x * kClassifyItems, ANNC_ERR_INVALID_ARGUMENT,
                 "row exchange: a table has more lookups than max_lookups_per_table");
    ClassifyTable& T = p.t[t];
    T.ids = in.ids;
    T.seg = reinterpret_cast<const long long*>(in.slice_input);
    T.num_buckets = (unsigned long long)x->tables[t].rows;
    T.magic = x->id_kind == 2 ? emb::mod_magic(T.num_buckets) : 0;
    T.hot_words = x->hot[t].words;
    T.hot_prefix = x->hot[t].prefix;
    T.nnz = (int)in.nnz;
    T.flat_base = (int)flat;
    T.local_rows = (int)x->tables[t].local_rows;
    T.hot_all = (x->tables[t].hot_count == x->tables[t].rows && !x->tables[t].hot_rows) ? 1 : 0;
    flat += in.nnz;
  }
  ANNC_REQUIRE(flat <= x->max_lookups, ANNC_ERR_INVALID_ARGUMENT,
               "row exchange: more lookups than max_lookups");
  p.ncols = ncols;
  p.batch = x->batch;
  p.num_tables = x->T;
  p.id_kind = x->id_kind;
  p.world = x->world;
  p.rank = x->rank;
  p.col = col;
  p.blocks_x = x->blocks_x;
  char* mine = x->peer[x->rank];
  const bool prof = x->profiling && x->begun == x->finished;  // phase times of steps run one at a time
  if (prof) cudaEventRecord(x->ev[0], s);
  if (x->combiner == 1)  // bag lengths for the mean
    ANNC_TRY(annc_embed_bag_prepass_dev(inputs, x->T, ncols, col, x->batch, x->offsets_ws[buf],
                                        x->offsets_ws_bytes, s));
  ANNC_CUDA(cudaMemsetAsync(x->mask[buf], 0, (size_t)x->T * (size_t)x->batch * sizeof(unsigned), s));
  ANNC_CUDA(cudaMemsetAsync(x->pos + (x->pos_n - 1), 0, sizeof(int), s));  // closing entry
  dim3 grid((unsigned)x->blocks_x, (unsigned)x->T);
  classify_kernel<<<grid, kClassifyThreads, 0, s>>>(p, x->owner, x->local, x->pos, x->err);
  exclusive_scan_inplace(x->pos, x->pos_n, x->scan_tiles, s);
  RecordDest dst;
  for (int g = 0; g < x->world; ++g)
    dst.list[g] = reinterpret_cast<int2*>(x->peer[g] + x->lay.records[buf] + (size_t)x->rank * x->lay.rec_bytes);
  scatter_kernel<<<grid, kClassifyThreads, 0, s>>>(p, x->owner, x->local, x->pos, dst, x->mask[buf], x->err);
  if (prof) cudaEventRecord(x->ev[1], s);
  x->begun += 1;
  arrive_kernel<<<1, 32, 0, s>>>(x->bar, kFlagWordsA, (int)x->begun, x->pos, (long long)x->T * x->blocks_x,
                                 reinterpret_cast<int*>(mine + x->lay.bounds) + buf * kBoundsInts);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_row_exchange_pool(annc_row_exchange* ex, void* stream) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null object");
  ANNC_REQUIRE(x->begun > x->pooled && x->pooled == x->finished, ANNC_ERR_INVALID_ARGUMENT,
               "row exchange: pool needs a begin before it and the previous step finished");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int buf = (int)(x->pooled & 1);
  const bool prof = x->profiling && x->begun == x->pooled + 1;
  wait_kernel<<<1, 32, 0, s>>>(x->bar, kFlagWordsA, (int)(x->pooled + 1), x->limit_ns, x->meta,
                               buf * kBoundsInts, (int)x->max_lookups, x->err);
  if (prof) cudaEventRecord(x->ev[2], s);
  for (int q = 0; q < x->world; ++q) {
    x->pool.list[q] = reinterpret_cast<const int2*>(x->peer[x->rank] + x->lay.records[buf] + (size_t)q * x->lay.rec_bytes);
    x->pool.out[q] = reinterpret_cast<float*>(x->peer[q] + x->lay.recv[buf]) + (size_t)x->rank * x->lay.slab_floats;
  }
  ANNC_TRY(run_pool(*x, s));
  if (prof) cudaEventRecord(x->ev[3], s);
  x->pooled += 1;
  arrive_kernel<<<1, 32, 0, s>>>(x->bar, kFlagWordsB, (int)x->pooled, nullptr, 0, nullptr);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_row_exchange_finish(annc_row_exchange* ex, void* out, int64_t out_stride, int out_bf16,
                             void* stream) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x && out, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null argument");
  ANNC_REQUIRE(x->pooled > x->finished, ANNC_ERR_INVALID_ARGUMENT, "row exchange: finish needs a pool before it");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int buf = (int)(x->finished & 1);
  const bool prof = x->profiling && x->begun == x->finished + 1;
  wait_kernel<<<1, 32, 0, s>>>(x->bar, kFlagWordsB, (int)(x->finished + 1), x->limit_ns, nullptr, 0, 0, x->err);
  if (prof) cudaEventRecord(x->ev[4], s);
  const float* recv = reinterpret_cast<const float*>(x->peer[x->rank] + x->lay.recv[buf]);
  const int32_t* mean_off = x->combiner == 1
                                ? reinterpret_cast<const int32_t*>(static_cast<char*>(x->offsets_ws[buf]) + 512)  // header of the bag workspace
                                : nullptr;
  x->finished += 1;
  ANNC_TRY(annc_sum_partials_masked_slot_major_dev(recv, x->mask[buf], x->world, (int64_t)x->lay.slab_floats,
                                                   x->batch, x->T, x->dim, mean_off,
                                                   x->out_slots_set ? x->out_slots : nullptr, out, out_stride,
                                                   out_bf16, s));
  if (prof) {
    cudaEventRecord(x->ev[5], s);
    x->ev_valid = true;
  }
  return ANNC_OK;
}

int annc_row_exchange_step(annc_row_exchange* ex, const annc_bag_table* inputs, int64_t ncols,
                           int32_t col, void* out, int64_t out_stride, int out_bf16, void* stream) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null object");
  if (x->begun == x->finished) ANNC_TRY(annc_row_exchange_begin(ex, inputs, ncols, col, stream));
  ANNC_TRY(annc_row_exchange_pool(ex, stream));
  return annc_row_exchange_finish(ex, out, out_stride, out_bf16, stream);
}

int annc_row_exchange_check(annc_row_exchange* ex, void* stream, int* error_bits) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x && error_bits, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ANNC_CUDA(cudaMemcpyAsync(error_bits, x->err, sizeof(int), cudaMemcpyDeviceToHost, s));
  ANNC_CUDA(cudaStreamSynchronize(s));
  if (x->combiner == 1) {  // segment errors seen by the prepass
    for (int b = 0; b < 2; ++b) {
      int pre = 0;
      ANNC_CUDA(cudaMemcpy(&pre, x->offsets_ws[b], sizeof(int), cudaMemcpyDeviceToHost));
      *error_bits |= pre & (kErrRow | kErrSegment);
    }
  }
  if (*error_bits & kErrTimeout)
    return fail(ANNC_ERR_TIMEOUT, "row exchange: a peer's flag did not arrive within the limit");
  return ANNC_OK;
}

int annc_row_exchange_clear_errors(annc_row_exchange* ex, void* stream) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null object");
  ANNC_CUDA(cudaMemsetAsync(x->err, 0, sizeof(int), static_cast<cudaStream_t>(stream)));
  return ANNC_OK;
}

int annc_row_exchange_phase_ms(annc_row_exchange* ex, float* ms5) {
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x && ms5, ANNC_ERR_INVALID_ARGUMENT, "row exchange: null argument");
  ANNC_REQUIRE(x->ev_valid, ANNC_ERR_INVALID_ARGUMENT, "row exchange: no profiled step yet");
  ANNC_CUDA(cudaEventSynchronize(x->ev[5]));
  for (int i = 0; i < 5; ++i) ANNC_CUDA(cudaEventElapsedTime(&ms5[i], x->ev[i], x->ev[i + 1]));
  return ANNC_OK;
}

int annc_row_exchange_stats(annc_row_exchange* ex, void* stream, int64_t* records_per_source,
                            int64_t* parts_per_owner) {
  // Debug / reporting aid: the sizes of the lists this rank pooled in the last step, and the
  // number of bags of its own batch every owner sent a part for (from the owner masks).
  auto* x = reinterpret_cast<Exchange*>(ex);
  ANNC_REQUIRE(x && records_per_source && parts_per_owner, ANNC_ERR_INVALID_ARGUMENT,
               "row exchange: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int meta[2 * kMaxWorld];
  ANNC_CUDA(cudaMemcpyAsync(meta, x->meta, sizeof(meta), cudaMemcpyDeviceToHost, s));
  std::vector<unsigned> mask((size_t)x->T * (size_t)x->batch);
  const int last = (int)((x->finished + 1) & 1);  // buffer of the last finished step
  ANNC_CUDA(cudaMemcpyAsync(mask.data(), x->mask[last], mask.size() * 4, cudaMemcpyDeviceToHost, s));
  ANNC_CUDA(cudaStreamSynchronize(s));
  for (int q = 0; q < x->world; ++q) {
    records_per_source[q] = meta[2 * q + 1];
    parts_per_owner[q] = 0;
  }
  for (unsigned m : mask)
    for (int q = 0; q < x->world; ++q) parts_per_owner[q] += (m >> q) & 1u;
  return ANNC_OK;
}

}  // extern "C"

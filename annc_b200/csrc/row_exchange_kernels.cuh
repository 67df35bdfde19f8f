// Device kernels of the row-sharded embedding exchange (one process per GPU of one node).
//
// Tables are split over `world` ranks with the reference's mod rule (owner = row % world,
// local row = row / world; annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc
// :70-71).  A rank may also hold a replicated set of hot rows per table; a lookup of a hot
// row is pooled by the rank that owns the sample and never crosses NVLink.
//
// One step on rank r:
//   classify   every lookup of r's batch -> (owner, local row); per-block counts per owner
//   scan       exclusive prefix of the counts: one contiguous record list per owner
//   scatter    records (row, bag key) written to the owner's list, lookup order kept;
//              per-bag mask of the owners that will send a part
//   arrive     list bounds published, flag stored into every peer's memory
//   wait       bounded spin on this rank's own flags; the bounds of the lists meant for r
//   pool       lookup-granular segmented reduce over the records of every source (read through
//              peer-mapped pointers), each finished partial sum stored straight into the
//              source rank's receive slab: pooling and exchange are one kernel
//   arrive / wait
//   (the masked sum of the parts is annc_sum_partials_masked_dev's kernel)
// No multicast object, no TMA: plain loads and stores through peer-mapped pointers.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "emb_device.cuh"

namespace annc {
namespace rowx {

constexpr int kMaxTables = 120;
constexpr int kMaxWorld = 16;
constexpr int kErrRow = 1;        // row outside its table (same bits as the bag kernels)
constexpr int kErrSegment = 2;    // segment id outside [0, batch)
constexpr int kErrUnsorted = 4;   // segment ids decrease: the exchange needs sorted bags
constexpr int kErrTimeout = 8;    // a peer's flag did not arrive within the limit
constexpr int kErrBounds = 16;    // a peer published list bounds outside its record buffer

constexpr int kClassifyThreads = 256;
constexpr int kClassifyTiles = 4;
constexpr int kClassifyItems = kClassifyThreads * kClassifyTiles;  // lookups per block

struct ClassifyTable {
  const void* ids;               // [nnz] u64 fingerprints (id_kind 2) or i32/i64 rows
  const long long* seg;          // slice_input i64[nnz, ncols]
  unsigned long long num_buckets;
  unsigned long long magic;
  const unsigned* hot_words;     // bitmap over the table's rows (null: no hot rows)
  const unsigned* hot_prefix;    // set bits before each word
  int nnz;
  int flat_base;                 // index of this table's first lookup in the flat arrays
  int local_rows;                // rows of this rank's shard; hot row h sits at local_rows + h
  int hot_all;                   // every row is replicated (hot index = row)
};
static_assert(sizeof(ClassifyTable) == 64, "parameter space is budgeted on 64-byte entries");

struct ClassifyParams {
  ClassifyTable t[kMaxTables];
  long long ncols;
  long long batch;
  int num_tables;
  int id_kind;
  int world;
  int rank;
  int col;
  int blocks_x;  // blocks per table
};

__device__ __forceinline__ long long raw_row(const void* ids, int id_kind, long long i,
                                             unsigned long long nb, unsigned long long magic) {
  return emb::load_row_id(ids, id_kind, i, nb, magic);
}

// Pass 1.  Block (x, t) looks at lookups [x * 1024, x * 1024 + 1024) of table t, writes the
// owner (u8) and local row (i32) of each and counts[(g * T + t) * blocks_x + x] per owner g.
__global__ void __launch_bounds__(kClassifyThreads)
classify_kernel(ClassifyParams p, unsigned char* __restrict__ owner_out, int* __restrict__ local_out,
                int* __restrict__ counts, int* __restrict__ err) {
  __shared__ int wcnt[kClassifyThreads / 32][kMaxWorld];
  const int t = blockIdx.y;
  const ClassifyTable& T = p.t[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int first = blockIdx.x * kClassifyItems;  // a block past the table's end writes zero counts
  int my_count = 0;  // lane g < world: lookups of owner g seen by this warp
  for (int j = 0; j < kClassifyTiles; ++j) {
    const int i = first + j * kClassifyThreads + threadIdx.x;
    int owner = -1, local = -1;
    if (i < T.nnz) {
      const long long r = raw_row(T.ids, p.id_kind, i, T.num_buckets, T.magic);
      if (r < 0 || r > 0x7fffffffLL) {
        atomicOr(err, kErrRow);  // no table has such a row: pooled by nobody
        owner = p.rank;
        local = -1;
      } else {
        const unsigned b = (unsigned)r;
        int hot = -1;
        if (T.hot_all) {
          hot = (int)b;
        } else if (T.hot_words) {
          const unsigned w = __ldg(T.hot_words + (b >> 5));
          if ((w >> (b & 31)) & 1u) hot = (int)(__ldg(T.hot_prefix + (b >> 5)) + __popc(w & ((1u << (b & 31)) - 1u)));
        }
        if (hot >= 0) {
          owner = p.rank;
          local = T.local_rows + hot;
        } else {
          const unsigned q = b / (unsigned)p.world;
          owner = (int)(b - q * (unsigned)p.world);
          local = (int)q;
        }
      }
      owner_out[T.flat_base + i] = (unsigned char)owner;
      local_out[T.flat_base + i] = local;
    }
    for (int g = 0; g < p.world; ++g) {
      const unsigned m = __ballot_sync(0xffffffffu, owner == g);
      if (lane == g) my_count += __popc(m);
    }
  }
  if (lane < kMaxWorld) wcnt[warp][lane] = my_count;
  __syncthreads();
  if (threadIdx.x < p.world) {
    int s = 0;
    for (int w = 0; w < kClassifyThreads / 32; ++w) s += wcnt[w][threadIdx.x];
    counts[((long long)threadIdx.x * p.num_tables + t) * p.blocks_x + blockIdx.x] = s;
  }
}

// Pass 2.  Same geometry; pos = exclusive scan of counts.  Writes record (local row, key) with
// key = t * batch + segment id at the lookup's place in its owner's list (lookup order is kept
// inside a list, so a bag's records are adjacent), ORs the owner into mask[key], and checks
// that segment ids are in range and do not decrease.
__global__ void __launch_bounds__(kClassifyThreads)
scatter_kernel(ClassifyParams p, const unsigned char* __restrict__ owner_in,
               const int* __restrict__ local_in, const int* __restrict__ pos,
               int2* __restrict__ records, unsigned* __restrict__ mask, int* __restrict__ err) {
  constexpr int kWarps = kClassifyThreads / 32;
  __shared__ int wcnt[kClassifyTiles * kWarps][kMaxWorld];
  const int t = blockIdx.y;
  const ClassifyTable& T = p.t[t];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int first = blockIdx.x * kClassifyItems;
  if (first >= T.nnz) return;
  int owner[kClassifyTiles], local[kClassifyTiles], key[kClassifyTiles], rank_in_warp[kClassifyTiles];
#pragma unroll
  for (int j = 0; j < kClassifyTiles; ++j) {
    const int i = first + j * kClassifyThreads + threadIdx.x;
    owner[j] = -1;
    local[j] = -1;
    key[j] = -1;
    long long seg = -1;
    if (i < T.nnz) {
      owner[j] = owner_in[T.flat_base + i];
      local[j] = local_in[T.flat_base + i];
      seg = T.seg[(long long)i * p.ncols + p.col];
      if (seg < 0 || seg >= p.batch) {
        atomicOr(err, kErrSegment);
      } else {
        key[j] = (int)((long long)t * p.batch + seg);
      }
    }
    // sortedness: compare with the previous lookup of the table
    long long prev = __shfl_up_sync(0xffffffffu, seg, 1);
    if (lane == 0) prev = (i > 0 && i < T.nnz) ? T.seg[(long long)(i - 1) * p.ncols + p.col] : -1;
    if (i < T.nnz && i > 0 && seg < prev) atomicOr(err, kErrUnsorted);
    int r = 0, cnt = 0;
    for (int g = 0; g < p.world; ++g) {
      const unsigned m = __ballot_sync(0xffffffffu, owner[j] == g);
      if (owner[j] == g) r = __popc(m & ((1u << lane) - 1u));
      if (lane == g) cnt = __popc(m);
    }
    rank_in_warp[j] = r;
    if (lane < kMaxWorld) wcnt[j * kWarps + warp][lane] = cnt;
    // one atomicOr per (bag, warp): the lanes that hold the same key combine their owner bits
    if (key[j] >= 0) {
      const unsigned peers = __match_any_sync(__activemask(), key[j]);
      const unsigned bits = __reduce_or_sync(peers, 1u << owner[j]);
      if ((int)(__ffs(peers) - 1) == lane) atomicOr(mask + key[j], bits);
    }
  }
  __syncthreads();
  if (threadIdx.x < p.world) {  // exclusive prefix over (tile, warp) in lookup order
    int run = pos[((long long)threadIdx.x * p.num_tables + t) * p.blocks_x + blockIdx.x];
    for (int e = 0; e < kClassifyTiles * kWarps; ++e) {
      const int c = wcnt[e][threadIdx.x];
      wcnt[e][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < kClassifyTiles; ++j) {
    if (owner[j] >= 0)
      records[wcnt[j * kWarps + warp][owner[j]] + rank_in_warp[j]] = make_int2(local[j], key[j]);
  }
}

// ---- flag barrier between the ranks ---------------------------------------------------
// Every rank owns flags[kMaxWorld] in its peer-visible buffer; flags[q] is written by rank q
// only and only grows (the step's epoch).  arrive: publishes this rank's list bounds, then
// stores the epoch into flags[rank] of every rank.  wait: spins on the own flags until all
// have reached the epoch, for at most `limit_ns`; a time-out sets kErrTimeout and returns.
struct BarrierParams {
  int* flags[kMaxWorld];         // rank q's flag array as seen from here ([rank] is local)
  const int* bounds[kMaxWorld];  // rank q's published list bounds int[world + 1]
  int world;
  int rank;
};

__global__ void arrive_kernel(BarrierParams b, int epoch, const int* __restrict__ pos,
                              long long pos_stride, int* __restrict__ my_bounds) {
  const int lane = threadIdx.x;
  if (pos && lane <= b.world) my_bounds[lane] = pos[(long long)lane * pos_stride];
  __threadfence_system();
  __syncwarp();
  if (lane < b.world) {
    volatile int* f = b.flags[lane] + b.rank;
    *f = epoch;
  }
}

// meta[2 q] = first record, meta[2 q + 1] = number of records of source q's list for this rank
// (zero when the source timed out or published bounds outside [0, capacity]).
__global__ void wait_kernel(BarrierParams b, int epoch, unsigned long long limit_ns,
                            int* __restrict__ meta, int capacity, int* __restrict__ err) {
  const int lane = threadIdx.x;
  bool ok = true;
  if (lane < b.world) {
    volatile const int* f = b.flags[b.rank] + lane;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    while (*f < epoch) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - t0 > limit_ns) {
        atomicOr(err, kErrTimeout);
        ok = false;
        break;
      }
      __nanosleep(200);
    }
  }
  __threadfence_system();
  __syncwarp();
  if (meta && lane < b.world) {
    int lo = 0, n = 0;
    if (ok) {
      volatile const int* bd = b.bounds[lane];
      lo = bd[b.rank];
      const int hi = bd[b.rank + 1];
      n = hi - lo;
      if (lo < 0 || n < 0 || hi > capacity) {
        atomicOr(err, kErrBounds);
        lo = 0;
        n = 0;
      }
    }
    meta[2 * lane] = lo;
    meta[2 * lane + 1] = n;
  }
}

// ---- pooling + exchange ----------------------------------------------------------------
// Lookup-granular: a group of LANES lanes takes CHUNK = LANES consecutive records of one
// source's list (one record per lane, one coalesced load) and owns the bags whose first record
// lies in that chunk; it follows its last bag into the next chunks until the key changes.  Rows
// are added in record order (= lookup order) into a zero accumulator, eight row loads in flight
// per group, and each finished partial sum is stored at once into the receive slab of the rank
// that owns the sample.  A chunk of 16 records keeps every lane busy whatever the bag lengths
// (1.3 lookups per (bag, owner) pair at eight ranks).
struct PoolParams {
  const float* tab[kMaxTables];   // this rank's shard of table t
  const float* hot[kMaxTables];   // replicated hot rows of table t (local row >= rows[t])
  int rows[kMaxTables];
  int hot_rows[kMaxTables];
  const int2* list[kMaxWorld];    // source q's record buffer as seen from here
  float* out[kMaxWorld];          // this rank's slab in source q's receive buffer
  const int* meta;                // (first, count) per source, written by wait_kernel
  unsigned batch;
  int num_tables;
  int world;
  int rank;
  int rounds;                     // interleave factor of the sources
};

template <int LANES, int VPL>
__global__ void __launch_bounds__(256)
pool_kernel(PoolParams p, int* __restrict__ err) {
  constexpr int GROUPS_PER_WARP = 32 / LANES;
  constexpr int CHUNK = LANES;
  constexpr int INFLIGHT = LANES < 8 ? LANES : 8;
  constexpr int ROW4 = LANES * VPL;  // float4 per row
  __shared__ int s_first[kMaxWorld], s_chunks[kMaxWorld], s_quota[kMaxWorld], s_qpre[kMaxWorld + 1];
  if (threadIdx.x == 0) {
    // sources in the order rank+1, rank+2, ..., rank: at any moment the ranks of a node store
    // towards different destinations
    int pre = 0;
    for (int j = 0; j < p.world; ++j) {
      const int q = (p.rank + 1 + j) % p.world;
      const int n = p.meta[2 * q + 1];
      const int chunks = (n + CHUNK - 1) / CHUNK;
      s_first[j] = p.meta[2 * q];
      s_chunks[j] = chunks;
      s_quota[j] = (chunks + p.rounds - 1) / p.rounds;
      s_qpre[j] = pre;
      pre += s_quota[j];
    }
    s_qpre[p.world] = pre;
  }
  __syncthreads();
  const int per_round = s_qpre[p.world];
  if (per_round == 0) return;
  const int lane_in_warp = threadIdx.x & 31;
  const int lane = lane_in_warp % LANES;
  const int shift = (lane_in_warp / LANES) * LANES;
  const unsigned gmask = (LANES == 32) ? 0xffffffffu : (((1u << LANES) - 1u) << shift);
  const long long group = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * GROUPS_PER_WARP +
                          lane_in_warp / LANES;
  const long long num_groups = (long long)gridDim.x * (blockDim.x >> 5) * GROUPS_PER_WARP;
  const long long virtual_chunks = (long long)per_round * p.rounds;
  const unsigned T = (unsigned)p.num_tables;

  for (long long vc = group; vc < virtual_chunks; vc += num_groups) {
    const int round = (int)(vc / per_round);
    const int rem = (int)(vc - (long long)round * per_round);
    int j = 0;
    while (rem >= s_qpre[j + 1]) ++j;
    const int chunk = round * s_quota[j] + (rem - s_qpre[j]);
    if (chunk >= s_chunks[j] || rem - s_qpre[j] >= s_quota[j]) continue;
    const int q = (p.rank + 1 + j) % p.world;
    const int2* __restrict__ rec = p.list[q] + s_first[j];
    const int n = p.meta[2 * q + 1];
    float4* __restrict__ out = reinterpret_cast<float4*>(p.out[q]);

    float4 acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    unsigned cur = 0xffffffffu;  // output slot (in float4 rows) of the bag being summed
    bool open = false;           // a bag of this group is being summed
    int base = chunk * CHUNK;
    bool first_tile = true;
    while (base < n) {
      // one record per lane; slot = where its bag's partial sum goes, tsel = table (+ hot flag)
      int2 r = make_int2(-1, -1);
      if (base + lane < n) r = __ldg(rec + base + lane);
      int prev_key = __shfl_up_sync(gmask, r.y, 1, LANES);
      if (lane == 0) prev_key = base > 0 ? __ldg(rec + base - 1).y : -2;
      unsigned slot = 0xfffffffeu;  // a record without a valid key is added nowhere
      int tsel = -1, row = -1;
      if (r.y >= 0) {
        const unsigned t = (unsigned)r.y / p.batch;
        const unsigned s = (unsigned)r.y - t * p.batch;
        slot = (s * T + t) * (unsigned)ROW4;
        if (t < T) {
          if (r.x >= 0 && r.x < p.rows[t]) {
            tsel = (int)t;
            row = r.x;
          } else if (r.x >= p.rows[t] && r.x - p.rows[t] < p.hot_rows[t]) {
            tsel = (int)t | 0x100;
            row = r.x - p.rows[t];
          } else {
            atomicOr(err, kErrRow);
          }
        }
      }
      const bool starts = (base + lane < n) && (r.y != prev_key);
      const unsigned smask = (__ballot_sync(gmask, starts) >> shift) & (LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u));
      int from = 0, to = min(CHUNK, n - base);
      if (first_tile) {
        // bags that began in an earlier chunk belong to the group of that chunk
        if (smask == 0) break;
        from = __ffs(smask) - 1;
        first_tile = false;
      } else {
        // a following tile: only the rest of the bag that is still open
        if (smask != 0) to = __ffs(smask) - 1;
      }
      for (int j0 = from; j0 < to; j0 += INFLIGHT) {
        unsigned sl[INFLIGHT];
        float4 v[INFLIGHT][VPL];
        bool has[INFLIGHT];
#pragma unroll
        for (int k = 0; k < INFLIGHT; ++k) {
          const int src_lane = (j0 + k) % LANES;
          sl[k] = __shfl_sync(gmask, slot, src_lane, LANES);
          const int ts = __shfl_sync(gmask, tsel, src_lane, LANES);
          const int rw = __shfl_sync(gmask, row, src_lane, LANES);
          has[k] = (j0 + k < to) && ts >= 0;
          if (j0 + k >= to) sl[k] = 0xffffffffu;
          if (has[k]) {
            const float* src = ((ts & 0x100) ? p.hot[ts & 0xff] : p.tab[ts]) + (long long)rw * (ROW4 * 4);
#pragma unroll
            for (int w = 0; w < VPL; ++w) v[k][w] = emb::ldg4(src + (w * LANES + lane) * 4);
          }
        }
#pragma unroll
        for (int k = 0; k < INFLIGHT; ++k) {
          if (sl[k] == 0xffffffffu) continue;  // past the end of this tile's share
          if (sl[k] != cur) {
            if (open && cur < 0xfffffffeu) {
#pragma unroll
              for (int w = 0; w < VPL; ++w) out[cur + w * LANES + lane] = acc[w];
            }
#pragma unroll
            for (int w = 0; w < VPL; ++w) acc[w] = make_float4(0.f, 0.f, 0.f, 0.f);
            cur = sl[k];
            open = true;
          }
          if (has[k]) {
#pragma unroll
            for (int w = 0; w < VPL; ++w) emb::add4(acc[w], v[k][w]);
          }
        }
      }
      if (to < min(CHUNK, n - base)) break;  // the open bag ended inside this tile
      base += CHUNK;
      // the next tile is only needed while the last bag may continue
      if (base >= n) break;
    }
    if (open && cur < 0xfffffffeu) {
#pragma unroll
      for (int w = 0; w < VPL; ++w) out[cur + w * LANES + lane] = acc[w];
    }
  }
}

// ---- hot-row set: bitmap + rank directory ------------------------------------------------
__global__ void hot_set_bits_kernel(const long long* __restrict__ hot_rows, long long n, long long rows,
                                    unsigned* __restrict__ words, int* __restrict__ err) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long r = hot_rows[i];
    if (r < 0 || r >= rows || (i > 0 && hot_rows[i - 1] >= r)) {
      atomicOr(err, kErrRow);  // the list must be strictly ascending rows of the table
      continue;
    }
    atomicOr(words + (r >> 5), 1u << (r & 31));
  }
}

__global__ void hot_popc_kernel(const unsigned* __restrict__ words, long long nwords, int* __restrict__ cnt) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nwords; i += stride)
    cnt[i] = __popc(words[i]);
}

}  // namespace rowx
}  // namespace annc

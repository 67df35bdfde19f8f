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
//   scatter    records (row, bag key) written to the owner's list IN THE OWNER'S MEMORY (r's
//              region of its record buffer), lookup order kept; per-bag mask of the owners
//              that will send a part
//   arrive     list lengths published, flag stored into every peer's memory
//   wait       bounded spin on this rank's own flags; the lengths of the lists meant for r
//   pool       lookup-granular segmented reduce over the records of every source (local
//              reads), each finished partial sum stored straight into the source rank's
//              receive slab: pooling and exchange are one kernel
//   arrive / wait
//   (the masked sum of the parts is annc_sum_partials_masked_slot_major_dev's kernel)
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
// that segment ids are in range and do not decrease.  The list for owner g is written straight
// into g's memory (dst.list[g]: this rank's region of g's record buffer), so the pooling kernel
// reads its lists locally: a list read over NVLink put the link's latency into every tile of
// eight records (0.14 ms of a 0.8 ms kernel on four GPUs).
struct RecordDest {
  int2* list[kMaxWorld];
};

__global__ void __launch_bounds__(kClassifyThreads)
scatter_kernel(ClassifyParams p, const unsigned char* __restrict__ owner_in,
               const int* __restrict__ local_in, const int* __restrict__ pos,
               RecordDest dst, unsigned* __restrict__ mask, int* __restrict__ err) {
  constexpr int kWarps = kClassifyThreads / 32;
  __shared__ int wcnt[kClassifyTiles * kWarps][kMaxWorld];
  __shared__ int blk_base[kMaxWorld];       // the block's first place in every owner's list
  __shared__ int seg_start[kMaxWorld + 1];  // where each owner's records start in `stage`
  __shared__ int2 stage[kClassifyItems];    // the block's records, grouped by owner, in list order
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
    // the run of adjacent lanes that hold this lane's key (a bag's lookups are adjacent)
    const int prev_key = __shfl_up_sync(0xffffffffu, key[j], 1);
    const bool head = lane == 0 || key[j] != prev_key;
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    const unsigned le = (2u << lane) - 1u;  // lanes 0..lane
    const int run_start = 31 - __clz(heads & le);
    const unsigned above = heads & ~le;
    const unsigned run = (above ? (1u << (__ffs(above) - 1)) - 1u : 0xffffffffu) & ~((1u << run_start) - 1u);
    int r = 0, cnt = 0;
    unsigned bits = 0;
    for (int g = 0; g < p.world; ++g) {
      const unsigned m = __ballot_sync(0xffffffffu, owner[j] == g);
      if (owner[j] == g) r = __popc(m & ((1u << lane) - 1u));
      if (lane == g) cnt = __popc(m);
      if (m & run) bits |= 1u << g;
    }
    rank_in_warp[j] = r;
    if (lane < kMaxWorld) wcnt[j * kWarps + warp][lane] = cnt;
    // one atomicOr per (bag, warp), by the first lane of the run, with the owners of the run
    if (head && key[j] >= 0) atomicOr(mask + key[j], bits);
  }
  __syncthreads();
  if (threadIdx.x < p.world) {  // exclusive prefix over (tile, warp) in lookup order
    // position inside the owner's list: the scan runs over all owners' counts
    const long long g0 = (long long)threadIdx.x * p.num_tables * p.blocks_x;
    blk_base[threadIdx.x] = pos[g0 + (long long)t * p.blocks_x + blockIdx.x] - pos[g0];
    int run = 0;  // place inside the block's records for this owner
    for (int e = 0; e < kClassifyTiles * kWarps; ++e) {
      const int c = wcnt[e][threadIdx.x];
      wcnt[e][threadIdx.x] = run;
      run += c;
    }
    seg_start[threadIdx.x + 1] = run;  // count, turned into a prefix below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    seg_start[0] = 0;
    for (int g = 0; g < p.world; ++g) seg_start[g + 1] += seg_start[g];
  }
  __syncthreads();
  // The records are grouped by owner in shared memory first and leave the block as one run of
  // consecutive 8-byte stores per owner: written one by one they were isolated 8-byte stores
  // into seven peers' memory (a third of the split's time on eight GPUs).
#pragma unroll
  for (int j = 0; j < kClassifyTiles; ++j) {
    if (owner[j] >= 0)
      stage[seg_start[owner[j]] + wcnt[j * kWarps + warp][owner[j]] + rank_in_warp[j]] = make_int2(local[j], key[j]);
  }
  __syncthreads();
  const int total = seg_start[p.world];
  for (int i = threadIdx.x; i < total; i += kClassifyThreads) {
    int g = 0;
    while (i >= seg_start[g + 1]) ++g;
    dst.list[g][blk_base[g] + (i - seg_start[g])] = stage[i];
  }
}

// ---- flag barrier between the ranks ---------------------------------------------------
// Every rank owns two sets of flag words in its peer-visible buffer (one per barrier of a
// step: "lists published" and "parts stored"); word q of a set is written by rank q only and
// only grows (the step number).  arrive: publishes this rank's list bounds, then stores the
// epoch into its word of every rank's set.  wait: spins on the own set until all words have
// reached the epoch, for at most `limit_ns`; a time-out sets kErrTimeout and returns.
struct BarrierParams {
  int* flags[kMaxWorld];         // rank q's flag array as seen from here ([rank] is local)
  const int* bounds[kMaxWorld];  // rank q's published list bounds int[world + 1]
  int world;
  int rank;
};

__global__ void arrive_kernel(BarrierParams b, int word0, int epoch, const int* __restrict__ pos,
                              long long pos_stride, int* __restrict__ my_bounds) {
  const int lane = threadIdx.x;
  if (pos && lane <= b.world) my_bounds[lane] = pos[(long long)lane * pos_stride];
  __threadfence_system();
  __syncwarp();
  if (lane < b.world) {
    volatile int* f = b.flags[lane] + word0 + b.rank;
    *f = epoch;
  }
}

// meta[2 q] = first record (always 0), meta[2 q + 1] = number of records of source q's list for
// this rank (zero when the source timed out or published bounds outside [0, capacity]).  word0 selects the
// barrier's flag words, bounds_off the set of published bounds (steps alternate between two).
__global__ void wait_kernel(BarrierParams b, int word0, int epoch, unsigned long long limit_ns,
                            int* __restrict__ meta, int bounds_off, int capacity, int* __restrict__ err) {
  const int lane = threadIdx.x;
  bool ok = true;
  if (lane < b.world) {
    volatile const int* f = b.flags[b.rank] + word0 + lane;
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
      volatile const int* bd = b.bounds[lane] + bounds_off;
      lo = bd[b.rank];
      const int hi = bd[b.rank + 1];
      n = hi - lo;
      if (lo < 0 || n < 0 || hi > capacity) {
        atomicOr(err, kErrBounds);
        lo = 0;
        n = 0;
      }
    }
    meta[2 * lane] = 0;  // every source's list starts at the head of its region of this rank's buffer
    meta[2 * lane + 1] = n;
  }
}

// ---- pooling + exchange ----------------------------------------------------------------
// Lookup-granular: a group of LANES lanes takes a chunk of TILES * LANES consecutive records
// of one source's list (read tile by tile: one record per lane, one coalesced load) and owns
// the bags whose first record lies in that chunk; it follows its last bag past the chunk until
// the key changes.  Rows are added in record order (= lookup order) into a zero accumulator,
// several row loads in flight per group, and each finished partial sum is stored at once into
// the receive slab of the rank that owns the sample.  Work per group does not depend on the
// bag lengths (1.3 lookups per (bag, owner) pair at eight ranks).
struct PoolParams {
  const float* tab[kMaxTables];   // table t on this rank: its shard's rows, then the hot rows
  int rows[kMaxTables];           // rows held (shard + hot)
  const int2* list[kMaxWorld];    // source q's list for this rank (in this rank's memory)
  float* out[kMaxWorld];          // this rank's slab in source q's receive buffer
  const int* meta;                // (first, count) per source, written by wait_kernel
  unsigned long long batch_magic; // key / batch = (key * batch_magic) >> batch_shift for key < 2^31
  unsigned batch;
  int batch_shift;
  int num_tables;
  int world;
  int rank;
  int rounds;                     // interleave factor of the sources
};

template <int LANES, int VPL, int TILES, int INFLIGHT_, int MINB>
__global__ void __launch_bounds__(256, MINB)
pool_kernel(PoolParams p, int* __restrict__ err) {
  constexpr int GROUPS_PER_WARP = 32 / LANES;
  constexpr int CHUNK = LANES * TILES;  // records per group: TILES tiles of one record per lane
  constexpr int INFLIGHT = LANES < INFLIGHT_ ? LANES : INFLIGHT_;
  constexpr int ROW4 = LANES * VPL;  // float4 per row
  constexpr unsigned kLaneMask = LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u);
  constexpr unsigned kNoSlot = 0xfffffffeu;  // a record without a valid key is added nowhere
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
  const unsigned per_round = (unsigned)s_qpre[p.world];
  if (per_round == 0) return;
  const int lane_in_warp = threadIdx.x & 31;
  const int lane = lane_in_warp % LANES;
  const int shift = (lane_in_warp / LANES) * LANES;
  const unsigned gmask = kLaneMask << shift;
  const unsigned group = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * GROUPS_PER_WARP +
                         lane_in_warp / LANES;
  const unsigned num_groups = gridDim.x * (blockDim.x >> 5) * GROUPS_PER_WARP;
  const unsigned virtual_chunks = per_round * (unsigned)p.rounds;
  const unsigned T = (unsigned)p.num_tables;

  for (unsigned vc = group; vc < virtual_chunks; vc += num_groups) {
    const unsigned round = vc / per_round;
    const int rem = (int)(vc - round * per_round);
    int j = 0;
    while (rem >= s_qpre[j + 1]) ++j;
    const int chunk = (int)round * s_quota[j] + (rem - s_qpre[j]);
    if (chunk >= s_chunks[j]) continue;
    const int q = (p.rank + 1 + j) % p.world;
    const int2* __restrict__ rec = p.list[q] + s_first[j];
    const int n = p.meta[2 * q + 1];
    float4* __restrict__ out = reinterpret_cast<float4*>(p.out[q]);

    float4 acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    unsigned cur = kNoSlot;              // output slot (float4 units) of the bag being summed
    const float4* tbase = nullptr;       // table of the bag whose rows are being loaded
    bool open = false;                   // a bag of this group is being summed
    const int chunk_end = min(n, (chunk + 1) * CHUNK);
    for (int base = chunk * CHUNK; base < n; base += LANES) {
      // one record per lane: slot = where its bag's partial sum goes, tsel = its table,
      // row = its row in that table (-1: not to be read)
      int2 r = make_int2(-1, -1);
      if (base + lane < n) r = __ldg(rec + base + lane);
      int prev_key = __shfl_up_sync(gmask, r.y, 1, LANES);
      if (lane == 0) prev_key = base > 0 ? __ldg(rec + base - 1).y : -2;
      unsigned slot = kNoSlot;
      int tsel = -1, row = -1;
      if (r.y >= 0) {
        const unsigned t = (unsigned)(((unsigned long long)(unsigned)r.y * p.batch_magic) >> p.batch_shift);
        if (t < T) {
          // the slab is laid out by key: the parts of a list land at ascending addresses, close
          // together, so the stores of the chunks in flight stay inside a few pages of each peer
          // (with a slab laid out [sample][table] every table sweeps the whole slab, and the
          // stores of one kernel spread over all pages of all peers: 2.0 ms instead of 0.7 ms
          // on four GPUs, address translation of the peer pages being the limit)
          slot = (unsigned)r.y * (unsigned)ROW4;
          tsel = (int)t;
          if (r.x >= 0 && r.x < p.rows[t]) row = r.x;
          else atomicOr(err, kErrRow);
        }
      }
      const bool starts = (base + lane < n) && (r.y != prev_key);
      const unsigned smask = (__ballot_sync(gmask, starts) >> shift) & kLaneMask;
      const int tile_n = min(LANES, n - base);
      int from = 0, to = tile_n;
      const bool inside = base < chunk_end;
      if (!open) {
        // nothing of this group is open yet: its first bag starts at the first start inside
        // the chunk; bags that began earlier belong to the group of that chunk
        if (!inside) break;
        if (smask == 0) continue;
        from = __ffs(smask) - 1;
      } else if (!inside) {
        // past the chunk: only the rest of the bag that is still open
        if (smask != 0) to = __ffs(smask) - 1;
      }
      // Bag boundaries inside the tile are the bits of smask, the same for every lane of the
      // group: no per-record comparison.  A bag's table and slot are fetched once, at its start.
      for (int j0 = from; j0 < to; j0 += INFLIGHT) {
        float4 v[INFLIGHT][VPL];
        bool has[INFLIGHT];
#pragma unroll
        for (int k = 0; k < INFLIGHT; ++k) {
          const int i = j0 + k;
          has[k] = false;
          if (i < to) {
            if ((smask >> i) & 1u) {
              const int ts = __shfl_sync(gmask, tsel, i, LANES);
              tbase = ts >= 0 ? reinterpret_cast<const float4*>(p.tab[ts]) : nullptr;
            }
            const int rw = __shfl_sync(gmask, row, i, LANES);
            has[k] = rw >= 0 && tbase != nullptr;
            if (has[k]) {
              const float4* src = tbase + (long long)rw * ROW4 + lane;
#pragma unroll
              for (int w = 0; w < VPL; ++w) v[k][w] = __ldg(src + w * LANES);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < INFLIGHT; ++k) {
          const int i = j0 + k;
          if (i < to) {
            if ((smask >> i) & 1u) {
              if (open && cur != kNoSlot) {
#pragma unroll
                for (int w = 0; w < VPL; ++w) out[cur + w * LANES + lane] = acc[w];
              }
#pragma unroll
              for (int w = 0; w < VPL; ++w) acc[w] = make_float4(0.f, 0.f, 0.f, 0.f);
              cur = __shfl_sync(gmask, slot, i, LANES);
              open = true;
            }
            if (has[k]) {
#pragma unroll
              for (int w = 0; w < VPL; ++w) emb::add4(acc[w], v[k][w]);
            }
          }
        }
      }
      if (!inside && to < tile_n) break;  // the open bag ended past the chunk
    }
    if (open && cur != kNoSlot) {
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

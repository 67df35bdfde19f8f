// Device kernels of the embedding path: segment prepass, bag (gather + segment
// reduce, with the fused uint64 hash-bucket modulo), the atomic route for
// unsorted segment ids, single-row gathers, and the helpers of the
// unique / non-zero ops.  HBM-bound: every table row is read once with 16-byte
// loads, every output row is written once.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "emb_device.cuh"

namespace annc {
namespace emb {

constexpr int kMaxTables = 120;         // tables per grouped launch: BagParams is 7.7 KB of the 32 KB
                                        // parameter space, the per-table marks fit the 512-byte header
constexpr int kErrRow = 1;              // row index outside its table
constexpr int kErrSegment = 2;          // segment id outside [0, batch)

// Head of the bag workspace (256 bytes), then int32 offsets[num_tables][batch + 1].
struct BagHeader {
  int err_bits;
  int pad[3];
  int unsorted[kMaxTables];  // per table: segment ids were seen to decrease
};
static_assert(sizeof(BagHeader) <= 512, "header layout");
constexpr size_t kHeaderBytes = 512;

struct BagTableDev {
  const float* table;
  const void* ids;
  const int64_t* seg;  // slice_input
  float* out;
  unsigned long long num_buckets;
  unsigned long long magic;  // floor((2^64 - 1) / num_buckets): reciprocal for the exact modulo
  const int* given_off;      // caller-supplied bag offsets [batch + 1] (then `seg` is not read)
  int rows;                  // (local) table rows and lookups: both below 2^31
  int nnz;
};
static_assert(sizeof(BagTableDev) == 64, "BagParams size is budgeted on 64-byte table entries");

struct BagParams {
  BagTableDev t[kMaxTables];
  int num_tables;
  int id_kind;  // 0 i32 rows, 1 i64 rows, 2 u64 fingerprints
  int combiner;
  int col;
  long long ncols;
  long long batch;
  long long dim;
  long long out_stride;
  int shard_count;  // row sharding: this rank owns rows r with r % shard_count == shard_rank,
  int shard_rank;   // stored at local row r / shard_count (the reference's mod-partition rule)
  int skip_empty;   // row sharding: bags without a lookup owned by this rank are not written
};

// ---- prepass: CSR offsets from the (sorted) segment column --------------------
// Thread i in [0, nnz] looks at the boundary between lookups i-1 and i and writes
// offsets[s] = i for every segment s in (seg[i-1], seg[i]] (empty bags included),
// with virtual seg[-1] = -1 and seg[nnz] = batch.  A decrease marks the table
// unsorted; ids outside [0, batch) set kErrSegment.
__global__ void bag_prepass_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  const int t = blockIdx.y;
  const BagTableDev& T = p.t[t];
  if (T.given_off) return;
  int* off = offsets + (long long)t * (p.batch + 1);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i <= T.nnz; i += stride) {
    long long prev = (i == 0) ? -1 : T.seg[(i - 1) * p.ncols + p.col];
    long long cur = (i == T.nnz) ? p.batch : T.seg[i * p.ncols + p.col];
    if (i < T.nnz && (cur < 0 || cur >= p.batch)) {
      atomicOr(&hdr->err_bits, kErrSegment);
      cur = cur < 0 ? 0 : p.batch;
    }
    if (prev < -1) prev = -1;
    if (prev > p.batch) prev = p.batch;
    if (cur < prev) {
      if (i < T.nnz) hdr->unsorted[t] = 1;
      continue;
    }
    for (long long s = prev + 1; s <= cur; ++s) off[s] = (int)i;
  }
}

// Same boundary walk for the common two-column index matrix (sample, position): every
// thread reads its whole 16-byte row, so a warp reads 512 contiguous bytes, and takes the
// previous lookup's segment id from its neighbour lane.
__global__ void __launch_bounds__(256)
bag_prepass2_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  const int t = blockIdx.y;
  const BagTableDev& T = p.t[t];
  if (T.given_off) return;
  int* off = offsets + (long long)t * (p.batch + 1);
  const int lane = threadIdx.x & 31;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n_round = (T.nnz + 1 + 31) / 32 * 32;  // whole warps walk the loop together
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_round; i += stride) {
    long long cur = p.batch;
    if (i < T.nnz) {
      const longlong2 v = __ldg(reinterpret_cast<const longlong2*>(T.seg) + i);
      cur = p.col == 0 ? v.x : v.y;
    }
    long long prev = __shfl_up_sync(0xffffffffu, cur, 1);
    if (lane == 0) prev = (i == 0) ? -1 : (i - 1 < T.nnz ? T.seg[(i - 1) * 2 + p.col] : p.batch);
    if (i > T.nnz) continue;
    if (i < T.nnz && (cur < 0 || cur >= p.batch)) {
      atomicOr(&hdr->err_bits, kErrSegment);
      cur = cur < 0 ? 0 : p.batch;
    }
    if (prev < -1) prev = -1;
    if (prev > p.batch) prev = p.batch;
    if (cur < prev) {
      if (i < T.nnz) hdr->unsorted[t] = 1;
      continue;
    }
    for (long long s = prev + 1; s <= cur; ++s) off[s] = (int)i;
  }
}

// Row sharding.  Returns the local row, or -2 when another rank owns the row.  Rows below
// 2^32 (every real table) take 32-bit arithmetic.
constexpr long long kNotMine = -2;
__device__ __forceinline__ long long shard_row(long long r, int shard_count, int shard_rank) {
  if (shard_count <= 1 || r < 0) return r;
  if ((unsigned long long)r <= 0xffffffffull) {
    const unsigned b = (unsigned)r, q = b / (unsigned)shard_count;
    return (b - q * (unsigned)shard_count == (unsigned)shard_rank) ? (long long)q : kNotMine;
  }
  if ((int)(r % shard_count) != shard_rank) return kNotMine;
  return r / shard_count;
}
// Owner rank of row r >= 0 under the same rule.
__device__ __forceinline__ int shard_owner(long long r, int shard_count) {
  if ((unsigned long long)r <= 0xffffffffull) return (int)((unsigned)r % (unsigned)shard_count);
  return (int)(r % shard_count);
}

// Position of the k-th (0-based) set bit of m; k must be below popc(m).
__device__ __forceinline__ int kth_set_bit(unsigned m, int k) {
  int pos = 0;
  int c = __popc(m & 0xffffu);
  if (k >= c) { k -= c; pos += 16; m >>= 16; }
  c = __popc(m & 0xffu);
  if (k >= c) { k -= c; pos += 8; m >>= 8; }
  c = __popc(m & 0xfu);
  if (k >= c) { k -= c; pos += 4; m >>= 4; }
  c = __popc(m & 0x3u);
  if (k >= c) { k -= c; pos += 2; m >>= 2; }
  if (k >= (int)(m & 1u)) pos += 1;
  return pos;
}

// ---- bag kernel: LANES lanes own one bag; each lane owns VPL float4 columns -----
// Rows are added in lookup order into a zero accumulator, the order of the
// reference's scalar loop, so sums are bit-identical for sorted input.  Four
// row loads are in flight per group.  For an unsorted table the group writes the
// zero row and clears the bag's counter; the scatter kernels then do the work.
// SHARDED (row sharding): the lookups this rank owns are first compacted inside the group
// (lookup order kept), so that the four loads in flight are all real ones, and with
// skip_empty a bag without an owned lookup is left unwritten (its owner knows from the
// bag's ids which ranks contribute, see bag_owner_mask_kernel).
template <int LANES, int VPL, bool SHARDED>
__global__ void __launch_bounds__(256, VPL == 1 ? 5 : 3)
bag_reduce_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  constexpr int GROUPS_PER_WARP = 32 / LANES;
  const int lane_in_warp = threadIdx.x & 31;
  const int lane = lane_in_warp % LANES;
  const unsigned gmask =
      (LANES == 32) ? 0xffffffffu : (((1u << LANES) - 1u) << ((lane_in_warp / LANES) * LANES));
  const long long group =
      ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * GROUPS_PER_WARP +
      lane_in_warp / LANES;
  const long long total = (long long)p.num_tables * p.batch;
  if (group >= total) return;
  const int t = (int)(group / p.batch);
  const long long s = group - (long long)t * p.batch;
  const BagTableDev& T = p.t[t];
  int* off = offsets + (long long)t * (p.batch + 1);
  const int* roff = T.given_off ? T.given_off : off;
  float* orow = T.out + s * p.out_stride;

  float4 acc[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) acc[v] = make_float4(0.f, 0.f, 0.f, 0.f);

  if (hdr->unsorted[t]) {
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      *reinterpret_cast<float4*>(orow + (v * LANES + lane) * 4) = acc[v];
    __syncwarp(gmask);
    if (lane == 0) off[s] = 0;  // becomes the bag's lookup counter
    return;
  }

  const int start = roff[s], end = roff[s + 1];
  if (!SHARDED && p.skip_empty && start == end) return;  // exchange: an empty part is not written
  int owned = 0;  // SHARDED: lookups of this bag that belong to this rank (group-uniform)
  for (int base = start; base < end; base += LANES) {
    int my = -1;  // local row (tables have fewer than 2^31 rows), -1 = skip
    bool mine = false;
    if (base + lane < end) {
      const long long r64 = shard_row(load_row_id(T.ids, p.id_kind, base + lane, T.num_buckets, T.magic),
                                      p.shard_count, p.shard_rank);
      mine = r64 != kNotMine;
      if (r64 != kNotMine && (r64 < 0 || r64 >= T.rows)) atomicOr(&hdr->err_bits, kErrRow);
      else if (r64 != kNotMine) my = (int)r64;
    }
    int n = min(LANES, end - base);
    if (SHARDED) {
      const int shift = (lane_in_warp / LANES) * LANES;
      owned += __popc(__ballot_sync(gmask, mine) >> shift & (LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u)));
      const unsigned bal = (__ballot_sync(gmask, my >= 0) >> shift) &
                           (LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u));
      n = __popc(bal);
      const int src = lane < n ? kth_set_bit(bal, lane) : lane;
      const int comp = __shfl_sync(gmask, my, src, LANES);
      my = lane < n ? comp : -1;
    }
    for (int j = 0; j < n; j += 4) {
      int r[4];
      float4 v[4][VPL];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        r[q] = __shfl_sync(gmask, my, (j + q) % LANES, LANES);
        if (j + q >= n) r[q] = -1;
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (r[q] >= 0) {
          const float* src = T.table + (long long)r[q] * p.dim;
#pragma unroll
          for (int w = 0; w < VPL; ++w) v[q][w] = ldg4(src + (w * LANES + lane) * 4);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (r[q] >= 0) {
#pragma unroll
          for (int w = 0; w < VPL; ++w) add4(acc[w], v[q][w]);
        }
      }
    }
  }
  if (SHARDED && p.skip_empty && owned == 0) return;
  if (p.combiner == 1 && end > start) {
    const float inv = __fdiv_rn(1.0f, (float)(end - start));
#pragma unroll
    for (int w = 0; w < VPL; ++w) {
      acc[w].x = __fmul_rn(acc[w].x, inv);
      acc[w].y = __fmul_rn(acc[w].y, inv);
      acc[w].z = __fmul_rn(acc[w].z, inv);
      acc[w].w = __fmul_rn(acc[w].w, inv);
    }
  }
#pragma unroll
  for (int w = 0; w < VPL; ++w)
    *reinterpret_cast<float4*>(orow + (w * LANES + lane) * 4) = acc[w];
}

// Which ranks contribute to each bag under row sharding: mask[t][s] has bit g set when bag s
// of table t has at least one lookup whose row r satisfies r % shard_count == g (in or out
// of range: the rule the senders use to decide whether they write the bag).  Half a warp per
// bag; `off` are the bag offsets of the table (given_off).
__global__ void __launch_bounds__(256)
bag_owner_mask_kernel(BagParams p, unsigned* mask) {
  const int lane = threadIdx.x & 15;
  const unsigned gmask = 0xffffu << (threadIdx.x & 16);
  const long long group = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const long long total = (long long)p.num_tables * p.batch;
  if (group >= total) return;
  const int t = (int)(group / p.batch);
  const long long s = group - (long long)t * p.batch;
  const BagTableDev& T = p.t[t];
  const int start = T.given_off[s], end = T.given_off[s + 1];
  unsigned m = 0;
  for (int i = start + lane; i < end; i += 16) {
    const long long r = load_row_id(T.ids, p.id_kind, i, T.num_buckets, T.magic);
    if (r >= 0) m |= 1u << shard_owner(r, p.shard_count);  // a negative row is nobody's
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) m |= __shfl_xor_sync(gmask, m, o, 16);
  if (lane == 0) mask[group] = m;
}

// Any dim (not a multiple of 4, or unaligned tables): one warp per bag, lanes
// stride over the columns; same summation order.
__global__ void __launch_bounds__(256)
bag_reduce_generic_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  const int lane = threadIdx.x & 31;
  const long long group = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long total = (long long)p.num_tables * p.batch;
  if (group >= total) return;
  const int t = (int)(group / p.batch);
  const long long s = group - (long long)t * p.batch;
  const BagTableDev& T = p.t[t];
  int* off = offsets + (long long)t * (p.batch + 1);
  float* orow = T.out + s * p.out_stride;
  if (hdr->unsorted[t]) {
    for (long long c = lane; c < p.dim; c += 32) orow[c] = 0.f;
    __syncwarp();
    if (lane == 0) off[s] = 0;
    return;
  }
  const int* roff = T.given_off ? T.given_off : off;
  const int start = roff[s], end = roff[s + 1];
  const float inv = (p.combiner == 1 && end > start) ? __fdiv_rn(1.0f, (float)(end - start)) : 1.0f;
  if (p.shard_count > 1 && p.skip_empty) {
    bool any = false;
    for (int i = start + lane; i < end; i += 32)
      any = any || shard_row(load_row_id(T.ids, p.id_kind, i, T.num_buckets, T.magic), p.shard_count,
                             p.shard_rank) != kNotMine;
    if (!__any_sync(0xffffffffu, any)) return;
  }
  for (long long c0 = 0; c0 < p.dim; c0 += 32) {
    const long long c = c0 + lane;
    float acc = 0.f;
    for (int i = start; i < end; ++i) {
      long long r = shard_row(load_row_id(T.ids, p.id_kind, i, T.num_buckets, T.magic), p.shard_count,
                              p.shard_rank);
      if (r == kNotMine) continue;
      if (r < 0 || r >= T.rows) {
        if (lane == 0 && c0 == 0) atomicOr(&hdr->err_bits, kErrRow);
        continue;
      }
      if (c < p.dim) acc = __fadd_rn(acc, __ldg(T.table + r * p.dim + c));
    }
    if (c < p.dim) orow[c] = (p.combiner == 1 && end > start) ? __fmul_rn(acc, inv) : acc;
  }
}

// ---- lookup-granular bag kernel ------------------------------------------------------
// The same pooling without a prepass: blockIdx.y = table; a group of LANES lanes takes a chunk
// of TILES * LANES consecutive lookups of the table (tile by tile: one lookup per lane, ids and
// segment ids read with coalesced loads, the hash-bucket modulo applied by the lane that read
// the id) and owns the bags whose first lookup lies in the chunk; it follows its last bag past
// the chunk until the segment id changes.  Bag boundaries inside a tile are one ballot; rows are
// added in lookup order into a zero accumulator (the reference's order, bit-identical sums),
// INFLIGHT row loads in flight per group.  Work per group does not depend on the bag lengths and
// short bags leave no lanes idle.  Bags without lookups are zero-filled by the group that owns
// the next bag (the first bag's owner fills from 0, the last bag's owner to the end).  A
// decrease of the segment ids marks the table unsorted: bag_stream_reset_kernel then clears its
// output and the atomic route below redoes it.
// Chunk numbering of bag_stream_kernel over all tables of a launch: table t owns the chunks
// [first[t], first[t + 1]); a table without lookups gets one chunk per 1024 bags to zero.
struct StreamChunks {
  int first[kMaxTables + 1];
};

template <int LANES, int VW, int VPL, int TILES, int INFLIGHT_, int MINB>
__global__ void __launch_bounds__(256, MINB)
bag_stream_kernel(BagParams p, StreamChunks sc, BagHeader* hdr) {
  constexpr int GROUPS_PER_WARP = 32 / LANES;
  constexpr int CHUNK = LANES * TILES;
  constexpr int INFLIGHT = LANES < INFLIGHT_ ? LANES : INFLIGHT_;
  constexpr int ROWF = LANES * VW * VPL;  // floats per row
  using Vec = RowVec<VW>;
  constexpr unsigned kLaneMask = LANES == 32 ? 0xffffffffu : ((1u << LANES) - 1u);
  constexpr int kNoBag = -3;  // a lookup whose segment id is out of range is added nowhere
  __shared__ int s_first[kMaxTables + 1];
  for (int i = threadIdx.x; i <= p.num_tables; i += blockDim.x) s_first[i] = sc.first[i];
  __syncthreads();
  const int batch = (int)p.batch;
  const int lane_in_warp = threadIdx.x & 31;
  const int lane = lane_in_warp % LANES;
  const int shift = (lane_in_warp / LANES) * LANES;
  const unsigned gmask = kLaneMask << shift;
  const unsigned group = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * GROUPS_PER_WARP +
                         lane_in_warp / LANES;
  const unsigned num_groups = gridDim.x * (blockDim.x >> 5) * GROUPS_PER_WARP;
  const unsigned total_chunks = (unsigned)s_first[p.num_tables];

  // Consecutive groups take consecutive chunks, so the whole grid works through one table
  // after the other and ends together.
  for (unsigned gc = group; gc < total_chunks; gc += num_groups) {
    int lo = 0, hi = p.num_tables - 1;  // table of chunk gc: last t with first[t] <= gc
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if ((unsigned)s_first[mid] <= gc) lo = mid;
      else hi = mid - 1;
    }
    const int t = lo;
    const unsigned chunk = gc - (unsigned)s_first[t];
    const BagTableDev& T = p.t[t];
    const int n = T.nnz;
    const float* __restrict__ tab = T.table;
    float* __restrict__ outp = T.out;

    // rows [a, b) of the output <- 0 (bags without lookups)
    auto zero_fill = [&](int a, int b) {
      Vec z;
      z.zero();
      for (int s = a; s < b; ++s) {
        float* o = outp + (long long)s * p.out_stride;
#pragma unroll
        for (int w = 0; w < VPL; ++w) z.store(o + (w * LANES + lane) * VW);
      }
    };
    if (n == 0) {  // a table without lookups: every bag is empty
      zero_fill((int)min((long long)chunk * 1024, (long long)batch), (int)min((long long)(chunk + 1) * 1024, (long long)batch));
      continue;
    }
    {
    Vec acc[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) acc[v].zero();
    int cur = kNoBag;   // bag being summed
    int count = 0;      // its lookups so far (for the mean)
    bool open = false;
    const int chunk_end = min(n, (int)(chunk + 1) * CHUNK);

    auto flush = [&]() {
      if (open && cur >= 0) {
        if (p.combiner == 1 && count > 0) {
          const float inv = __fdiv_rn(1.0f, (float)count);
#pragma unroll
          for (int w = 0; w < VPL; ++w) acc[w].scale(inv);
        }
        float* o = outp + (long long)cur * p.out_stride;
#pragma unroll
        for (int w = 0; w < VPL; ++w) acc[w].store(o + (w * LANES + lane) * VW);
      }
    };

    for (int base = (int)chunk * CHUNK; base < n; base += LANES) {
      const int i = base + lane;
      int key = kNoBag, row = -1;
      if (i < n) {
        const long long seg = T.seg[(long long)i * p.ncols + p.col];
        const long long r64 = load_row_id(T.ids, p.id_kind, i, T.num_buckets, T.magic);
        if (seg < 0 || seg >= batch) atomicOr(&hdr->err_bits, kErrSegment);
        else key = (int)seg;
        if (r64 < 0 || r64 >= T.rows) atomicOr(&hdr->err_bits, kErrRow);
        else row = (int)r64;
      }
      int prev_key = __shfl_up_sync(gmask, key, 1, LANES);
      if (lane == 0) {
        prev_key = -1;  // before the first lookup: bags 0 .. key-1 are empty
        if (base > 0) {
          const long long ps = T.seg[(long long)(base - 1) * p.ncols + p.col];
          prev_key = (ps < 0 || ps >= batch) ? kNoBag : (int)ps;
        }
      }
      const bool starts = (i < n) && (key != prev_key);
      if (starts && key >= 0 && prev_key >= 0 && key < prev_key) hdr->unsorted[t] = 1;
      const unsigned smask = (__ballot_sync(gmask, starts) >> shift) & kLaneMask;
      const int tile_n = min(LANES, n - base);
      int from = 0, to = tile_n;
      const bool inside = base < chunk_end;
      if (!open) {
        if (!inside) break;
        if (smask == 0) continue;
        from = __ffs(smask) - 1;
      } else if (!inside) {
        if (smask != 0) to = __ffs(smask) - 1;
      }
      for (int j0 = from; j0 < to; j0 += INFLIGHT) {
        Vec v[INFLIGHT][VPL];
        bool has[INFLIGHT];
#pragma unroll
        for (int k = 0; k < INFLIGHT; ++k) {
          const int j = j0 + k;
          has[k] = false;
          if (j < to) {
            const int rw = __shfl_sync(gmask, row, j, LANES);
            has[k] = rw >= 0;
            if (has[k]) {
              const float* src = tab + (long long)rw * ROWF + lane * VW;
#pragma unroll
              for (int w = 0; w < VPL; ++w) v[k][w].load(src + w * LANES * VW);
            }
          }
        }
#pragma unroll
        for (int k = 0; k < INFLIGHT; ++k) {
          const int j = j0 + k;
          if (j < to) {
            if ((smask >> j) & 1u) {
              flush();
#pragma unroll
              for (int w = 0; w < VPL; ++w) acc[w].zero();
              cur = __shfl_sync(gmask, key, j, LANES);
              const int before = __shfl_sync(gmask, prev_key, j, LANES);
              // empty bags between the previous lookup's bag and this one (sorted input only)
              if (cur >= 0 && before >= -1 && before < cur - 1) zero_fill(before + 1, cur);
              count = 0;
              open = true;
            }
            ++count;
            if (has[k]) {
#pragma unroll
              for (int w = 0; w < VPL; ++w) acc[w].add(v[k][w]);
            }
          }
        }
      }
      if (!inside && to < tile_n) break;
      // the table's last lookup: bags after its bag are empty
      if (base + tile_n >= n && to == tile_n && open && cur >= 0) zero_fill(cur + 1, batch);
    }
    flush();
    }
  }
}

// Tables marked unsorted: zero the output and the per-bag counters for the atomic route.
__global__ void __launch_bounds__(256)
bag_stream_reset_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  const int t = blockIdx.y;
  if (!hdr->unsorted[t]) return;
  const BagTableDev& T = p.t[t];
  int* counts = offsets + (long long)t * (p.batch + 1);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long total = p.batch * p.dim;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long s = e / p.dim, c = e - s * p.dim;
    T.out[s * p.out_stride + c] = 0.f;
    if (c == 0) counts[s] = 0;
  }
}

// ---- unsorted route: atomic scatter (sum order not defined; within 1e-5 rel) ----
__global__ void __launch_bounds__(256)
bag_scatter_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  const int t = blockIdx.y;
  if (!hdr->unsorted[t]) return;
  const BagTableDev& T = p.t[t];
  int* counts = offsets + (long long)t * (p.batch + 1);
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < T.nnz;
       i += warps) {
    long long seg = T.seg[i * p.ncols + p.col];
    long long r = shard_row(load_row_id(T.ids, p.id_kind, i, T.num_buckets, T.magic), p.shard_count,
                            p.shard_rank);
    if (seg < 0 || seg >= p.batch) continue;  // flagged by the prepass
    if (lane == 0) atomicAdd(&counts[seg], 1);  // bag length counts every rank's lookups
    if (r == kNotMine) continue;
    if (r < 0 || r >= T.rows) {
      if (lane == 0) atomicOr(&hdr->err_bits, kErrRow);
      continue;
    }
    float* orow = T.out + seg * p.out_stride;
    for (long long c = lane; c < p.dim; c += 32) atomicAdd(orow + c, __ldg(T.table + r * p.dim + c));
  }
}

__global__ void __launch_bounds__(256)
bag_scatter_mean_kernel(BagParams p, BagHeader* hdr, int* offsets) {
  const int t = blockIdx.y;
  if (!hdr->unsorted[t]) return;
  const BagTableDev& T = p.t[t];
  const int* counts = offsets + (long long)t * (p.batch + 1);
  const long long total = p.batch * p.dim;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long s = e / p.dim, c = e - s * p.dim;
    const int n = counts[s];
    if (n > 0) {
      float* q = T.out + s * p.out_stride + c;
      *q = __fmul_rn(*q, __fdiv_rn(1.0f, (float)n));
    }
  }
}

// ---- max segment id (+1 = batch of the reference) ------------------------------
__global__ void seg_max_kernel(const int64_t* seg, long long nnz, long long ncols, int col,
                               long long* out_max) {
  long long m = 0;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += stride) {
    long long v = seg[i * ncols + col];
    m = v > m ? v : m;
  }
  for (int o = 16; o > 0; o >>= 1) {
    long long w = __shfl_xor_sync(0xffffffffu, m, o);
    m = w > m ? w : m;
  }
  if ((threadIdx.x & 31) == 0 && m > 0) atomicMax(out_max, m);
}

// ---- single-row gathers ---------------------------------------------------------
// out[i,:] = skip(i) ? 0 : table[row(i),:]; one warp per output row.
// mode 0: KPFusedEmbeddingWithHashBucket (row = fp % num_buckets, empty -> zeros)
// mode 1: bounded variant (row outside [0, rows) -> zeros)
// mode 2: sparse_embedding2 (valid = lo <= id < hi; out = m * table[valid ? id : dflt])
struct GatherParams {
  const float* table;
  const void* ids;
  const unsigned char* empty;
  float* out;
  long long n, rows, dim;
  unsigned long long num_buckets;
  long long lo, hi, dflt;
  int mode;
  int ids64;
};

__global__ void __launch_bounds__(256) row_gather_kernel(GatherParams g, int* err) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  const bool vec = (g.dim % 4 == 0) && ((((uintptr_t)g.table) | ((uintptr_t)g.out)) % 16 == 0);
  for (long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < g.n;
       i += warps) {
    long long row = -1;
    float scale = 1.0f;
    bool use_scale = false;
    if (g.mode == 2) {
      long long id = g.ids64 ? ((const long long*)g.ids)[i] : (long long)((const int*)g.ids)[i];
      const bool valid = id >= g.lo && id < g.hi;
      row = valid ? id : g.dflt;
      scale = valid ? 1.0f : 0.0f;
      use_scale = true;
      if (row < 0 || row >= g.rows) {
        if (lane == 0) atomicOr(err, kErrRow);
        row = -1;
      }
    } else if (!(g.empty && g.empty[i])) {
      unsigned long long b = ((const unsigned long long*)g.ids)[i] % g.num_buckets;
      row = (long long)b;
      if (row < 0 || row >= g.rows) {
        if (g.mode == 0 && lane == 0) atomicOr(err, kErrRow);
        row = -1;
      }
    }
    float* o = g.out + i * g.dim;
    const float* src = row >= 0 ? g.table + row * g.dim : nullptr;
    if (vec) {
      for (long long c = lane * 4; c < g.dim; c += 128) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (src) v = ldg4(src + c);
        if (use_scale) {
          v.x = __fmul_rn(scale, v.x);
          v.y = __fmul_rn(scale, v.y);
          v.z = __fmul_rn(scale, v.z);
          v.w = __fmul_rn(scale, v.w);
        }
        *reinterpret_cast<float4*>(o + c) = v;
      }
    } else {
      for (long long c = lane; c < g.dim; c += 32) {
        float v = src ? __ldg(src + c) : 0.f;
        o[c] = use_scale ? __fmul_rn(scale, v) : v;
      }
    }
  }
}

// KPFusedSparseDynamicStitch: table = id % N, row = id / N.
struct StitchParams {
  const float* const* tables;  // device array [N]
  const long long* table_rows; // device array [N]
  const long long* x;
  float* out;
  long long n, dim;
  int num_partitions;
};

__global__ void __launch_bounds__(256) stitch_kernel(StitchParams g, int* err) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < g.n;
       i += warps) {
    const long long id = g.x[i];
    const long long t = id % g.num_partitions;
    const long long r = id / g.num_partitions;
    float* o = g.out + i * g.dim;
    if (id < 0 || !(r < g.table_rows[t])) {
      if (lane == 0) atomicOr(err, kErrRow);
      for (long long c = lane; c < g.dim; c += 32) o[c] = 0.f;
      continue;
    }
    const float* src = g.tables[t] + r * g.dim;
    const bool vec = (g.dim % 4 == 0) && ((((uintptr_t)src) | ((uintptr_t)o)) % 16 == 0);
    if (vec) {
      for (long long c = lane * 4; c < g.dim; c += 128)
        *reinterpret_cast<float4*>(o + c) = ldg4(src + c);
    } else {
      for (long long c = lane; c < g.dim; c += 32) o[c] = __ldg(src + c);
    }
  }
}

// ---- first-appearance unique (KPFusedGather, segment order of the Nonzero op) ---
// Open-addressing table of int64 keys; the empty marker is INT64_MIN, a key equal
// to the marker lives in the extra last slot.  first[slot] = smallest position
// that holds the key.
constexpr long long kEmptyKey = (long long)0x8000000000000000ull;

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 33;
  x *= 0xff51afd7ed558ccdull;
  x ^= x >> 33;
  x *= 0xc4ceb9fe1a85ec53ull;
  x ^= x >> 33;
  return x;
}

__device__ __forceinline__ long long find_or_insert(long long* keys, long long cap, long long key) {
  if (key == kEmptyKey) return cap;  // dedicated slot
  unsigned long long h = mix64((unsigned long long)key) & (unsigned long long)(cap - 1);
  for (long long probe = 0; probe < cap; ++probe) {
    long long old = atomicCAS((unsigned long long*)&keys[h], (unsigned long long)kEmptyKey,
                              (unsigned long long)key);
    if (old == kEmptyKey || old == key) return (long long)h;
    h = (h + 1) & (unsigned long long)(cap - 1);
  }
  return -1;  // table full: cannot happen with cap >= 2 * n
}

__global__ void unique_init_kernel(long long* keys, int* first, long long cap) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i <= cap; i += stride) {
    keys[i] = kEmptyKey;
    first[i] = 0x7fffffff;
  }
}

__global__ void unique_insert_kernel(const int64_t* src, long long n, long long ncols, int col,
                                     long long* keys, int* first, long long cap, int* slot_of) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    long long slot = find_or_insert(keys, cap, src[i * ncols + col]);
    slot_of[i] = (int)slot;
    if (slot >= 0) atomicMin(&first[slot], (int)i);
  }
}

__global__ void unique_flag_kernel(const int* slot_of, const int* first, long long n, int* flag) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    flag[i] = (slot_of[i] >= 0 && first[slot_of[i]] == (int)i) ? 1 : 0;
}

// rank[] = exclusive scan of flag[].  Writes unique keys in first-appearance order and
// turns first[slot] into the key's rank.
__global__ void unique_emit_kernel(const int64_t* src, long long n, long long ncols, int col,
                                   const int* slot_of, const int* flag, const int* rank,
                                   int* first, long long* out_unique) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (flag[i]) {
      if (out_unique) out_unique[rank[i]] = src[i * ncols + col];
      first[slot_of[i]] = rank[i];
    }
  }
}

// inverse[i] = rank of key i; optionally as int64 (segment column for the bag kernels).
__global__ void unique_inverse_kernel(const int* slot_of, const int* first, long long n,
                                      int* inverse32, long long* inverse64) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int r = slot_of[i] >= 0 ? first[slot_of[i]] : 0;
    if (inverse32) inverse32[i] = r;
    if (inverse64) inverse64[i] = r;
  }
}

// out[u,:] = table[unique[u],:] with the `idx < rows` check of the reference.
__global__ void __launch_bounds__(256)
unique_rows_kernel(const float* table, long long rows, long long dim, const long long* unique,
                   long long nu, float* out, int* err) {
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long u = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); u < nu;
       u += warps) {
    const long long r = unique[u];
    if (!(r < rows) || r < 0) {
      if (lane == 0) atomicOr(err, kErrRow);
      continue;
    }
    for (long long c = lane; c < dim; c += 32) out[u * dim + c] = __ldg(table + r * dim + c);
  }
}

// ---- non-zero compaction of the Nonzero op --------------------------------------
// dense f32[nseg, dim] (already scaled for mean); flag = value != 0.
__global__ void nonzero_flag_kernel(const float* dense, long long total, int* flag) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride)
    flag[e] = dense[e] != 0.0f ? 1 : 0;
}

__global__ void nonzero_emit_kernel(const float* dense, long long total, long long dim, int rank,
                                    const long long* seg_order, const int* flag, const int* pos,
                                    int* out_indices, float* out_values) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    if (!flag[e]) continue;
    const long long u = e / dim, d = e - u * dim;
    const int o = pos[e];
    out_indices[(long long)o * rank] = (int)seg_order[u];
    if (rank == 2) out_indices[(long long)o * 2 + 1] = (int)d;
    out_values[o] = dense[e];
  }
}

}  // namespace emb
}  // namespace annc

// The kn4 prepacked-weight layout written by annc-opt's layout_matmul pass
// (python/annc/optimize/data_pack.py, called with vector 12 and tiles
// (axis 0: 352), (axis 1: 128) from python/annc/optimize/constant_folding.py:77-88):
// K is cut into chunks of 352 and N into chunks of 128; when a dimension is not a
// multiple of its tile the last two chunks share the remainder, the first of the
// two rounded to a multiple of 12 (data_pack.py:53-70).  Blocks are stored K-chunk
// outer, N-chunk inner; inside a block come panels of 12 columns, then 4, 4, ..,
// 2, 1 for the tail (data_pack.py:129-149), each panel row-major [k_len, width].
#pragma once

#include <cstdint>

#ifdef __CUDACC__
#define ANNC_HD __host__ __device__ __forceinline__
#else
#define ANNC_HD inline
#endif

namespace annc {
namespace kn4 {

constexpr long long kVec = 12, kTileK = 352, kTileN = 128;

struct Chunk {
  long long start, len;
};

// Chunk of one axis that holds coordinate x.
ANNC_HD Chunk axis_chunk(long long dim, long long tile, long long x) {
  if (dim < tile) return {0, dim};
  const long long rem = dim % tile;
  if (rem == 0) return {x / tile * tile, tile};
  const long long num = dim / tile + 1;
  const long long base = (num - 2) * tile;
  if (x < base) return {x / tile * tile, tile};
  const long long res = dim - base;
  long long first = (res / 2) / kVec * kVec;
  if (res - first > first + 1) first += kVec;
  if (x < base + first) return {base, first};
  return {base + first, dim - base - first};
}

struct Panel {
  long long start, width;  // start relative to the N-chunk
};

// Panel of an N-chunk of length nlen that holds local column c.
ANNC_HD Panel panel_of(long long nlen, long long c) {
  const long long full = nlen / kVec * kVec;
  if (c < full) return {c / kVec * kVec, kVec};
  const long long rest = nlen - full;
  const long long rc = c - full;
  const long long fours = rest / 4 * 4;
  if (rc < fours) return {full + rc / 4 * 4, 4};
  const long long r2 = rest - fours, rc2 = rc - fours;
  if (r2 >= 2) {
    if (rc2 < 2) return {full + fours, 2};
    return {full + fours + 2, 1};
  }
  return {full + fours, 1};
}

// Position of B[k, n] inside the packed buffer of a [K, N] matrix.
ANNC_HD long long offset(long long K, long long N, long long k, long long n) {
  const Chunk kc = axis_chunk(K, kTileK, k);
  const Chunk nc = axis_chunk(N, kTileN, n);
  const long long c = n - nc.start;
  const Panel p = panel_of(nc.len, c);
  return kc.start * N + kc.len * (nc.start + p.start) + (k - kc.start) * p.width + (c - p.start);
}

}  // namespace kn4
}  // namespace annc

// Device helpers shared by the embedding kernels and the row-sharded exchange: the exact
// uint64 modulo of the hash-bucket mapping, id loading, 16-byte row loads with round-to-nearest
// adds, and the three-pass exclusive scan.  Kernels here are `static`: every translation unit
// that includes the header gets its own copy.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace annc {
namespace emb {

// x % d in uint64 without a division: with magic = floor((2^64 - 1) / d) the estimate
// q = hi64(x * magic) is floor(x / d) or one less, for every x and every d >= 1, so the
// remainder needs at most one correction (a second one is kept as a guard).  Bit-exact with
// the `hash % num_buckets` of fused_embedding_with_hash_bucket.cc:63-64.
__host__ __device__ __forceinline__ unsigned long long mod_magic(unsigned long long d) {
  return ~0ull / d;
}
__device__ __forceinline__ unsigned long long fast_mod_u64(unsigned long long x, unsigned long long d,
                                                           unsigned long long magic) {
  unsigned long long r = x - __umul64hi(x, magic) * d;
  if (r >= d) r -= d;
  if (r >= d) r -= d;
  return r;
}

__device__ __forceinline__ long long load_row_id(const void* ids, int id_kind, long long i,
                                                 unsigned long long num_buckets,
                                                 unsigned long long magic) {
  if (id_kind == 0) return (long long)((const int*)ids)[i];
  if (id_kind == 1) return ((const long long*)ids)[i];
  return (long long)fast_mod_u64(((const unsigned long long*)ids)[i], num_buckets, magic);
}

__device__ __forceinline__ float4 ldg4(const float* p) {
  return __ldg(reinterpret_cast<const float4*>(p));
}
__device__ __forceinline__ void add4(float4& a, const float4& b) {
  a.x = __fadd_rn(a.x, b.x);
  a.y = __fadd_rn(a.y, b.y);
  a.z = __fadd_rn(a.z, b.z);
  a.w = __fadd_rn(a.w, b.w);
}

// A lane's share of a row: VW consecutive floats (16, 8 or 4 bytes), loaded through the
// read-only path and added with round-to-nearest adds (no contraction).
template <int VW> struct RowVec;
template <> struct RowVec<4> {
  float4 v;
  __device__ __forceinline__ void zero() { v = make_float4(0.f, 0.f, 0.f, 0.f); }
  __device__ __forceinline__ void load(const float* p) { v = __ldg(reinterpret_cast<const float4*>(p)); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = v; }
  __device__ __forceinline__ void add(const RowVec& o) {
    v.x = __fadd_rn(v.x, o.v.x); v.y = __fadd_rn(v.y, o.v.y); v.z = __fadd_rn(v.z, o.v.z); v.w = __fadd_rn(v.w, o.v.w);
  }
  __device__ __forceinline__ void scale(float f) {
    v.x = __fmul_rn(v.x, f); v.y = __fmul_rn(v.y, f); v.z = __fmul_rn(v.z, f); v.w = __fmul_rn(v.w, f);
  }
};
template <> struct RowVec<2> {
  float2 v;
  __device__ __forceinline__ void zero() { v = make_float2(0.f, 0.f); }
  __device__ __forceinline__ void load(const float* p) { v = __ldg(reinterpret_cast<const float2*>(p)); }
  __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float2*>(p) = v; }
  __device__ __forceinline__ void add(const RowVec& o) { v.x = __fadd_rn(v.x, o.v.x); v.y = __fadd_rn(v.y, o.v.y); }
  __device__ __forceinline__ void scale(float f) { v.x = __fmul_rn(v.x, f); v.y = __fmul_rn(v.y, f); }
};
template <> struct RowVec<1> {
  float v;
  __device__ __forceinline__ void zero() { v = 0.f; }
  __device__ __forceinline__ void load(const float* p) { v = __ldg(p); }
  __device__ __forceinline__ void store(float* p) const { *p = v; }
  __device__ __forceinline__ void add(const RowVec& o) { v = __fadd_rn(v, o.v); }
  __device__ __forceinline__ void scale(float f) { v = __fmul_rn(v, f); }
};

// ---- exclusive scan of int32 (three passes, 2048 items per block) ---------------
constexpr int kScanThreads = 512;
constexpr int kScanItems = 4;
constexpr int kScanTile = kScanThreads * kScanItems;

__device__ __forceinline__ int block_exclusive_scan(int v, int* total_out) {
  __shared__ int warp_sums[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  if (lane == 31) warp_sums[warp] = x;
  __syncthreads();
  if (warp == 0) {
    int w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
    for (int o = 1; o < 32; o <<= 1) {
      int y = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += y;
    }
    warp_sums[lane] = w;
  }
  __syncthreads();
  const int warp_off = warp == 0 ? 0 : warp_sums[warp - 1];
  if (total_out) *total_out = warp_sums[(blockDim.x >> 5) - 1];
  const int r = warp_off + x - v;
  __syncthreads();
  return r;
}

static __global__ void __launch_bounds__(kScanThreads)
scan_tile_sums_kernel(const int* in, long long n, int* tile_sums) {
  const long long base = (long long)blockIdx.x * kScanTile + threadIdx.x * kScanItems;
  int s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k)
    if (base + k < n) s += in[base + k];
  int total;
  block_exclusive_scan(s, &total);
  if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

// One block walks all tile sums with a running carry; tile_sums becomes exclusive
// offsets and *grand_total the overall sum.
static __global__ void __launch_bounds__(kScanThreads)
scan_tile_offsets_kernel(int* tile_sums, long long ntiles, int* grand_total) {
  __shared__ int carry;
  if (threadIdx.x == 0) carry = 0;
  __syncthreads();
  for (long long base = 0; base < ntiles; base += kScanThreads) {
    const long long i = base + threadIdx.x;
    const int v = i < ntiles ? tile_sums[i] : 0;
    int total;
    const int ex = block_exclusive_scan(v, &total);
    const int c = carry;
    if (i < ntiles) tile_sums[i] = c + ex;
    __syncthreads();
    if (threadIdx.x == 0) carry = c + total;
    __syncthreads();
  }
  if (threadIdx.x == 0) *grand_total = carry;
}

static __global__ void __launch_bounds__(kScanThreads)
scan_apply_kernel(const int* in, long long n, const int* tile_offsets, int* out) {
  const long long base = (long long)blockIdx.x * kScanTile + threadIdx.x * kScanItems;
  int v[kScanItems];
  int s = 0;
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    v[k] = base + k < n ? in[base + k] : 0;
    s += v[k];
  }
  int ex = block_exclusive_scan(s, nullptr) + tile_offsets[blockIdx.x];
#pragma unroll
  for (int k = 0; k < kScanItems; ++k) {
    if (base + k < n) out[base + k] = ex;
    ex += v[k];
  }
}

}  // namespace emb
}  // namespace annc

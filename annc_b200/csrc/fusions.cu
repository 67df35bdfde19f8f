// Bandwidth-bound fusions: row softmax, masked-mean pooling, mean of absolute
// values, arg-max with last-wins ties, GEMV and the DLRM dot interaction.
#include <cfloat>

#include <cuda_bf16.h>

#include "common.h"

namespace annc {
int dot_interaction_tc(const float* z, int64_t batch, int F, int dim, int64_t z_stride, float* out,
                       int64_t out_stride, cudaStream_t s);  // interaction_tc.cu
namespace {

__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- softmax: one warp per row; rows of up to 32*4*NV floats stay in registers,
// so the row is read once and written once.
template <int NV>
__global__ void __launch_bounds__(256)
softmax_rows_reg_kernel(const float* __restrict__ in, float* __restrict__ out, long long batch,
                        int channels) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= batch) return;
  const float4* x = reinterpret_cast<const float4*>(in + row * channels);
  float4* y = reinterpret_cast<float4*>(out + row * channels);
  const int nvec = channels >> 2;
  float4 v[NV];
  float mx = -FLT_MAX;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = k * 32 + lane;
    if (c < nvec) {
      v[k] = __ldg(x + c);
      mx = fmaxf(mx, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)));
    }
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = k * 32 + lane;
    if (c < nvec) {
      v[k].x = expf(v[k].x - mx);
      v[k].y = expf(v[k].y - mx);
      v[k].z = expf(v[k].z - mx);
      v[k].w = expf(v[k].w - mx);
      sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int c = k * 32 + lane;
    if (c < nvec) {
      v[k].x = __fdiv_rn(v[k].x, sum);
      v[k].y = __fdiv_rn(v[k].y, sum);
      v[k].z = __fdiv_rn(v[k].z, sum);
      v[k].w = __fdiv_rn(v[k].w, sum);
      y[c] = v[k];
    }
  }
}

// Any channel count: three passes over the row (second and third hit L1/L2).
__global__ void __launch_bounds__(256)
softmax_rows_generic_kernel(const float* __restrict__ in, float* __restrict__ out,
                            long long batch, long long channels) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= batch) return;
  const float* x = in + row * channels;
  float* y = out + row * channels;
  float mx = -FLT_MAX;
  for (long long c = lane; c < channels; c += 32) mx = fmaxf(mx, x[c]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (long long c = lane; c < channels; c += 32) sum += expf(x[c] - mx);
  sum = warp_sum(sum);
  for (long long c = lane; c < channels; c += 32) y[c] = __fdiv_rn(expf(x[c] - mx), sum);
}

// ---- __pooling: thread per (i, p); count and sum run over j in ascending order,
// the order of the reference loops, with true division.
__global__ void pooling_kernel(float* out, const long long* arg, const float* mul_out, long long m,
                               long long k, long long n, long long s0, long long s1, long long s2,
                               long long l0, long long l1, long long l2) {
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= m * n) return;
  const long long i = e / n, p = e - i * n;
  float red = 0.f, sum = 0.f;
  const bool in_ip = i >= s0 && i < l0 && p >= s2 && p < l2;
  for (long long j = 0; j < k; ++j) {
    const bool on = arg[i * k + j] > 0;
    red = __fadd_rn(red, on ? 1.0f : 0.0f);
    float v = 0.f;
    if (on && in_ip && j >= s1 && j < l1) v = mul_out[(i * k + j) * n + p];
    sum = __fadd_rn(sum, v);
  }
  out[e] = (red == 0.f) ? 0.f : __fdiv_rn(sum, red);
}

// ---- __reduce_mean: out[i] = sum_j |value[i*m + j]| / m; warp per output.
__global__ void __launch_bounds__(256)
reduce_mean_abs_kernel(float* out, const float* value, long long m, long long n) {
  const int lane = threadIdx.x & 31;
  const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= n) return;
  float s = 0.f;
  for (long long j = lane; j < m; j += 32) s += fabsf(value[i * m + j]);
  s = warp_sum(s);
  if (lane == 0) out[i] = __fdiv_rn(s, (float)(int)m);
}

// ---- arg-max over the last dim; `val >= max` in a forward scan means the last
// position holding the maximum wins, and the initial pair wins only when it is
// strictly greater than every element.
__global__ void __launch_bounds__(256)
argmax_kernel(long long rows, long long n, const float* invals, const int* inidxs, float init_value,
              int init_idx, float* outvals, int* outidxs) {
  const int lane = threadIdx.x & 31;
  const long long r = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  float best = init_value;
  long long pos = -1;
  for (long long i = lane; i < n; i += 32) {
    const float v = invals[r * n + i];
    if (v >= best) {  // within a lane positions ascend, so >= keeps the last
      best = v;
      pos = i;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const long long op = __shfl_xor_sync(0xffffffffu, pos, o);
    if (ob > best || (ob == best && op > pos)) {
      best = ob;
      pos = op;
    }
  }
  if (lane == 0) {
    outvals[r] = best;
    outidxs[r] = pos < 0 ? init_idx : inidxs[r * n + pos];
  }
}

// ---- GEMV.  No-trans: warp per output row.  Trans: thread per output column.
__global__ void __launch_bounds__(256)
gemv_n_kernel(long long m, long long n, float alpha, const float* a, const float* x, float beta,
              float* y) {
  const int lane = threadIdx.x & 31;
  const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= m) return;
  float s = 0.f;
  for (long long j = lane; j < n; j += 32) s = fmaf(a[i * n + j], x[j], s);
  s = warp_sum(s);
  if (lane == 0) y[i] = (beta == 0.f) ? alpha * s : alpha * s + beta * y[i];
}

__global__ void __launch_bounds__(256)
gemv_t_kernel(long long m, long long n, float alpha, const float* a, const float* x, float beta,
              float* y) {
  const long long j = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float s = 0.f;
  for (long long i = 0; i < m; ++i) s = fmaf(a[i * n + j], x[i], s);
  y[j] = (beta == 0.f) ? alpha * s : alpha * s + beta * y[j];
}

// ---- DLRM dot interaction.  One warp per sample: the F x D block is staged in
// shared memory (rows padded by one float), lane i keeps row i in registers and
// walks rows j < i, which every lane reads at the same address (a broadcast).
// The 64-wide row 0 and the strict lower triangle are then written as one
// contiguous output row.
template <int D>
__global__ void __launch_bounds__(128)
dot_interaction_kernel(const float* __restrict__ z, long long batch, int F, long long z_stride,
                       float* __restrict__ out, long long out_stride) {
  constexpr int LD = D + 4;  // keeps 16-byte alignment of every row
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long b = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (b >= batch) return;
  const int tri = F * (F - 1) / 2;
  float* zs = smem + (size_t)warp * (32 * LD + 32 * 32);
  float* res = zs + 32 * LD;  // up to 496 pair results
  const float* zb = z + b * z_stride;
  for (int e = lane; e < F * (D / 4); e += 32) {
    const int r = e / (D / 4), c = e - r * (D / 4);
    const float4 v = __ldg(reinterpret_cast<const float4*>(zb + (long long)r * D) + c);
    *reinterpret_cast<float4*>(zs + r * LD + c * 4) = v;
  }
  __syncwarp();
  float mine[D];
  if (lane < F) {
#pragma unroll
    for (int c = 0; c < D; c += 4) {
      const float4 v = *reinterpret_cast<const float4*>(zs + lane * LD + c);
      mine[c] = v.x;
      mine[c + 1] = v.y;
      mine[c + 2] = v.z;
      mine[c + 3] = v.w;
    }
  }
  for (int j = 0; j < F - 1; ++j) {
    if (lane > j && lane < F) {
      float acc = 0.f;
      const float* rj = zs + j * LD;
#pragma unroll
      for (int c = 0; c < D; c += 4) {
        const float4 v = *reinterpret_cast<const float4*>(rj + c);
        acc = fmaf(mine[c], v.x, acc);
        acc = fmaf(mine[c + 1], v.y, acc);
        acc = fmaf(mine[c + 2], v.z, acc);
        acc = fmaf(mine[c + 3], v.w, acc);
      }
      res[lane * (lane - 1) / 2 + j] = acc;
    }
  }
  __syncwarp();
  float* ob = out + b * out_stride;
  for (int c = lane; c < D; c += 32) ob[c] = zs[c];
  for (int e = lane; e < tri; e += 32) ob[D + e] = res[e];
  for (long long e = D + tri + lane; e < out_stride; e += 32) ob[e] = 0.f;
}

// ---- sum of partial pooled vectors, ascending part order (deterministic).
__global__ void __launch_bounds__(256)
sum_partials_kernel(const float* __restrict__ src, int parts, long long part_stride, long long rows,
                    long long width4, long long src_stride, float* __restrict__ out,
                    long long out_stride) {
  const long long total = rows * width4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long r = e / width4, c = (e - r * width4) * 4;
    const float* s0 = src + r * src_stride + c;
    float4 acc = __ldg(reinterpret_cast<const float4*>(s0));
    for (int p = 1; p < parts; ++p) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(s0 + p * part_stride));
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    *reinterpret_cast<float4*>(out + r * out_stride + c) = acc;
  }
}

// Same sum restricted to the parts named by mask[slot][row] (bit p = part p holds this row's
// slot); parts whose bit is clear were never written and are not read.
__global__ void __launch_bounds__(256)
sum_partials_masked_kernel(const float* __restrict__ src, const unsigned* __restrict__ mask,
                           int parts, long long part_stride, long long rows, int slots,
                           int slot_w4, const int* __restrict__ mean_off, float* __restrict__ out,
                           long long out_stride, int out_bf16, int slot_major,
                           const int* __restrict__ out_slot) {
  const long long width4 = (long long)slots * slot_w4;
  const long long total = rows * width4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long r = e / width4;
    const int c4 = (int)(e - r * width4);
    const int slot = c4 / slot_w4;
    unsigned m = __ldg(mask + (long long)slot * rows + r);
    // a part holds [rows, slots, slot_width], or [slots, rows, slot_width] when slot_major
    const float* s0 = src + (slot_major ? ((long long)slot * rows + r) * slot_w4 + (c4 - slot * slot_w4)
                                        : r * width4 + c4) * 4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool first = true;
    // (keeping several part loads in flight per thread before the first add was tried and is
    // slower: 0.31 ms against 0.28 ms on four GPUs; the pass has enough threads in flight)
    while (m) {
      const int p = __ffs(m) - 1;
      m &= m - 1;
      if (p >= parts) break;
      const float4 v = __ldg(reinterpret_cast<const float4*>(s0 + p * part_stride));
      if (first) {
        acc = v;
        first = false;
      } else {
        acc.x = __fadd_rn(acc.x, v.x);
        acc.y = __fadd_rn(acc.y, v.y);
        acc.z = __fadd_rn(acc.z, v.z);
        acc.w = __fadd_rn(acc.w, v.w);
      }
    }
    if (mean_off) {  // mean pooling: the sum times 1/len(bag), like the reference's second pass
      const int* o = mean_off + (long long)slot * (rows + 1) + r;
      const int len = o[1] - o[0];
      if (len > 0) {
        const float inv = __fdiv_rn(1.0f, (float)len);
        acc.x = __fmul_rn(acc.x, inv);
        acc.y = __fmul_rn(acc.y, inv);
        acc.z = __fmul_rn(acc.z, inv);
        acc.w = __fmul_rn(acc.w, inv);
      }
    }
    // slot t of the parts lands in slot out_slot[t] of the output row (identity without a map)
    const long long oc = out_slot ? ((long long)__ldg(out_slot + slot) * slot_w4 + (c4 - slot * slot_w4)) * 4
                                  : (long long)c4 * 4;
    if (out_bf16) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
      uint2 o;
      o.x = *reinterpret_cast<uint32_t*>(&lo);
      o.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + r * out_stride + oc) = o;
    } else {
      *reinterpret_cast<float4*>(out + r * out_stride + oc) = acc;
    }
  }
}

// ---- synthetic table rows from a counter-based hash ---------------------------------
// value(seed, table, row, col) in [-0.05, 0.05): splitmix64 of the counter, top 24 bits scaled
// with one fp32 multiply and one fp32 subtract (no fused multiply-add), so a numpy restatement
// of the same integer and fp32 steps reproduces every element bit for bit and a table too
// large for host memory can still be checked row by row.
__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__global__ void __launch_bounds__(256)
synth_fill_rows_kernel(float* __restrict__ table, long long local_rows, int dim4,
                       unsigned long long seed, unsigned long long table_id,
                       unsigned long long first_row, unsigned long long row_step,
                       const long long* __restrict__ row_list) {
  const long long total = local_rows * dim4;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const unsigned long long base = seed ^ (table_id * 0x9E3779B97F4A7C15ull);
  const float scale = 0.1f * 5.9604644775390625e-8f;  // 0.1f * 2^-24, exact
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long i = e / dim4;
    const int c0 = (int)(e - i * dim4) * 4;
    const unsigned long long row = row_list ? (unsigned long long)row_list[i]
                                            : first_row + (unsigned long long)i * row_step;
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned long long h = splitmix64(base + row * 0xD1B54A32D192ED03ull +
                                              (unsigned long long)(c0 + j) * 0x8CB92BA72F3D8DD7ull);
      v[j] = __fsub_rn(__fmul_rn((float)(unsigned)(h >> 40), scale), 0.05f);
    }
    *reinterpret_cast<float4*>(table + e * 4) = make_float4(v[0], v[1], v[2], v[3]);
  }
}

}  // namespace
}  // namespace annc

using namespace annc;

extern "C" {

int annc_softmax_dev(const float* in, float* out, int64_t batch, int64_t channels, void* stream) {
  ANNC_REQUIRE(in && out, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (batch <= 0 || channels <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((batch + 7) / 8);
  const bool vec = channels % 4 == 0 && channels <= 1024 &&
                   ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  if (vec && channels <= 128) {
    softmax_rows_reg_kernel<1><<<blocks, 256, 0, s>>>(in, out, batch, (int)channels);
  } else if (vec && channels <= 256) {
    softmax_rows_reg_kernel<2><<<blocks, 256, 0, s>>>(in, out, batch, (int)channels);
  } else if (vec && channels <= 512) {
    softmax_rows_reg_kernel<4><<<blocks, 256, 0, s>>>(in, out, batch, (int)channels);
  } else if (vec) {
    softmax_rows_reg_kernel<8><<<blocks, 256, 0, s>>>(in, out, batch, (int)channels);
  } else {
    softmax_rows_generic_kernel<<<blocks, 256, 0, s>>>(in, out, batch, channels);
  }
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_pooling_dev(float* out, const int64_t* arg, const float* mul_out, int64_t m, int64_t k,
                     int64_t n, const int64_t slice_starts[3], const int64_t slice_limits[3],
                     void* stream) {
  ANNC_REQUIRE(out && arg && mul_out && slice_starts && slice_limits, ANNC_ERR_INVALID_ARGUMENT,
               "null argument");
  if (m * n <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  pooling_kernel<<<(unsigned)((m * n + 255) / 256), 256, 0, s>>>(
      out, (const long long*)arg, mul_out, m, k, n, slice_starts[0], slice_starts[1],
      slice_starts[2], slice_limits[0], slice_limits[1], slice_limits[2]);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_reduce_mean_dev(float* out, const float* value, int64_t m, int64_t n, void* stream) {
  ANNC_REQUIRE(out && value, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (n <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  reduce_mean_abs_kernel<<<(unsigned)((n + 7) / 8), 256, 0, s>>>(out, value, m, n);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_argmax_dev(int64_t rows, int64_t n, const float* invals, const int32_t* inidxs,
                    float init_value, int32_t init_idx, float* outvals, int32_t* outidxs,
                    void* stream) {
  ANNC_REQUIRE(invals && inidxs && outvals && outidxs, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (rows <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  argmax_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(rows, n, invals, inidxs, init_value,
                                                          init_idx, outvals, outidxs);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_gemv_dev(int trans_a, int64_t m, int64_t n, float alpha, const float* a, const float* x,
                  float beta, float* y, void* stream) {
  ANNC_REQUIRE(a && x && y, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (m <= 0 || n <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!trans_a) {
    gemv_n_kernel<<<(unsigned)((m + 7) / 8), 256, 0, s>>>(m, n, alpha, a, x, beta, y);
  } else {
    gemv_t_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(m, n, alpha, a, x, beta, y);
  }
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_sum_partials_dev(const float* src, int parts, int64_t part_stride, int64_t rows,
                          int64_t width, int64_t src_stride, float* out, int64_t out_stride,
                          void* stream) {
  ANNC_REQUIRE(src && out && parts >= 1, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE((width & 3) == 0 && (src_stride & 3) == 0 && (out_stride & 3) == 0 &&
                   (part_stride & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
               ANNC_ERR_INVALID_ARGUMENT, "sum_partials needs 16-byte aligned rows");
  if (rows * width <= 0) return ANNC_OK;
  long long g = (rows * (width / 4) + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  sum_partials_kernel<<<(unsigned)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, parts, part_stride, rows, width / 4, src_stride, out, out_stride);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

static int sum_partials_masked(const float* src, const uint32_t* mask, int parts,
                                 int64_t part_stride, int64_t rows, int slots, int64_t slot_width,
                                 const int32_t* mean_offsets, void* out, int64_t out_stride,
                                 int out_bf16, void* stream, int slot_major, const int32_t* out_slot) {
  ANNC_REQUIRE(src && out && mask && parts >= 1 && parts <= 32 && slots >= 1,
               ANNC_ERR_INVALID_ARGUMENT, "null or bad argument");
  ANNC_REQUIRE((slot_width & 3) == 0 && slot_width > 0 && (out_stride & 3) == 0 &&
                   (part_stride & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(out)) & 15) == 0,
               ANNC_ERR_INVALID_ARGUMENT, "sum_partials needs 16-byte aligned rows");
  if (rows <= 0) return ANNC_OK;
  long long g = (rows * slots * (slot_width / 4) + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  sum_partials_masked_kernel<<<(unsigned)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, mask, parts, part_stride, rows, slots, (int)(slot_width / 4), mean_offsets,
      static_cast<float*>(out), out_stride, out_bf16 ? 1 : 0, slot_major, out_slot);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_sum_partials_masked_dev(const float* src, const uint32_t* mask, int parts,
                                 int64_t part_stride, int64_t rows, int slots, int64_t slot_width,
                                 const int32_t* mean_offsets, void* out, int64_t out_stride,
                                 int out_bf16, void* stream) {
  return sum_partials_masked(src, mask, parts, part_stride, rows, slots, slot_width, mean_offsets, out,
                             out_stride, out_bf16, stream, 0, nullptr);
}

int annc_sum_partials_masked_slot_major_dev(const float* src, const uint32_t* mask, int parts,
                                            int64_t part_stride, int64_t rows, int slots,
                                            int64_t slot_width, const int32_t* mean_offsets,
                                            const int32_t* out_slots, void* out, int64_t out_stride,
                                            int out_bf16, void* stream) {
  return sum_partials_masked(src, mask, parts, part_stride, rows, slots, slot_width, mean_offsets, out,
                             out_stride, out_bf16, stream, 1, out_slots);
}

int annc_synth_fill_rows_dev(float* table, int64_t local_rows, int64_t dim, uint64_t seed,
                             int64_t table_id, int64_t first_row, int64_t row_step, void* stream) {
  ANNC_REQUIRE(table && local_rows >= 0 && dim >= 4 && (dim & 3) == 0 && first_row >= 0 && row_step >= 1 &&
                   (reinterpret_cast<uintptr_t>(table) & 15) == 0,
               ANNC_ERR_INVALID_ARGUMENT, "synth fill: bad arguments");
  if (local_rows == 0) return ANNC_OK;
  synth_fill_rows_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      table, local_rows, (int)(dim / 4), seed, (unsigned long long)table_id,
      (unsigned long long)first_row, (unsigned long long)row_step, nullptr);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_synth_fill_row_list_dev(float* table, const int64_t* rows, int64_t count, int64_t dim,
                                 uint64_t seed, int64_t table_id, void* stream) {
  ANNC_REQUIRE(table && rows && count >= 0 && dim >= 4 && (dim & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(table) & 15) == 0,
               ANNC_ERR_INVALID_ARGUMENT, "synth fill: bad arguments");
  if (count == 0) return ANNC_OK;
  synth_fill_rows_kernel<<<148 * 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      table, count, (int)(dim / 4), seed, (unsigned long long)table_id, 0ull, 1ull,
      reinterpret_cast<const long long*>(rows));
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_copy_rows_dev(float* dst, int64_t dst_stride, const float* src, int64_t src_stride,
                       int64_t width, int64_t rows, void* stream) {
  ANNC_REQUIRE(dst && src, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (rows <= 0 || width <= 0) return ANNC_OK;
  ANNC_CUDA(cudaMemcpy2DAsync(dst, (size_t)dst_stride * 4, src, (size_t)src_stride * 4,
                              (size_t)width * 4, (size_t)rows, cudaMemcpyDeviceToDevice,
                              static_cast<cudaStream_t>(stream)));
  return ANNC_OK;
}

int annc_dot_interaction_dev(const float* z, int64_t batch, int features, int dim,
                             int64_t z_stride, float* out, int64_t out_stride, int math,
                             void* stream) {
  ANNC_REQUIRE(z && out, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (math != ANNC_MATH_FP32 && batch > 0 && features >= 2 &&
      out_stride >= dim + features * (features - 1) / 2) {
    const int rc = dot_interaction_tc(z, batch, features, dim, z_stride, out, out_stride,
                                      static_cast<cudaStream_t>(stream));
    if (rc != ANNC_ERR_UNSUPPORTED) return rc;
    if (math == ANNC_MATH_TF32)
      return fail(ANNC_ERR_UNSUPPORTED, "dot interaction: shape not supported by the tensor-core kernel");
  }
  ANNC_REQUIRE(features >= 1 && features <= 32, ANNC_ERR_UNSUPPORTED,
               "dot interaction supports up to 32 feature vectors");
  ANNC_REQUIRE(dim == 64 || dim == 128 || dim == 32 || dim == 16, ANNC_ERR_UNSUPPORTED,
               "dot interaction supports dim 16, 32, 64 or 128");
  const int tri = features * (features - 1) / 2;
  ANNC_REQUIRE(out_stride >= dim + tri && z_stride >= (int64_t)features * dim,
               ANNC_ERR_INVALID_ARGUMENT, "strides too small");
  ANNC_REQUIRE(((reinterpret_cast<uintptr_t>(z) & 15) == 0) && z_stride % 4 == 0,
               ANNC_ERR_INVALID_ARGUMENT, "z must be 16-byte aligned");
  if (batch <= 0) return ANNC_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned blocks = (unsigned)((batch + 3) / 4);
  const size_t smem = 4 * (size_t)(32 * (dim + 4) + 32 * 32) * sizeof(float);
#define ANNC_LAUNCH_DOT(D)                                                                     \
  {                                                                                            \
    ANNC_CUDA(cudaFuncSetAttribute(dot_interaction_kernel<D>,                                  \
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));   \
    dot_interaction_kernel<D><<<blocks, 128, smem, s>>>(z, batch, features, z_stride, out,     \
                                                        out_stride);                           \
  }
  if (dim == 16) ANNC_LAUNCH_DOT(16)
  else if (dim == 32) ANNC_LAUNCH_DOT(32)
  else if (dim == 64) ANNC_LAUNCH_DOT(64)
  else ANNC_LAUNCH_DOT(128)
#undef ANNC_LAUNCH_DOT
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

}  // extern "C"

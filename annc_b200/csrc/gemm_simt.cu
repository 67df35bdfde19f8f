// fp32 GEMM on the CUDA cores: the route for shapes the tensor-core kernel does
// not take (tiny or unaligned problems, transposed A, fp32-exact requests such
// as KPFusedBatchMatMulAddSigmoid whose reference tolerance is 1e-5).
// 64x64x16 block tile, 4x4 register tile, strided batch on blockIdx.z.
#include "common.h"
#include "gemm.h"
#include "kn4.h"

namespace annc {
namespace gemm {
namespace {

constexpr int BM = 64, BN = 64, BK = 16;

__device__ __forceinline__ float apply_act(float v, int act) {
  if (act == ANNC_ACT_RELU) return fmaxf(v, 0.0f);
  if (act == ANNC_ACT_SIGMOID) return __fdiv_rn(1.0f, 1.0f + expf(-v));
  return v;
}

__global__ void __launch_bounds__(256) sgemm_simt_kernel(annc_gemm_desc d, int bias_mode,
                                                        long long bias_s0, long long bias_s1,
                                                        long long bias_s2) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const long long bz = blockIdx.z;
  const float* A = d.a + bz * d.stride_a;
  const float* B = d.b + bz * d.stride_b;
  float* C = d.c + bz * d.stride_c;
  const float* Add = d.addend ? d.addend + bz * d.stride_addend : nullptr;
  const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (long long k0 = 0; k0 < d.k; k0 += BK) {
    // A tile: BM x BK, element (i, kk) = op(A)[m0+i, k0+kk]
    for (int e = tid; e < BM * BK; e += 256) {
      int i, kk;
      if (d.trans_a) {  // A stored [k, m]: consecutive threads walk m
        i = e % BM;
        kk = e / BM;
      } else {  // A stored [m, k]: consecutive threads walk k
        kk = e % BK;
        i = e / BK;
      }
      const long long gm = m0 + i, gk = k0 + kk;
      float v = 0.f;
      if (gm < d.m && gk < d.k) v = d.trans_a ? A[gk * d.lda + gm] : A[gm * d.lda + gk];
      As[kk][i] = v;
    }
    for (int e = tid; e < BN * BK; e += 256) {
      int j, kk;
      if (d.trans_b) {  // B stored [n, k]
        kk = e % BK;
        j = e / BK;
      } else {  // B stored [k, n]
        j = e % BN;
        kk = e / BN;
      }
      const long long gn = n0 + j, gk = k0 + kk;
      float v = 0.f;
      if (gn < d.n && gk < d.k) {
        if (d.b_format == ANNC_B_KN4) {
          v = B[kn4::offset(d.k, d.n, gk, gn)];
        } else {
          v = d.trans_b ? B[gn * d.ldb + gk] : B[gk * d.ldb + gn];
        }
      }
      Bs[kk][j] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long gm = m0 + ty * 4 + i;
    if (gm >= d.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long gn = n0 + tx * 4 + j;
      if (gn >= d.n) continue;
      float v = d.alpha * acc[i][j];
      if (d.beta != 0.f) v += d.beta * C[gm * d.ldc + gn];
      if (Add) v += Add[gm * d.ld_addend + gn];
      if (d.bias) {
        v += bias_mode ? d.bias[bz * bias_s0 + gm * bias_s1 + gn * bias_s2] : d.bias[gn];
      }
      C[gm * d.ldc + gn] = apply_act(v, d.activation);
    }
  }
}

// n == 1 with row-major A: one warp per output row (a GEMV with the GEMM epilogue).
__global__ void __launch_bounds__(256) sgemm_n1_kernel(annc_gemm_desc d) {
  const int lane = threadIdx.x & 31;
  const long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (i >= d.m) return;
  const float* a = d.a + i * d.lda;
  float s = 0.f;
  for (long long k = lane; k < d.k; k += 32) s = fmaf(a[k], d.b[k], s);
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    float v = d.alpha * s;
    if (d.beta != 0.f) v += d.beta * d.c[i * d.ldc];
    if (d.addend) v += d.addend[i * d.ld_addend];
    if (d.bias) v += d.bias[0];
    d.c[i * d.ldc] = apply_act(v, d.activation);
  }
}

// k <= 16 with row-major A and B (the first DLRM layer, 13 dense features): the work is
// writing C.  A thread keeps its four columns of B in registers, 64 rows of A sit in
// shared memory, every output row is written with coalesced 16-byte stores.
constexpr int SK_ROWS = 64, SK_MAXK = 16;
__global__ void __launch_bounds__(128) sgemm_smallk_kernel(annc_gemm_desc d) {
  __shared__ float As[SK_ROWS][SK_MAXK];
  const long long m0 = (long long)blockIdx.y * SK_ROWS;
  const long long col = ((long long)blockIdx.x * 128 + threadIdx.x) * 4;
  for (int e = threadIdx.x; e < SK_ROWS * SK_MAXK; e += 128) {
    const int r = e / SK_MAXK, k = e % SK_MAXK;
    As[r][k] = (m0 + r < d.m && k < d.k) ? d.a[(m0 + r) * d.lda + k] : 0.f;
  }
  float4 w[SK_MAXK];
#pragma unroll
  for (int k = 0; k < SK_MAXK; ++k) {
    w[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (k < d.k && col < d.n) w[k] = __ldg(reinterpret_cast<const float4*>(d.b + k * d.ldb + col));
  }
  float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
  if (d.bias && col < d.n) bias = __ldg(reinterpret_cast<const float4*>(d.bias + col));
  __syncthreads();
  if (col >= d.n) return;
  const int rows = (int)(d.m - m0 < SK_ROWS ? d.m - m0 : SK_ROWS);
  for (int r = 0; r < rows; ++r) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < SK_MAXK; ++k) {
      const float a = As[r][k];
      acc.x = fmaf(a, w[k].x, acc.x);
      acc.y = fmaf(a, w[k].y, acc.y);
      acc.z = fmaf(a, w[k].z, acc.z);
      acc.w = fmaf(a, w[k].w, acc.w);
    }
    float* crow = d.c + (m0 + r) * d.ldc + col;
    float v[4] = {d.alpha * acc.x, d.alpha * acc.y, d.alpha * acc.z, d.alpha * acc.w};
    if (d.beta != 0.f) {
      const float4 o = *reinterpret_cast<const float4*>(crow);
      v[0] += d.beta * o.x; v[1] += d.beta * o.y; v[2] += d.beta * o.z; v[3] += d.beta * o.w;
    }
    if (d.addend) {
      const float4 a4 = __ldg(reinterpret_cast<const float4*>(d.addend + (m0 + r) * d.ld_addend + col));
      v[0] += a4.x; v[1] += a4.y; v[2] += a4.z; v[3] += a4.w;
    }
    float4 o;
    o.x = apply_act(v[0] + bias.x, d.activation);
    o.y = apply_act(v[1] + bias.y, d.activation);
    o.z = apply_act(v[2] + bias.z, d.activation);
    o.w = apply_act(v[3] + bias.w, d.activation);
    *reinterpret_cast<float4*>(crow) = o;
  }
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

int run_simt(const annc_gemm_desc& d, cudaStream_t s, const BiasBroadcast* bb) {
  if (d.m <= 0 || d.n <= 0 || d.batch <= 0) return ANNC_OK;
  if (d.n == 1 && d.batch == 1 && !d.trans_a && !bb && d.b_format == ANNC_B_PLAIN &&
      (d.trans_b || d.ldb == 1)) {
    sgemm_n1_kernel<<<(unsigned)((d.m + 7) / 8), 256, 0, s>>>(d);
    ANNC_CUDA(cudaGetLastError());
    return ANNC_OK;
  }
  if (d.k <= SK_MAXK && d.k >= 1 && d.m >= 1024 && d.batch == 1 && !d.trans_a && !d.trans_b && !bb &&
      d.b_format == ANNC_B_PLAIN && (d.n & 3) == 0 && (d.ldb & 3) == 0 && (d.ldc & 3) == 0 &&
      aligned16(d.b) && aligned16(d.c) && (!d.bias || aligned16(d.bias)) &&
      (!d.addend || (aligned16(d.addend) && (d.ld_addend & 3) == 0)) &&
      (d.m + SK_ROWS - 1) / SK_ROWS <= 65535) {
    dim3 grid((unsigned)((d.n / 4 + 127) / 128), (unsigned)((d.m + SK_ROWS - 1) / SK_ROWS));
    sgemm_smallk_kernel<<<grid, 128, 0, s>>>(d);
    ANNC_CUDA(cudaGetLastError());
    return ANNC_OK;
  }
  const long long gx = (d.n + BN - 1) / BN, gy = (d.m + BM - 1) / BM;
  if (gy > 65535) return fail(ANNC_ERR_UNSUPPORTED, "simt gemm: more than 4M rows");
  // blockIdx.z is limited to 65535: walk the batch in slabs.
  for (long long b0 = 0; b0 < d.batch; b0 += 65535) {
    annc_gemm_desc e = d;
    e.batch = d.batch - b0 < 65535 ? d.batch - b0 : 65535;
    e.a = d.a + b0 * d.stride_a;
    e.b = d.b + b0 * d.stride_b;
    e.c = d.c + b0 * d.stride_c;
    if (d.addend) e.addend = d.addend + b0 * d.stride_addend;
    if (d.bias && bb) e.bias = d.bias + b0 * bb->s0;
    dim3 grid((unsigned)gx, (unsigned)gy, (unsigned)e.batch);
    sgemm_simt_kernel<<<grid, 256, 0, s>>>(e, bb ? 1 : 0, bb ? bb->s0 : 0, bb ? bb->s1 : 0,
                                           bb ? bb->s2 : 0);
  }
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

}  // namespace gemm
}  // namespace annc

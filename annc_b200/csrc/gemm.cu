// GEMM dispatcher, the kn4 converters and the KPFusedBatchMatMulAddSigmoid twin.
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

#include "common.h"
#include "gemm.h"
#include "kn4.h"

namespace annc {
namespace gemm {

static int validate(const annc_gemm_desc& d) {
  ANNC_REQUIRE(d.a && d.b && d.c, ANNC_ERR_INVALID_ARGUMENT, "gemm: null operand");
  ANNC_REQUIRE(d.m >= 0 && d.n >= 0 && d.k >= 0 && d.batch >= 1, ANNC_ERR_INVALID_ARGUMENT,
               "gemm: bad extents");
  ANNC_REQUIRE(d.activation >= ANNC_ACT_NONE && d.activation <= ANNC_ACT_SIGMOID,
               ANNC_ERR_INVALID_ARGUMENT, "gemm: bad activation");
  ANNC_REQUIRE(d.b_format == ANNC_B_PLAIN || d.b_format == ANNC_B_KN4, ANNC_ERR_INVALID_ARGUMENT,
               "gemm: bad b_format");
  ANNC_REQUIRE(d.b_format == ANNC_B_PLAIN || !d.trans_b, ANNC_ERR_INVALID_ARGUMENT,
               "gemm: kn4 B cannot be transposed");
  ANNC_REQUIRE(d.math >= ANNC_MATH_AUTO && d.math <= ANNC_MATH_BF16, ANNC_ERR_INVALID_ARGUMENT,
               "gemm: bad math mode");
  return ANNC_OK;
}

// The CTA-pair kernel works on 256 x 256 tiles with a long main loop per tile: it takes the
// compute-bound GEMMs.  Skinny layers (small K, output-bound) stay on the single-CTA kernel,
// whose two resident CTAs per SM and staged, coalesced epilogue stream C faster.
static bool use_pair(const annc_gemm_desc& d, int math) {
  if (!pair_supported(d, math)) return false;
  if (math == ANNC_MATH_BF16 || (d.io_flags & (ANNC_IO_SOFTMAX | ANNC_IO_PAIR))) return true;
  if (!tc_supported(d, math)) return true;
  // 256 x 256 pair tiles pay off when there are enough of them to occupy the SM pairs; a
  // smaller product runs on the single-CTA kernel (128 x 128 tiles, split K inside a cluster
  // when even those are few).
  const long long pair_tiles = ((d.m + 255) / 256) * ((d.n + 255) / 256) * d.batch;
  return d.m >= 256 && d.n >= 192 && d.k >= 1024 && pair_tiles >= 74;
}

// AUTO: tensor cores (TF32) when the shape fits a tcgen05 kernel, else CUDA cores.
static int pick_math(const annc_gemm_desc& d) {
  if (d.math == ANNC_MATH_FP32) return ANNC_MATH_FP32;
  const int want = d.math == ANNC_MATH_AUTO ? ANNC_MATH_TF32 : d.math;
  if (d.math == ANNC_MATH_AUTO && d.io_flags == 0 && (d.m < 64 || d.n < 16 || d.k < 32))
    return ANNC_MATH_FP32;  // tiny shapes stay on the CUDA cores
  return (tc_supported(d, want) || pair_supported(d, want)) ? want : ANNC_MATH_FP32;
}

const char* route_name(const annc_gemm_desc& d) {
  const int math = pick_math(d);
  switch (math) {
    case ANNC_MATH_TF32: return use_pair(d, math) ? "tcgen05_pair_tf32" : "tcgen05_tf32";
    case ANNC_MATH_BF16: return "tcgen05_pair_bf16";
    default: return "simt_fp32";
  }
}

namespace {

__global__ void kn4_convert_kernel(const float* src, float* dst, long long K, long long N,
                                   int to_packed) {
  const long long total = K * N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long k = e / N, n = e - k * N;
    const long long o = kn4::offset(K, N, k, n);
    if (to_packed) dst[o] = src[e];
    else dst[e] = src[o];
  }
}

// kn4 -> [K,N] in 16-byte chunks (N % 4 == 0, so a chunk never straddles two panels);
// thread per chunk, rows on blockIdx.y.
__global__ void __launch_bounds__(256)
kn4_unpack_chunks_kernel(const float* __restrict__ src, float* __restrict__ dst, int K, int N) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int n = c * 4;
  if (n >= N) return;
  const kn4::Chunk nc = kn4::axis_chunk(N, kn4::kTileN, n);
  const kn4::Panel pn = kn4::panel_of(nc.len, n - nc.start);
  const long long term = nc.start + pn.start, in0 = n - nc.start - pn.start;
  for (int k = blockIdx.y; k < K; k += gridDim.y) {
    const kn4::Chunk kc = kn4::axis_chunk(K, kn4::kTileK, k);
    const float* p = src + kc.start * N + kc.len * term + (k - kc.start) * pn.width + in0;
    *reinterpret_cast<float4*>(dst + (long long)k * N + n) = __ldg(reinterpret_cast<const float4*>(p));
  }
}

// kn4 -> [N,K] (the K-major layout the TMA route likes best): a block moves a 32 (k) x 32 (n)
// tile through shared memory, reading the packed buffer along n and writing rows of k.
__global__ void __launch_bounds__(256)
kn4_unpack_transposed_kernel(const float* __restrict__ src, float* __restrict__ dst, long long K,
                             long long N) {
  __shared__ float tile[32][33];
  const long long n0 = (long long)blockIdx.x * 32, k0 = (long long)blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {
    const long long k = k0 + r, n = n0 + tx;
    tile[r][tx] = (k < K && n < N) ? src[kn4::offset(K, N, k, n)] : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const long long n = n0 + r, k = k0 + tx;
    if (n < N && k < K) dst[n * K + k] = tile[tx][r];
  }
}

__global__ void cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                 long long n) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dst[i] = __float2bfloat16_rn(src[i]);
}

// [K,N] fp32 -> [N,K] bf16 through a 32 x 32 shared-memory tile.
__global__ void __launch_bounds__(256)
bf16_weight_kernel(const float* __restrict__ src, long long ldb, __nv_bfloat16* __restrict__ dst,
                   long long K, long long N) {
  __shared__ float tile[32][33];
  const long long k0 = (long long)blockIdx.y * 32, n0 = (long long)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8)
    tile[r][tx] = (k0 + r < K && n0 + tx < N) ? src[(k0 + r) * ldb + n0 + tx] : 0.f;
  __syncthreads();
  for (int r = ty; r < 32; r += 8)
    if (n0 + r < N && k0 + tx < K) dst[(n0 + r) * K + k0 + tx] = __float2bfloat16_rn(tile[tx][r]);
}

}  // namespace

// Re-laying a kn4 B into a workspace of 4*K*N bytes.  relaid_desc() says whether that pays off
// for this descriptor and returns the descriptor of the equivalent plain-layout GEMM over `ws`
// together with the form the weight has to take there (1 = [N,K], 2 = [K,N]); relay_kn4() runs
// the conversion.  Kept apart so that a caller that owns a cache of constants converts once.
int relaid_desc(const annc_gemm_desc& d, void* ws, size_t ws_bytes, annc_gemm_desc* plain) {
  if (d.b_format != ANNC_B_KN4 || !ws || d.batch != 1) return 0;
  if (ws_bytes < (size_t)d.k * (size_t)d.n * sizeof(float)) return 0;
  if ((reinterpret_cast<uintptr_t>(ws) & 15) || (d.n & 3) || d.m < 64) return 0;
  if (d.k >= (1LL << 31) || d.n >= (1LL << 31)) return 0;
  *plain = d;
  plain->b = static_cast<const float*>(ws);
  plain->b_format = ANNC_B_PLAIN;
  plain->ldb = d.n;
  plain->workspace = nullptr;
  plain->workspace_bytes = 0;
  // Re-laid as [N,K] the weight takes the K-major TMA route (one 16 KB box per stage), the
  // fastest one; [K,N] is the fallback when K rows would not be 16-byte pitched.
  if ((d.k & 3) == 0 && (d.k + 31) / 32 <= 65535) {
    annc_gemm_desc t = *plain;
    t.trans_b = 1;
    t.ldb = d.k;
    if (pair_supported(t, ANNC_MATH_TF32) && use_pair(t, ANNC_MATH_TF32)) {
      *plain = t;
      return 1;
    }
  }
  if (!tc_supported(*plain, ANNC_MATH_TF32)) return 0;
  return 2;
}

void relay_kn4(const float* packed, float* ws, long long k, long long n, int form, cudaStream_t s) {
  if (form == 1) {
    dim3 grid((unsigned)((n + 31) / 32), (unsigned)((k + 31) / 32));
    kn4_unpack_transposed_kernel<<<grid, 256, 0, s>>>(packed, ws, k, n);
  } else {
    dim3 grid((unsigned)((n / 4 + 255) / 256), (unsigned)(k < 1024 ? k : 1024));
    kn4_unpack_chunks_kernel<<<grid, 256, 0, s>>>(packed, ws, (int)k, (int)n);
  }
}

static bool unpack_kn4_into_workspace(const annc_gemm_desc& d, cudaStream_t s, annc_gemm_desc* plain) {
  const int form = relaid_desc(d, d.workspace, d.workspace_bytes, plain);
  if (!form) return false;
  relay_kn4(d.b, static_cast<float*>(d.workspace), d.k, d.n, form, s);
  return true;
}

}  // namespace gemm
}  // namespace annc

using namespace annc;

extern "C" {

int annc_gemm_run(const annc_gemm_desc* desc, void* stream) {
  ANNC_REQUIRE(desc, ANNC_ERR_INVALID_ARGUMENT, "gemm: null descriptor");
  ANNC_TRY(gemm::validate(*desc));
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int math = gemm::pick_math(*desc);
  if (desc->math != ANNC_MATH_AUTO && desc->math != math)
    return fail(ANNC_ERR_UNSUPPORTED, "gemm: shape not supported by the requested math mode");
  if (math == ANNC_MATH_FP32) {
    if (desc->io_flags != 0)
      return fail(ANNC_ERR_UNSUPPORTED, "gemm: io_flags need a tensor-core route this shape does not fit");
    return gemm::run_simt(*desc, s);
  }
  annc_gemm_desc plain;
  if (gemm::unpack_kn4_into_workspace(*desc, s, &plain))
    return gemm::use_pair(plain, math) ? gemm::run_pair(plain, math, s) : gemm::run_tc(plain, math, s);
  return gemm::use_pair(*desc, math) ? gemm::run_pair(*desc, math, s) : gemm::run_tc(*desc, math, s);
}

const char* annc_gemm_kernel_name(const annc_gemm_desc* desc) {
  if (!desc) return "";
  return gemm::route_name(*desc);
}

int annc_cast_bf16_dev(const float* src, void* dst_bf16, int64_t n, void* stream) {
  ANNC_REQUIRE(src && dst_bf16 && n >= 0, ANNC_ERR_INVALID_ARGUMENT, "cast: bad arguments");
  if (n == 0) return ANNC_OK;
  long long g = (n + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  gemm::cast_bf16_kernel<<<(unsigned)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<__nv_bfloat16*>(dst_bf16), n);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_bf16_weight_dev(const float* b_kn, int64_t ldb, void* b_nk_bf16, int64_t k, int64_t n,
                         void* stream) {
  ANNC_REQUIRE(b_kn && b_nk_bf16 && k >= 1 && n >= 1 && ldb >= n, ANNC_ERR_INVALID_ARGUMENT,
               "bf16 weight: bad arguments");
  dim3 grid((unsigned)((n + 31) / 32), (unsigned)((k + 31) / 32));
  ANNC_REQUIRE(grid.y <= 65535, ANNC_ERR_UNSUPPORTED, "bf16 weight: k too large");
  gemm::bf16_weight_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      b_kn, ldb, static_cast<__nv_bfloat16*>(b_nk_bf16), k, n);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_kn4_pack_dev(const float* b_kn, float* b_packed, int64_t k, int64_t n, void* stream) {
  ANNC_REQUIRE(b_kn && b_packed && b_kn != b_packed, ANNC_ERR_INVALID_ARGUMENT, "kn4: bad buffers");
  if (k * n <= 0) return ANNC_OK;
  long long g = (k * n + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  gemm::kn4_convert_kernel<<<(unsigned)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      b_kn, b_packed, k, n, 1);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int annc_kn4_unpack_dev(const float* b_packed, float* b_kn, int64_t k, int64_t n, void* stream) {
  ANNC_REQUIRE(b_kn && b_packed && b_kn != b_packed, ANNC_ERR_INVALID_ARGUMENT, "kn4: bad buffers");
  if (k * n <= 0) return ANNC_OK;
  long long g = (k * n + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  gemm::kn4_convert_kernel<<<(unsigned)g, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      b_packed, b_kn, k, n, 0);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int64_t annc_kn4_offset(int64_t K, int64_t N, int64_t k, int64_t n) {
  if (k < 0 || n < 0 || k >= K || n >= N) return -1;
  return kn4::offset(K, N, k, n);
}

int annc_KPFusedBatchMatMulAddSigmoid(const annc_tensor* lhs, const annc_tensor* rhs,
                                      const annc_tensor* bias, annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(lhs && rhs && bias && alloc, ANNC_ERR_INVALID_ARGUMENT, "null argument");
  ANNC_REQUIRE(lhs->rank == 3, ANNC_ERR_INVALID_ARGUMENT, "lhs must be rank 3");
  ANNC_REQUIRE(rhs->rank == 2 || rhs->rank == 3, ANNC_ERR_INVALID_ARGUMENT, "rhs must be rank 2 or 3");
  ANNC_REQUIRE(bias->rank <= 3, ANNC_ERR_INVALID_ARGUMENT, "bias rank must be <= 3");
  const int64_t batch = lhs->dims[0], m = lhs->dims[1], k = lhs->dims[2];
  const bool rhs_batched = rhs->rank == 3;
  ANNC_REQUIRE(!rhs_batched || rhs->dims[0] == batch, ANNC_ERR_INVALID_ARGUMENT,
               "lhs/rhs batch mismatch");
  ANNC_REQUIRE(rhs->dims[rhs_batched ? 1 : 0] == k, ANNC_ERR_INVALID_ARGUMENT,
               "lhs/rhs contracting dim mismatch");
  const int64_t n = rhs->dims[rhs_batched ? 2 : 1];
  const int64_t out_dims[3] = {batch, m, n};
  float* out = static_cast<float*>(alloc(ctx, 0, ANNC_F32, 3, out_dims));
  // BuildBiasInfo (fused_batchmatmul_add_sigmoid.cc:197-214)
  int64_t bd[3] = {1, 1, 1};
  for (int i = 0; i < bias->rank; ++i) bd[3 - bias->rank + i] = bias->dims[i];
  ANNC_REQUIRE((bd[0] == 1 || bd[0] == batch) && (bd[1] == 1 || bd[1] == m) &&
                   (bd[2] == 1 || bd[2] == n),
               ANNC_ERR_INVALID_ARGUMENT, "bias shape is not broadcast-compatible");
  gemm::BiasBroadcast bb;
  bb.s2 = bd[2] == 1 ? 0 : 1;
  bb.s1 = bd[1] == 1 ? 0 : bd[2];
  bb.s0 = bd[0] == 1 ? 0 : bd[1] * bd[2];
  if (batch * m * n == 0) return ANNC_OK;
  ANNC_REQUIRE(out, ANNC_ERR_INTERNAL, "output allocation failed");
  Call call;
  annc_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.m = m;
  d.n = n;
  d.k = k;
  d.batch = batch;
  d.lda = k;
  d.ldb = n;
  d.ldc = n;
  d.stride_a = m * k;
  d.stride_b = rhs_batched ? k * n : 0;
  d.stride_c = m * n;
  d.alpha = 1.0f;
  d.beta = 0.0f;
  d.a = call.in((const float*)lhs->data, (size_t)numel(*lhs));
  d.b = call.in((const float*)rhs->data, (size_t)numel(*rhs));
  d.bias = call.in((const float*)bias->data, (size_t)numel(*bias));
  d.c = call.out(out, (size_t)(batch * m * n));
  d.activation = ANNC_ACT_SIGMOID;
  d.math = ANNC_MATH_FP32;  // the reference test asks for 1e-5
  if (call.status() != ANNC_OK) return call.status();
  ANNC_TRY(gemm::run_simt(d, call.stream(), &bb));
  return call.finish();
}

}  // extern "C"

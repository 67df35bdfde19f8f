// DLRM dot interaction on the tensor cores (TF32): out[b] = [ Z[b,0,:] | strict lower
// triangle of Z[b] Z[b]^T | 0 padding ], Z f32[batch, F, 64].
//
// A tile is SPT = 128 / F consecutive samples = R = SPT * F rows of the [batch*F, 64]
// matrix.  One TMA box per 32-float half of the rows lands in a 128-byte-swizzled stage;
// the same stage is both the A and the B operand of UMMA 128x128x8 (kind::tf32, both
// K-major), eight instructions per tile, so the 128x128 accumulator holds every pairwise
// dot product of the tile's rows and the wanted ones are the diagonal F x F blocks.
// Rows R..127 of a stage are never written; whatever they hold only reaches accumulator
// rows and columns that are not read.
//
// Persistent CTAs (one per SM): warp 0 TMA producer over a 2-stage ring, warp 1 MMA
// issuer with two TMEM accumulators in ping-pong, warps 2-9 two epilogue groups of four
// warps, group g taking the tiles that use accumulator g: tcgen05.ld of the needed column
// chunks into the group's padded shared-memory copy of the accumulator, then the group's four
// warps together write the tile's output rows contiguously (row 0 of every sample comes
// from global memory unrounded, the products are TF32 x TF32 with fp32 sums).  The epilogue
// is the longest stage of a tile, so two of them run side by side.
// The kernel is bound by HBM (F*64*4 bytes read and (64 + F(F-1)/2)*4 written per sample).
// All mbarrier waits are bounded (tc_ptx.cuh).
#include <cstring>

#include "common.h"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace annc {
namespace {

using namespace annc::tc;

constexpr int ID = 64;              // embedding dim
constexpr int I_STAGES = 2;
constexpr int I_BOX = 128 * 128;    // bytes reserved per 32-float half (128 rows x 128 B)
constexpr int I_STAGE = 2 * I_BOX;
constexpr int I_LD = 132;           // padded accumulator row in shared memory (floats)
constexpr int I_THREADS = 320;     // producer, MMA issuer, two epilogue groups of 128
// Row-0 floats each epilogue thread carries per tile: samples_per_tile * 64 / 128, rounded up
// to the template instance (2 covers F >= 26, the DLRM case; 32 covers F = 2).
constexpr int I_DSM = 128 * I_LD * 4;  // one group's accumulator copy
constexpr size_t I_SMEM = 1024 + (size_t)I_STAGES * I_STAGE + 2 * I_DSM + 1024 + 256;

__device__ int g_inter_error = 0;

struct InterParams {
  const float* z;
  float* out;
  long long batch, out_stride;
  int F, spt, rows, tri;
  long long tiles;
};

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void epi_sync(int group) {  // the 128 threads of one epilogue group
  asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory");
}

template <int ROW0_PER_THREAD>
__global__ void __launch_bounds__(I_THREADS, 1)
dot_interaction_tc_kernel(const __grid_constant__ CUtensorMap tmap, InterParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  float* dsm_all = reinterpret_cast<float*>(gen + I_STAGES * I_STAGE);
  uint8_t* pair_i = gen + I_STAGES * I_STAGE + 2 * I_DSM;
  uint8_t* pair_j = pair_i + 512;
  const uint32_t bars = base + I_STAGES * I_STAGE + 2 * I_DSM + 1024;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * I_STAGES;
  const uint32_t bar_tfull = bars + 16 * I_STAGES, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + I_STAGES * I_STAGE + 2 * I_DSM +
                                                    1024 + 16 * I_STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_fail_all = reinterpret_cast<volatile int*>(tmem_slot + 2);  // one word per group

  if (*reinterpret_cast<volatile int*>(&g_inter_error) != 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < I_STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    epi_fail_all[0] = 0;
    epi_fail_all[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int e = threadIdx.x; e < p.tri; e += I_THREADS) {  // pair e -> (i, j), j < i, row-major
    int i = 1, rem = e;
    while (rem >= i) { rem -= i; ++i; }
    pair_i[e] = (uint8_t)i;
    pair_j[e] = (uint8_t)rem;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)), "r"(256u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t box_bytes = (uint32_t)p.rows * 128u;

  if (warp == 0) {
    if (lane == 0) {
      long long li = 0;
      for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++li) {
        const int s = (int)(li % I_STAGES);
        const uint32_t ph = (uint32_t)(li / I_STAGES) & 1u;
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, &g_inter_error)) break;
        const uint32_t st = base + s * I_STAGE;
        mbar_expect_tx(bar_full + 8 * s, 2 * box_bytes);
        tma_load_2d(st, &tmap, 0, (int)(t * p.rows), bar_full + 8 * s);
        tma_load_2d(st + I_BOX, &tmap, 32, (int)(t * p.rows), bar_full + 8 * s);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (16u << 17) | (8u << 24);
      long long li = 0;
      for (long long t = blockIdx.x; t < p.tiles; t += gridDim.x, ++li) {
        const int s = (int)(li % I_STAGES), buf = (int)(li & 1);
        const uint32_t ph = (uint32_t)(li / I_STAGES) & 1u, tph = (uint32_t)(li >> 1) & 1u;
        if (!mbar_wait(bar_tempty + 8 * buf, tph ^ 1u, abort_flag, &g_inter_error)) break;
        if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, &g_inter_error)) break;
        tc_fence_after();
        const uint32_t st = base + s * I_STAGE;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t a = st + (kk >> 2) * I_BOX + (kk & 3) * 32;
          const uint64_t d = smem_desc(a, 16, 1024, 2);
          umma_tf32(tmem_base + buf * 128, d, d, idesc, kk != 0 ? 1u : 0u);
        }
        umma_commit(bar_empty + 8 * s);
        umma_commit(bar_tfull + 8 * buf);
      }
    }
  } else {
    const int group = (warp - 2) >> 2;                // accumulator and tiles of this group
    const int q = warp & 3, te = (threadIdx.x - 64) & 127;
    float* dsm = dsm_all + group * (I_DSM / 4);
    volatile int* epi_fail = epi_fail_all + group;
    const int row_lo = 32 * q;
    // columns this warp's rows need: the diagonal blocks of the samples they belong to
    int c_lo = 0, c_hi = 0;
    if (row_lo < p.rows) {
      const int row_hi = min(row_lo + 31, p.rows - 1);
      c_lo = (row_lo / p.F) * p.F;
      c_hi = (row_hi / p.F + 1) * p.F;
    }
    long long li = group;
    for (long long t = blockIdx.x + (long long)group * gridDim.x; t < p.tiles;
         t += 2LL * gridDim.x, li += 2) {
      const int buf = group;
      const uint32_t tph = (uint32_t)(li >> 1) & 1u;
      const long long b0 = t * p.spt;
      float row0[ROW0_PER_THREAD];
#pragma unroll
      for (int r = 0; r < ROW0_PER_THREAD; ++r) {  // unrounded copy of Z[b, 0, :]
        const int idx = te + 128 * r;
        const int s = idx / ID, col = idx - s * ID;
        row0[r] = (s < p.spt && b0 + s < p.batch) ? __ldg(p.z + (b0 + s) * p.F * ID + col) : 0.f;
      }
      // All four warps leave together: a warp that gave up still joins the barrier.
      const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * buf, tph, abort_flag,
                                                        &g_inter_error)) != 0;
      if (!ok) *epi_fail = 1;
      epi_sync(group);
      if (*epi_fail) break;  // written before the barrier by epilogue warps only: same answer for all
      tc_fence_after();
#pragma unroll 1
      for (int c0 = 0; c0 < 128; c0 += 32) {
        if (c0 + 32 <= c_lo || c0 >= c_hi) continue;  // warp-uniform
        uint32_t r[32];
        tmem_ld32(tmem_base + buf * 128 + ((uint32_t)row_lo << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        float* drow = dsm + (row_lo + lane) * I_LD + c0;
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(drow + j) =
              make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                          __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);  // accumulator may be overwritten
      epi_sync(group);
      // Output rows of the tile's samples.  Triangle: pair index outer (its (i, j) is read
      // once), sample inner; for one sample consecutive threads write consecutive floats.
      for (int pe = te; pe < p.tri; pe += 128) {
        const int pi = pair_i[pe], pj = pair_j[pe];
        for (int s = 0; s < p.spt; ++s) {
          const long long b = b0 + s;
          if (b >= p.batch) break;
          p.out[b * p.out_stride + ID + pe] = dsm[(s * p.F + pi) * I_LD + s * p.F + pj];
        }
      }
      // Row 0 of every sample (loaded before the wait on the accumulator) and the padding.
#pragma unroll
      for (int r = 0; r < ROW0_PER_THREAD; ++r) {
        const int idx = te + 128 * r;
        const int s = idx / ID, col = idx - s * ID;
        if (s < p.spt && b0 + s < p.batch) p.out[(b0 + s) * p.out_stride + col] = row0[r];
      }
      const int pad = (int)p.out_stride - ID - p.tri;
      for (int e = te; e < p.spt * pad; e += 128) {
        const int s = e / pad, col = ID + p.tri + (e - s * pad);
        if (b0 + s < p.batch) p.out[(b0 + s) * p.out_stride + col] = 0.f;
      }
      epi_sync(group);  // dsm is rewritten by the next tile
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u)
                 : "memory");
  }
}

}  // namespace

// Launch; returns ANNC_ERR_UNSUPPORTED when the shape does not fit this kernel.
int dot_interaction_tc(const float* z, int64_t batch, int F, int dim, int64_t z_stride, float* out,
                       int64_t out_stride, cudaStream_t s) {
  if (dim != ID || F < 2 || F > 32 || z_stride != (int64_t)F * ID ||
      (reinterpret_cast<uintptr_t>(z) & 15) != 0 || batch * F >= (1LL << 31) ||
      out_stride >= (1 << 20))
    return ANNC_ERR_UNSUPPORTED;
  static bool attr_set_dev[kMaxDevices] = {};
  bool& attr_set = attr_set_dev[device_slot()];
  if (!attr_set) {
    ANNC_CUDA(cudaFuncSetAttribute(dot_interaction_tc_kernel<2>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)I_SMEM));
    ANNC_CUDA(cudaFuncSetAttribute(dot_interaction_tc_kernel<8>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)I_SMEM));
    ANNC_CUDA(cudaFuncSetAttribute(dot_interaction_tc_kernel<32>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)I_SMEM));
    attr_set = true;
  }
  InterParams p;
  memset(&p, 0, sizeof(p));
  p.z = z;
  p.out = out;
  p.batch = batch;
  p.out_stride = out_stride;
  p.F = F;
  p.spt = 128 / F;
  p.rows = p.spt * F;
  p.tri = F * (F - 1) / 2;
  p.tiles = (batch + p.spt - 1) / p.spt;
  CUtensorMap tm;
  ANNC_TRY(tc::make_map(&tm, z, batch * F, ID, ID, p.rows, false));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const unsigned grid = (unsigned)(p.tiles < sms ? p.tiles : sms);
  const int need = (p.spt * ID + 127) / 128;
  if (need <= 2) dot_interaction_tc_kernel<2><<<grid, I_THREADS, I_SMEM, s>>>(tm, p);
  else if (need <= 8) dot_interaction_tc_kernel<8><<<grid, I_THREADS, I_SMEM, s>>>(tm, p);
  else dot_interaction_tc_kernel<32><<<grid, I_THREADS, I_SMEM, s>>>(tm, p);
  ANNC_CUDA(cudaGetLastError());
  return ANNC_OK;
}

int dot_interaction_error_flag(int* flag) {
  ANNC_CUDA(cudaMemcpyFromSymbol(flag, g_inter_error, sizeof(int)));
  return ANNC_OK;
}

}  // namespace annc

// Persistent CTA-pair GEMM on the 5th-generation tensor cores (tcgen05, cta_group::2).
//
//   C[M,N] = epilogue(alpha * A[M,K] * B + beta * C + addend + bias)
//
// Two CTAs of a cluster own one 256 x 256 tile of C: CTA r holds rows 128 r .. 128 r + 127 of
// the accumulator in its tensor memory and loads, per k-step, its own 128 rows of A and its
// own 128 columns of B (32 KB per CTA per 128-byte k-step, half of what a single-CTA 128 x 128
// tile moves per flop; the MMA of the leader CTA reads both halves of B from the two shared
// memories).  No load is multicast.  TF32 takes fp32 operands as they lie in memory (B as [N,K]
// or [K,N]); BF16 takes bf16 A [M,K] and B [N,K].
//
//   warp 0   TMA producer of this CTA's operand halves; every load counts on the leader's
//            "full" barrier of the stage (cp.async.bulk.tensor ... cta_group::2)
//   warp 1   allocates tensor memory for the pair; in the leader one thread issues the MMAs
//            (UMMA 256 x 256 x {8,16}), commits to the "empty" barrier of both CTAs and, after
//            the last k-step of a tile, to the "accumulator full" barrier of both CTAs
//   warps 2-9  epilogue, two warps per 32 accumulator rows (128 columns each): tcgen05.ld of a
//            32 x 32 chunk (the next chunk's load already in flight), transpose through a
//            swizzled shared-memory tile, then scale / addend / bias / activation and stores
//            in whole 128-byte lines; or a thread-per-row softmax.  Each warp then releases
//            the accumulator to the leader
//
// The kernel is persistent (one pair per two SMs, tiles taken round robin) and the accumulator
// is double-buffered in the 512 tensor-memory columns, so the epilogue of tile i runs under
// the main loop of tile i + 1.  Every wait is bounded (about a second): a role that gives up
// raises the error word read by annc_gemm_check and leaves; all roles meet at the end, where
// tensor memory is freed.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdint>
#include <cstring>

#include "common.h"
#include "gemm.h"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace annc {
namespace gemm {

int* gemm_error_word();  // device address of the tcgen05 GEMM error word (gemm_tc.cu)

namespace {

using namespace annc::tc;

constexpr int PM = 128;           // accumulator rows per CTA
constexpr int PN = 256;           // tile columns (each CTA loads 128 of them)
constexpr int P_A_BYTES = 16384;  // 128 rows x 128 bytes
constexpr int P_B_BYTES = 16384;  // 128 columns x 128 bytes
constexpr int P_STAGE = P_A_BYTES + P_B_BYTES;
constexpr int P_STAGES = 6;
constexpr int P_THREADS = 320;      // producer, MMA issuer, eight epilogue warps
constexpr int P_TMEM_COLS = 512;
constexpr int P_EPI_WARPS = 8;                       // two per TMEM lane quadrant, 128 columns each
constexpr int P_STG_BYTES = P_EPI_WARPS * 32 * 32 * 4;  // one swizzled 32 x 32 chunk per epilogue warp
constexpr size_t P_SMEM = 1024 + (size_t)P_STAGES * P_STAGE + 256 + P_STG_BYTES;

struct PairParams {
  int M, N, K;
  int b_n_major;  // B stored [K,N] (TF32 only)
  void* C;
  long long ldc;
  const float* addend;
  long long ld_addend;
  const float* bias;
  float alpha, beta;
  int act;
  int softmax;  // row softmax over the N <= 256 columns after the epilogue
  int c_bf16;   // C is bf16
  int batched, b_batched;
  long long stride_c, stride_addend;
  int tiles_m, tiles_n;
  long long tiles;
  int* error_word;
};

// Tile order: bands of P_BAND row tiles; inside a band the column tile advances slowest and the
// row tile fastest, so the ~74 tiles in flight at any time cover about 8 row tiles x 9 column
// tiles: every A and B panel they stream is shared through L2 by several pairs instead of
// being fetched from DRAM once per column (or row) tile.
constexpr int P_BAND = 8;
__device__ __forceinline__ void tile_coords(const PairParams& p, long long tile, long long* bz, int* tm,
                                            int* tn) {
  const long long per_batch = (long long)p.tiles_m * p.tiles_n;
  *bz = tile / per_batch;
  const int t2 = (int)(tile - *bz * per_batch);
  const int band = t2 / (P_BAND * p.tiles_n);
  const int rem = t2 - band * (P_BAND * p.tiles_n);
  const int rows = min(P_BAND, p.tiles_m - band * P_BAND);
  *tn = rem / rows;
  *tm = band * P_BAND + (rem - *tn * rows);
}

__device__ __forceinline__ float act_apply(float v, int act) {
  if (act == ANNC_ACT_RELU) return fmaxf(v, 0.0f);
  if (act == ANNC_ACT_SIGMOID) return __fdiv_rn(1.0f, 1.0f + expf(-v));
  return v;
}

// Per-row form of the epilogue (the softmax needs whole rows in one thread): values of one
// 32-column chunk of this thread's row before the activation,
// alpha * acc (+ beta * C) (+ addend) (+ bias).
__device__ __forceinline__ void chunk_values(const PairParams& p, const uint32_t (&r)[32], float (&v)[32],
                                             long long grow, int col0, long long bz, bool row_ok) {
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = p.alpha * __uint_as_float(r[j]);
  if (!row_ok) return;
  if (p.beta != 0.f) {
    if (p.c_bf16) {
      const __nv_bfloat16* c = static_cast<const __nv_bfloat16*>(p.C) + bz * p.stride_c + grow * p.ldc + col0;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += p.beta * __bfloat162float(c[j]);
    } else {
      const float* c = static_cast<const float*>(p.C) + bz * p.stride_c + grow * p.ldc + col0;
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) v[j] += p.beta * c[j];
    }
  }
  if (p.addend) {
    const float* a = p.addend + bz * p.stride_addend + grow * p.ld_addend + col0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) v[j] += __ldg(a + j);
  }
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < p.N) v[j] += __ldg(p.bias + col0 + j);
  }
}

// Staging tile of one epilogue warp: 32 rows x 32 floats, the 16-byte granule g of row r
// stored at granule g ^ (r & 7), so that both the row-wise writes (lane = row) and the
// reads of four rows x 128 bytes are free of bank conflicts beyond the 512 bytes they move.
__device__ __forceinline__ float* stg_at(float* stg, int row, int granule) {
  return stg + row * 32 + ((granule ^ (row & 7)) << 2);
}

// Coalesced half of the epilogue.  The warp has put a 32-row x 32-column chunk into its
// staging tile (row = TMEM lane); here lane l takes columns 4 (l % 8) .. + 3 of rows l / 8 + 4 i,
// so one instruction covers four rows with 128 contiguous bytes each: C and the addend are
// read and C is written in whole lines, all eight loads of a lane in flight together.
// `finalize` adds beta * C, addend, bias (bias4: this lane's four columns, loaded by the
// caller before the accumulator was ready) and the activation; the softmax route stages
// finished values and only stores them.
__device__ __forceinline__ void chunk_store_staged(const PairParams& p, float* stg, int lane,
                                                   long long row0, int col0, long long bz, bool finalize,
                                                   const float (&bias4)[4]) {
  const int g = lane & 7;
  const int c = col0 + g * 4;
  if (c >= p.N) return;
  const bool full4 = c + 3 < p.N;
  const bool c_vec = full4 && ((p.ldc & 3) == 0) && ((p.stride_c & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.C) & 15) == 0);
  const bool a_vec = full4 && ((p.ld_addend & 3) == 0) && ((p.stride_addend & 3) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.addend) & 15) == 0);
  const bool use_beta = finalize && p.beta != 0.f;
  const bool use_add = finalize && p.addend != nullptr;
#pragma unroll
  for (int i0 = 0; i0 < 8; i0 += 4) {  // two batches of four rows: four loads of each kind in flight
  float v[4][4];
  float4 ld_c[4], ld_a[4];
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int i = ii, rl = (lane >> 3) + 4 * (i0 + ii);
    const long long grow = row0 + rl;
    const float4 s4 = *reinterpret_cast<const float4*>(stg_at(stg, rl, g));
    v[i][0] = s4.x; v[i][1] = s4.y; v[i][2] = s4.z; v[i][3] = s4.w;
    ld_c[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    ld_a[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (grow < p.M) {
      const long long coff = bz * p.stride_c + grow * p.ldc + c;
      if (use_beta) {
        if (p.c_bf16) {
          const __nv_bfloat16* cp = static_cast<const __nv_bfloat16*>(p.C) + coff;
          float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (c + e < p.N) t[e] = __bfloat162float(cp[e]);
          ld_c[i] = make_float4(t[0], t[1], t[2], t[3]);
        } else if (c_vec) {
          ld_c[i] = *reinterpret_cast<const float4*>(static_cast<const float*>(p.C) + coff);
        } else {
          const float* cp = static_cast<const float*>(p.C) + coff;
          float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (c + e < p.N) t[e] = cp[e];
          ld_c[i] = make_float4(t[0], t[1], t[2], t[3]);
        }
      }
      if (use_add) {
        const float* ap = p.addend + bz * p.stride_addend + grow * p.ld_addend + c;
        if (a_vec) {
          ld_a[i] = __ldg(reinterpret_cast<const float4*>(ap));
        } else {
          float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (c + e < p.N) t[e] = __ldg(ap + e);
          ld_a[i] = make_float4(t[0], t[1], t[2], t[3]);
        }
      }
    }
  }
#pragma unroll
  for (int ii = 0; ii < 4; ++ii) {
    const int i = ii, rl = (lane >> 3) + 4 * (i0 + ii);
    const long long grow = row0 + rl;
    if (grow >= p.M) continue;
    const long long coff = bz * p.stride_c + grow * p.ldc + c;
    if (finalize) {
      v[i][0] = act_apply(v[i][0] + p.beta * ld_c[i].x + ld_a[i].x + bias4[0], p.act);
      v[i][1] = act_apply(v[i][1] + p.beta * ld_c[i].y + ld_a[i].y + bias4[1], p.act);
      v[i][2] = act_apply(v[i][2] + p.beta * ld_c[i].z + ld_a[i].z + bias4[2], p.act);
      v[i][3] = act_apply(v[i][3] + p.beta * ld_c[i].w + ld_a[i].w + bias4[3], p.act);
    }
    if (p.c_bf16) {
      __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(p.C) + coff;
      if (full4 && ((p.ldc & 3) == 0) && ((p.stride_c & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 7) == 0)) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[i][0], v[i][1]), hi = __floats2bfloat162_rn(v[i][2], v[i][3]);
        uint2 o;
        o.x = *reinterpret_cast<uint32_t*>(&lo);
        o.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(cp) = o;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < p.N) cp[e] = __float2bfloat16_rn(v[i][e]);
      }
    } else {
      float* cp = static_cast<float*>(p.C) + coff;
      if (c_vec) {
        *reinterpret_cast<float4*>(cp) = make_float4(v[i][0], v[i][1], v[i][2], v[i][3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (c + e < p.N) cp[e] = v[i][e];
      }
    }
  }
  }
}

// Row `lane` of the warp's staging tile <- 32 accumulator values scaled by alpha.
__device__ __forceinline__ void stage_row(float* stg, int lane, const uint32_t (&r)[32], float alpha) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<float4*>(stg_at(stg, lane, j)) =
        make_float4(alpha * __uint_as_float(r[4 * j]), alpha * __uint_as_float(r[4 * j + 1]),
                    alpha * __uint_as_float(r[4 * j + 2]), alpha * __uint_as_float(r[4 * j + 3]));
}

// DT 0: TF32 (fp32 elements, 32 per 128-byte k-step, UMMA K = 8); DT 1: BF16 (64, K = 16).
template <int DT, bool SOFTMAX>
__global__ void __launch_bounds__(P_THREADS, 1)
gemm_pair_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b, PairParams p) {
  constexpr int KELTS = DT == 0 ? 32 : 64;  // elements per 128-byte k-step row
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen_base = smem_raw + (base - raw);
  const uint32_t bars = base + P_STAGES * P_STAGE;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * P_STAGES;
  const uint32_t bar_tfull = bars + 16 * P_STAGES, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + P_STAGES * P_STAGE + 16 * P_STAGES + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* staging = reinterpret_cast<float*>(gen_base + P_STAGES * P_STAGE + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const long long pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
  const int KT = (p.K + KELTS - 1) / KELTS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);   // the leader's expect_tx arrival; bytes come from both CTAs
      mbar_init(bar_empty + 8 * s, 1);  // one commit
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);   // one commit
      mbar_init(bar_tempty + 8 * a, 2 * P_EPI_WARPS);  // the epilogue warps of both CTAs
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(smem_u32(tmem_slot), P_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool poisoned = *reinterpret_cast<volatile int*>(p.error_word) != 0;  // an earlier launch gave up

  if (!poisoned) {
    if (warp == 0) {
      // ---------------- producer (both CTAs)
      if (lane == 0) {
        uint32_t kit = 0;
        bool ok = true;
        for (long long tile = pair; tile < p.tiles && ok; tile += pairs) {
          long long bz;
          int tm, tn;
          tile_coords(p, tile, &bz, &tm, &tn);
          const int m0 = tm * (2 * PM) + (int)rank * PM;
          const int n0 = tn * PN + (int)rank * (PN / 2);
          for (int kt = 0; kt < KT; ++kt, ++kit) {
            const int s = kit % P_STAGES;
            const uint32_t ph = (kit / P_STAGES) & 1u;
            ok = mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.error_word);
            if (!ok) break;
            const uint32_t sa = base + s * P_STAGE, sb = sa + P_A_BYTES;
            const uint32_t full_leader = mapa_u32(bar_full + 8 * s, 0);
            if (leader) mbar_expect_tx(bar_full + 8 * s, 2 * P_STAGE);
            const int k0 = kt * KELTS;
            if (p.batched) tma_load_3d_pair(sa, &tmap_a, k0, m0, (int)bz, full_leader);
            else tma_load_2d_pair(sa, &tmap_a, k0, m0, full_leader);
            if (!p.b_n_major) {
              if (p.b_batched) tma_load_3d_pair(sb, &tmap_b, k0, n0, (int)bz, full_leader);
              else tma_load_2d_pair(sb, &tmap_b, k0, n0, full_leader);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) {  // one 32-column x 32-row box per 4 KB block
                if (p.b_batched)
                  tma_load_3d_pair(sb + j * 4096, &tmap_b, n0 + 32 * j, k0, (int)bz, full_leader);
                else
                  tma_load_2d_pair(sb + j * 4096, &tmap_b, n0 + 32 * j, k0, full_leader);
              }
            }
          }
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer (leader CTA only)
      if (leader && lane == 0) {
        // D fp32; A/B tf32 or bf16; A K-major; B K- or N-major; N = 256; M = 256
        const uint32_t fmt = DT == 0 ? 2u : 1u;
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((p.b_n_major ? 1u : 0u) << 16) |
                               ((uint32_t)(PN >> 3) << 17) | ((uint32_t)((2 * PM) >> 4) << 24);
        uint32_t kit = 0, tcount = 0;
        bool ok = true;
        for (long long tile = pair; tile < p.tiles && ok; tile += pairs, ++tcount) {
          const uint32_t acc = tcount & 1u, aph = (tcount >> 1) & 1u;
          ok = mbar_wait(bar_tempty + 8 * acc, aph ^ 1u, abort_flag, p.error_word);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + acc * (uint32_t)PN;
          for (int kt = 0; kt < KT; ++kt, ++kit) {
            const int s = kit % P_STAGES;
            const uint32_t ph = (kit / P_STAGES) & 1u;
            ok = mbar_wait(bar_full + 8 * s, ph, abort_flag, p.error_word);
            if (!ok) break;
            tc_fence_after();
            const uint32_t sa = base + s * P_STAGE, sb = sa + P_A_BYTES;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {  // four UMMA k-steps of 32 bytes per stage
              const uint64_t ad = smem_desc(sa + kk * 32, 16, 1024, 2);
              const uint64_t bd = p.b_n_major ? smem_desc(sb + kk * 1024, 4096, 512, 1)
                                              : smem_desc(sb + kk * 32, 16, 1024, 2);
              if (DT == 0) umma_pair_tf32(tmem_d, ad, bd, idesc, (kt | kk) != 0 ? 1u : 0u);
              else umma_pair_f16(tmem_d, ad, bd, idesc, (kt | kk) != 0 ? 1u : 0u);
            }
            umma_commit_pair(bar_empty + 8 * s);
          }
          if (ok) umma_commit_pair(bar_tfull + 8 * acc);
        }
      }
    } else {
      // ---------------- epilogue (both CTAs): eight warps; warp (q, half) owns TMEM lanes
      // 32 q .. 32 q + 31 and accumulator columns 128 half .. 128 half + 127 (four chunks of 32)
      const int q = warp & 3, half = (warp - 2) >> 2;
      float* stg = staging + (warp - 2) * (32 * 32);
      uint32_t tcount = 0;
      bool ok = true;
      for (long long tile = pair; tile < p.tiles && ok; tile += pairs, ++tcount) {
        const uint32_t acc = tcount & 1u, aph = (tcount >> 1) & 1u;
        long long bz;
        int tm, tn;
        tile_coords(p, tile, &bz, &tm, &tn);
        const long long row0 = (long long)tm * (2 * PM) + rank * PM + q * 32;  // first row of this warp
        const long long grow = row0 + lane;
        const bool row_ok = grow < p.M;
        constexpr int WCOLS = PN / (P_EPI_WARPS / 4);  // columns per epilogue warp (128)
        const int nb = tn * PN + half * WCOLS;  // first column of this warp
        // Bias of the warp's 128 columns, four per lane, fetched once per tile while the MMAs
        // still run: a load per chunk would put an L2 round trip on every chunk's critical path.
        float4 bias_w = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!SOFTMAX && p.bias) {
          const int c = nb + lane * 4;
          if (c + 3 < p.N && (reinterpret_cast<uintptr_t>(p.bias) & 15) == 0) {
            bias_w = __ldg(reinterpret_cast<const float4*>(p.bias + c));
          } else {
            if (c < p.N) bias_w.x = __ldg(p.bias + c);
            if (c + 1 < p.N) bias_w.y = __ldg(p.bias + c + 1);
            if (c + 2 < p.N) bias_w.z = __ldg(p.bias + c + 2);
            if (c + 3 < p.N) bias_w.w = __ldg(p.bias + c + 3);
          }
        }
        ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * acc, aph, abort_flag, p.error_word)) != 0;
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + acc * (uint32_t)PN;
        if (!SOFTMAX) {
          // chunk i + 1 is read from tensor memory (into the registers staging has just
          // freed) while chunk i goes from the staging tile to global memory
          uint32_t ra[32];
          const uint32_t tcol = taddr + (uint32_t)(half * WCOLS);
          if (nb < p.N) tmem_ld32(tcol, ra);
          // not unrolled: the body is large, and unrolled copies of it thrash the instruction cache
#pragma unroll 1
          for (int i = 0; i < WCOLS / 32; ++i) {
            const int c0 = nb + 32 * i;
            if (c0 < p.N) {  // warp-uniform
              float bias4[4];  // this lane's columns of the chunk, from the lane that fetched them
              const int src = 8 * i + (lane & 7);
              bias4[0] = __shfl_sync(0xffffffffu, bias_w.x, src);
              bias4[1] = __shfl_sync(0xffffffffu, bias_w.y, src);
              bias4[2] = __shfl_sync(0xffffffffu, bias_w.z, src);
              bias4[3] = __shfl_sync(0xffffffffu, bias_w.w, src);
              tmem_ld_wait();
              stage_row(stg, lane, ra, p.alpha);
              if (i + 1 < WCOLS / 32 && c0 + 32 < p.N) tmem_ld32(tcol + 32u * (i + 1), ra);
              __syncwarp();
              chunk_store_staged(p, stg, lane, row0, c0, bz, true, bias4);
              __syncwarp();
            }
          }
        } else if (half == 0) {
          // row softmax: one thread per row over all N <= 256 columns, three passes over the
          // row in tensor memory: max, sum of exp, normalised store (warps of half 1 idle)
          const float no_bias[4] = {0.f, 0.f, 0.f, 0.f};
          float mx = -INFINITY, sum = 0.f;
#pragma unroll 1
          for (int pass = 0; pass < 3; ++pass) {
#pragma unroll 1
            for (int c0 = 0; c0 < PN && c0 < p.N; c0 += 32) {
              uint32_t r[32];
              float v[32];
              tmem_ld32(taddr + (uint32_t)c0, r);
              tmem_ld_wait();
              chunk_values(p, r, v, grow, c0, bz, row_ok);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = act_apply(v[j], p.act);
              if (pass == 0) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (c0 + j < p.N) mx = fmaxf(mx, v[j]);
              } else if (pass == 1) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                  if (c0 + j < p.N) sum += expf(v[j] - mx);
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  *reinterpret_cast<float4*>(stg_at(stg, lane, j)) =
                      make_float4(__fdiv_rn(expf(v[4 * j] - mx), sum), __fdiv_rn(expf(v[4 * j + 1] - mx), sum),
                                  __fdiv_rn(expf(v[4 * j + 2] - mx), sum), __fdiv_rn(expf(v[4 * j + 3] - mx), sum));
                __syncwarp();
                chunk_store_staged(p, stg, lane, row0, c0, bz, false, no_bias);
                __syncwarp();
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_u32(bar_tempty + 8 * acc, 0));
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer may read this CTA's shared memory until its last MMA is done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, P_TMEM_COLS);
  }
}

bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Tensor map over [batch,] rows x cols elements (fp32 or bf16), box = `box_cols` x `box_rows`.
int make_map_any(CUtensorMap* map, const void* ptr, bool bf16, long long batch, long long rows,
                 long long cols, long long ld, long long batch_stride, int box_cols, int box_rows,
                 bool n_major) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(ANNC_ERR_CUDA, "cuTensorMapEncodeTiled is not available");
  const size_t es = bf16 ? 2 : 4;
  const bool three = batch > 1;
  const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)ld * es, (cuuint64_t)batch_stride * es};
  const cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1u};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                  three ? 3 : 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  n_major ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ANNC_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return ANNC_OK;
}

}  // namespace

bool pair_supported(const annc_gemm_desc& d, int math) {
  const int io = d.io_flags;
  const bool bf16 = math == ANNC_MATH_BF16;
  if (math != ANNC_MATH_TF32 && !bf16) return false;
  if (d.trans_a || d.b_format != ANNC_B_PLAIN || d.batch < 1 || d.batch > (1 << 20)) return false;
  if (bf16) {
    if ((io & (ANNC_IO_A_BF16 | ANNC_IO_B_BF16)) != (ANNC_IO_A_BF16 | ANNC_IO_B_BF16)) return false;
    if (!d.trans_b) return false;  // bf16 B is [N,K]
  } else if (io & (ANNC_IO_A_BF16 | ANNC_IO_B_BF16)) {
    return false;
  }
  const int es = bf16 ? 2 : 4, per16 = 16 / es;
  if (d.m < 1 || d.n < 8 || d.k < 1) return false;
  if (d.m > (1LL << 30) || d.n > (1LL << 30) || d.k > (1LL << 30)) return false;
  if (!al16(d.a) || (d.lda % per16) || !al16(d.b) || (d.ldb % per16)) return false;
  if (!d.trans_b && (d.n & 3)) return false;
  if (d.batch > 1) {
    if ((d.stride_a % per16) || d.stride_a <= 0 || (d.stride_b % per16) || d.stride_b < 0 ||
        d.stride_c <= 0)
      return false;
  }
  if ((io & ANNC_IO_SOFTMAX) && d.n > PN) return false;
  return true;
}

int run_pair(const annc_gemm_desc& d, int math, cudaStream_t s) {
  if (!pair_supported(d, math)) return fail(ANNC_ERR_UNSUPPORTED, "tcgen05 pair gemm: unsupported shape");
  const bool bf16 = math == ANNC_MATH_BF16;
  static int max_pairs_dev[kMaxDevices][2] = {};
  int (&max_pairs)[2] = max_pairs_dev[device_slot()];
  const bool softmax = (d.io_flags & ANNC_IO_SOFTMAX) != 0;
  auto kern = bf16 ? (softmax ? gemm_pair_tcgen05_kernel<1, true> : gemm_pair_tcgen05_kernel<1, false>)
                   : (softmax ? gemm_pair_tcgen05_kernel<0, true> : gemm_pair_tcgen05_kernel<0, false>);
  static bool attr_done_dev[kMaxDevices][2][2] = {};
  bool (&attr_done)[2][2] = attr_done_dev[device_slot()];
  if (!attr_done[bf16][softmax]) {
    ANNC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P_SMEM));
    attr_done[bf16][softmax] = true;
  }
  if (max_pairs[bf16] == 0) {
    ANNC_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P_SMEM));
    cudaLaunchConfig_t q;
    memset(&q, 0, sizeof(q));
    cudaLaunchAttribute qa[1];
    qa[0].id = cudaLaunchAttributeClusterDimension;
    qa[0].val.clusterDim.x = 2;
    qa[0].val.clusterDim.y = 1;
    qa[0].val.clusterDim.z = 1;
    q.gridDim = dim3(2, 1, 1);
    q.blockDim = dim3(P_THREADS, 1, 1);
    q.dynamicSmemBytes = P_SMEM;
    q.attrs = qa;
    q.numAttrs = 1;
    int n = 0;
    ANNC_CUDA(cudaOccupancyMaxActiveClusters(&n, kern, &q));
    if (n < 1) return fail(ANNC_ERR_CUDA, "no CTA pair fits this device");
    max_pairs[bf16] = n;
  }
  const int kelts = bf16 ? 64 : 32;
  const bool batched = d.batch > 1, b_batched = batched && d.stride_b > 0;
  CUtensorMap ta, tb;
  ANNC_TRY(make_map_any(&ta, d.a, bf16, batched ? d.batch : 1, d.m, d.k, d.lda, d.stride_a, kelts, PM, false));
  PairParams p;
  memset(&p, 0, sizeof(p));
  if (d.trans_b) {
    ANNC_TRY(make_map_any(&tb, d.b, bf16, b_batched ? d.batch : 1, d.n, d.k, d.ldb, d.stride_b, kelts,
                          PN / 2, false));
  } else {
    p.b_n_major = 1;
    ANNC_TRY(make_map_any(&tb, d.b, false, b_batched ? d.batch : 1, d.k, d.n, d.ldb, d.stride_b, 32, 32, true));
  }
  p.M = (int)d.m;
  p.N = (int)d.n;
  p.K = (int)d.k;
  p.C = d.c;
  p.ldc = d.ldc;
  p.addend = d.addend;
  p.ld_addend = d.ld_addend;
  p.bias = d.bias;
  p.alpha = d.alpha;
  p.beta = d.beta;
  p.act = d.activation;
  p.softmax = (d.io_flags & ANNC_IO_SOFTMAX) ? 1 : 0;
  p.c_bf16 = (d.io_flags & ANNC_IO_C_BF16) ? 1 : 0;
  p.batched = batched;
  p.b_batched = b_batched;
  p.stride_c = batched ? d.stride_c : 0;
  p.stride_addend = batched ? d.stride_addend : 0;
  p.tiles_m = (int)((d.m + 2 * PM - 1) / (2 * PM));
  p.tiles_n = (int)((d.n + PN - 1) / PN);
  p.tiles = (long long)p.tiles_m * p.tiles_n * d.batch;
  p.error_word = gemm_error_word();
  if (!p.error_word) return fail(ANNC_ERR_CUDA, "gemm error word is not addressable");
  const long long pairs = p.tiles < max_pairs[bf16] ? p.tiles : max_pairs[bf16];
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(P_THREADS, 1, 1);
  cfg.dynamicSmemBytes = P_SMEM;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ANNC_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, p));
  return ANNC_OK;
}

}  // namespace gemm
}  // namespace annc

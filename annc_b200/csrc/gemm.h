// Internal interface of the GEMM core.
#pragma once

#include <cuda_runtime.h>

#include "annc_b200.h"

namespace annc {
namespace gemm {

// bias[b*s0 + i*s1 + j*s2]: the numpy-style broadcast of
// KPFusedBatchMatMulAddSigmoid (fused_batchmatmul_add_sigmoid.cc:197-214).
struct BiasBroadcast {
  long long s0, s1, s2;
};

// CUDA-core fp32 route; takes every shape, both transposes and the kn4 B format.
int run_simt(const annc_gemm_desc& d, cudaStream_t s, const BiasBroadcast* bb = nullptr);

// tcgen05 route: whether the descriptor fits, and the launch.
bool tc_supported(const annc_gemm_desc& d, int math);
int run_tc(const annc_gemm_desc& d, int math, cudaStream_t s);

// Persistent CTA-pair tcgen05 kernel (TF32 with fp32 operands, BF16 with bf16 operands).
bool pair_supported(const annc_gemm_desc& d, int math);
int run_pair(const annc_gemm_desc& d, int math, cudaStream_t s);

// A kn4-packed B re-laid into `ws` (4*K*N bytes): relaid_desc returns 0 when that does not
// pay off, else the form the weight takes in ws (1 = [N,K], 2 = [K,N]) and fills `plain`
// with the equivalent plain-layout descriptor; relay_kn4 runs the conversion.
int relaid_desc(const annc_gemm_desc& d, void* ws, size_t ws_bytes, annc_gemm_desc* plain);
void relay_kn4(const float* packed, float* ws, long long k, long long n, int form, cudaStream_t s);
// Device-side error word of the tensor-core kernels (a bounded wait that ran out).
int read_error_flag(int* flag);

// Picks the route the way annc_gemm_run does; returns a static name.
const char* route_name(const annc_gemm_desc& d);

}  // namespace gemm
}  // namespace annc

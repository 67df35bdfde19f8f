// TEST INFRASTRUCTURE ONLY.  Compiles the reference's own custom-call bodies into
// oracle/_ref/libannc_xla_ref.so: __matmul, __batch_matmul, __matmul_add, __matmul_add_relu
// (annc/service/cpu/gemm_rewriter.cc:161-281), __pooling (annc/service/cpu/graph_opt.cc:131-176)
// and __reduce_mean (annc/service/cpu/reduce_rewriter.cc:31-46), and the sequential runtime symbols
// __xla_cpu_runtime_KernelSelectorGEMMSequential, ...Batch3DSequential, ...GEMV,
// ...Batch4DSequential, __xla_cpu_runtime_ArgMaxTask and ...ArgMax3DSequential
// (annc/service/cpu/xla/kernel_selector.cc:31-43, 99-116, 168-178, 234-251, 317-339, 376-389; the
// Parallel variants need Eigen's thread pool and XLA's run options, the MLIR variants an external
// library, and are left out).
//
// The bodies use nothing of XLA: plain pointers, memcpy, std::max, variable-length arrays and
// two CBLAS calls.  oracle/Makefile cuts those line ranges out of the reference files where
// they lie into oracle/_ref/*.inc (never into the repository) and this file supplies what
// they need around them: the CBLAS names, forwarded to function pointers that the Python side
// points at an OpenBLAS (cblas_sgemm / cblas_sasum of the library numpy or scipy bundles: the
// library family the reference links, third_party/repo.bzl:3-12).
#include <algorithm>
#include <cstddef>
#include <cstdint>
#include <cstring>

extern "C" {
typedef enum { CblasRowMajor = 101, CblasColMajor = 102 } CBLAS_LAYOUT;
typedef enum { CblasNoTrans = 111, CblasTrans = 112, CblasConjTrans = 113 } CBLAS_TRANSPOSE;
typedef void (*sgemm_fn)(CBLAS_LAYOUT, CBLAS_TRANSPOSE, CBLAS_TRANSPOSE, int, int, int, float,
                         const float*, int, const float*, int, float, float*, int);
typedef float (*sasum_fn)(int, const float*, int);
typedef void (*sgemv_fn)(CBLAS_LAYOUT, CBLAS_TRANSPOSE, int, int, float, const float*, int, const float*,
                         int, float, float*, int);
static sgemm_fn g_sgemm = nullptr;
static sasum_fn g_sasum = nullptr;
static sgemv_fn g_sgemv = nullptr;
void annc_xla_ref_set_sgemv(void* sgemv) { g_sgemv = reinterpret_cast<sgemv_fn>(sgemv); }
void annc_xla_ref_set_blas(void* sgemm, void* sasum) {
  g_sgemm = reinterpret_cast<sgemm_fn>(sgemm);
  g_sasum = reinterpret_cast<sasum_fn>(sasum);
}
}

static inline void cblas_sgemm(CBLAS_LAYOUT l, CBLAS_TRANSPOSE ta, CBLAS_TRANSPOSE tb, int m, int n,
                               int k, float alpha, const float* a, int lda, const float* b, int ldb,
                               float beta, float* c, int ldc) {
  g_sgemm(l, ta, tb, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}
static inline float cblas_sasum(int n, const float* x, int inc) { return g_sasum(n, x, inc); }
static inline void cblas_sgemv(CBLAS_LAYOUT l, CBLAS_TRANSPOSE ta, int m, int n, float alpha, const float* a,
                               int lda, const float* x, int incx, float beta, float* y, int incy) {
  g_sgemv(l, ta, m, n, alpha, a, lda, x, incx, beta, y, incy);
}

#define ANNC_ENABLED_OPENBLAS 1

namespace xla {
namespace cpu {
#include "_ref/xla_gemm_bodies.inc"
#include "_ref/xla_pooling_body.inc"
#include "_ref/xla_reduce_mean_body.inc"
#include "_ref/xla_kernel_selector_bodies.inc"
}  // namespace cpu
}  // namespace xla

extern "C" {
void annc_ref_matmul(void* out, const void** in) { xla::cpu::__matmul(out, in); }
void annc_ref_batch_matmul(void* out, const void** in) { xla::cpu::__batch_matmul(out, in); }
void annc_ref_matmul_add(void* out, const void** in) { xla::cpu::__matmul_add(out, in); }
void annc_ref_matmul_add_relu(void* out, const void** in) { xla::cpu::__matmul_add_relu(out, in); }
void annc_ref_pooling(void* out, void** in) { xla::cpu::__pooling(out, in); }
void annc_ref_reduce_mean(void* out, const void** in) { xla::cpu::__reduce_mean(out, in); }
void annc_ref_ks_gemm(int trA, int trB, const float* A, const float* B, int M, int N, int K, float alpha,
                      float beta, float* C) {
  xla::cpu::__xla_cpu_runtime_KernelSelectorGEMMSequential(nullptr, trA != 0, trB != 0, A, B, M, N, K, alpha,
                                                           beta, C);
}
void annc_ref_ks_batch3d(int trA, int trB, const float* A, const float* B, int P, int M, int N, int K,
                         float* C) {
  xla::cpu::__xla_cpu_runtime_KernelSelectorBatch3DSequential(nullptr, trA != 0, trB != 0, A, B, P, M, N, K, C);
}
void annc_ref_ks_batch4d(int trA, int trB, const float* A, const float* B, int Q, int P, int M, int N,
                         int K, float* C) {
  xla::cpu::__xla_cpu_runtime_KernelSelectorBatch4DSequential(nullptr, trA != 0, trB != 0, A, B, Q, P, M, N, K,
                                                              C);
}
void annc_ref_ks_gemv(int trA, const float* A, const float* X, int M, int N, float alpha, float beta,
                      float* Y) {
  xla::cpu::__xla_cpu_runtime_KernelSelectorGEMV(nullptr, trA != 0, A, X, M, N, alpha, beta, Y);
}
void annc_ref_ks_argmax3d(int B, int M, int N, float* invals, int32_t* inidxs, float init_value,
                          int32_t init_idx, float* outvals, int32_t* outidxs) {
  xla::cpu::__xla_cpu_runtime_ArgMax3DSequential(nullptr, B, M, N, invals, inidxs, init_value, init_idx,
                                                 outvals, outidxs);
}
}

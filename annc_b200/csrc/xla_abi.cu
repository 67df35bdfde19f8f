// The reference's own entry points: XLA custom-call targets and XLA:CPU runtime
// symbols, with unchanged names, operand order and shape-info operands.  Each
// accepts host or device pointers (see the pointer rule in annc_b200.h).  These
// functions return void, as in the reference; a failure is reported on stderr
// and through annc_last_error(), and the output is left untouched.
#include <cstdio>
#include <cstring>

#include "common.h"
#include "gemm.h"

extern "C" int annc_reduce_mean_dev(float* out, const float* value, int64_t m, int64_t n,
                                    void* stream);

namespace annc {
namespace {

void report(const char* who, int rc) {
  if (rc != ANNC_OK) fprintf(stderr, "[annc_b200] %s failed (%d): %s\n", who, rc, annc_last_error());
}

// Operand roles: in the dots the reference's matchers rewrite, rhs is the weight and the addend
// is the broadcast bias; they are constants of the executable, so they are looked up as such
// (reused even when only constants are cached).  A kn4-packed constant weight is re-laid once
// into the form the TMA-fed route wants and that copy is kept with the weight's mirror: no
// per-call workspace traffic.  Strided-batch operands are activations.
int gemm_host(const char* who, float* out, const float* a, const float* b, const float* addend,
              int64_t batch, int64_t m, int64_t n, int64_t k, bool trA, bool trB, float alpha,
              float beta, int act, int b_format, bool weights = true) {
  if (batch * m * n <= 0) return ANNC_OK;
  Call call;
  annc_gemm_desc d;
  memset(&d, 0, sizeof(d));
  d.trans_a = trA;
  d.trans_b = trB;
  d.m = m;
  d.n = n;
  d.k = k;
  d.batch = batch;
  d.lda = trA ? m : k;
  d.ldb = trB ? k : n;
  d.ldc = n;
  d.ld_addend = n;
  d.stride_a = m * k;
  d.stride_b = k * n;
  d.stride_c = m * n;
  d.stride_addend = m * n;
  d.alpha = alpha;
  d.beta = beta;
  const size_t b_count = (size_t)(batch * k * n);
  d.a = call.in(a, (size_t)(batch * m * k));
  d.b = weights ? call.in_constant(b, b_count) : call.in(b, b_count);
  if (addend) d.addend = weights ? call.in_constant(addend, (size_t)(batch * m * n)) : call.in(addend, (size_t)(batch * m * n));
  d.c = call.out(out, (size_t)(batch * m * n), beta != 0.0f);
  d.activation = act;
  d.b_format = b_format;
  d.math = ANNC_MATH_AUTO;
  if (call.status() != ANNC_OK) return call.status();
  if (b_format == ANNC_B_KN4 && (n & 3) == 0 && batch == 1) {
    const size_t ws_bytes = (size_t)k * (size_t)n * sizeof(float);
    bool fresh = false;
    void* ws = call.derived(b, b_count * sizeof(float), /*tag: re-laid kn4*/ 1, ws_bytes, &fresh);
    annc_gemm_desc plain;
    const int form = ws ? gemm::relaid_desc(d, ws, ws_bytes, &plain) : 0;
    if (form) {
      if (fresh) gemm::relay_kn4(d.b, static_cast<float*>(ws), k, n, form, call.stream());
      d = plain;
    }
  }
  ANNC_TRY(annc_gemm_run(&d, call.stream()));
  ANNC_TRY(call.finish());
  if (call.synced()) {  // a tensor-core CTA that gave up on a bounded wait left invalid output
    int flag = 0;
    if (gemm::read_error_flag(&flag) == ANNC_OK && flag)
      return fail(ANNC_ERR_TIMEOUT, "%s: a tensor-core GEMM wait ran out; the output is not valid", who);
  }
  return ANNC_OK;
}

// Reads `count` leading s64 entries of a shape-info operand
// ([dims..., minor_to_major...], annc/service/hlo_util.h:14-21).
int read_info(const void* p, int count, int64_t* dst) {
  Call call;
  return call.read_host(p, sizeof(int64_t) * count, dst);
}

}  // namespace
}  // namespace annc

using namespace annc;

extern "C" {

void __matmul(void* out, const void** in) {
  int64_t sa[2], sb[2];
  int rc = read_info(in[2], 2, sa);
  if (rc == ANNC_OK) rc = read_info(in[3], 2, sb);
  if (rc == ANNC_OK)
    rc = gemm_host("__matmul", (float*)out, (const float*)in[0], (const float*)in[1], nullptr, 1,
                   sa[0], sb[1], sa[1], false, false, 1.0f, 0.0f, ANNC_ACT_NONE, ANNC_B_PLAIN);
  report("__matmul", rc);
}

void __layout_matmul(void* out, const void** in) {
  int64_t sa[2], sb[2];
  int rc = read_info(in[2], 2, sa);
  if (rc == ANNC_OK) rc = read_info(in[3], 2, sb);
  if (rc == ANNC_OK)
    rc = gemm_host("__layout_matmul", (float*)out, (const float*)in[0], (const float*)in[1],
                   nullptr, 1, sa[0], sb[1], sa[1], false, false, 1.0f, 0.0f, ANNC_ACT_NONE,
                   ANNC_B_KN4);
  report("__layout_matmul", rc);
}

void __batch_matmul(void* out, const void** in) {
  int64_t sa[3], sb[3];
  int rc = read_info(in[2], 3, sa);
  if (rc == ANNC_OK) rc = read_info(in[3], 3, sb);
  if (rc == ANNC_OK)
    rc = gemm_host("__batch_matmul", (float*)out, (const float*)in[0], (const float*)in[1],
                   nullptr, sa[0], sa[1], sb[2], sa[2], false, false, 1.0f, 0.0f, ANNC_ACT_NONE,
                   ANNC_B_PLAIN, /*weights=*/false);
  report("__batch_matmul", rc);
}

// in = {addend[m,n], lhs, rhs, info(addend), info(lhs), info(rhs)}
void __matmul_add(void* out, const void** in) {
  int64_t sa[2], sb[2];
  int rc = read_info(in[4], 2, sa);
  if (rc == ANNC_OK) rc = read_info(in[5], 2, sb);
  if (rc == ANNC_OK)
    rc = gemm_host("__matmul_add", (float*)out, (const float*)in[1], (const float*)in[2],
                   (const float*)in[0], 1, sa[0], sb[1], sa[1], false, false, 1.0f, 0.0f,
                   ANNC_ACT_NONE, ANNC_B_PLAIN);
  report("__matmul_add", rc);
}

// in = {max operand (ignored: the reference clamps at a literal 0), addend, lhs, rhs, 4 x info}
void __matmul_add_relu(void* out, const void** in) {
  int64_t sa[2], sb[2];
  int rc = read_info(in[6], 2, sa);
  if (rc == ANNC_OK) rc = read_info(in[7], 2, sb);
  if (rc == ANNC_OK)
    rc = gemm_host("__matmul_add_relu", (float*)out, (const float*)in[2], (const float*)in[3],
                   (const float*)in[1], 1, sa[0], sb[1], sa[1], false, false, 1.0f, 0.0f,
                   ANNC_ACT_RELU, ANNC_B_PLAIN);
  report("__matmul_add_relu", rc);
}

// in = {axis, value, (unused), shape}; m = shape[0], n = shape[1]
void __reduce_mean(void* out, const void** in) {
  int64_t sh[2];
  int rc = read_info(in[3], 2, sh);
  if (rc == ANNC_OK && sh[1] > 0) {
    Call call;
    const float* v = call.in((const float*)in[1], (size_t)(sh[0] * sh[1]));
    float* o = call.out((float*)out, (size_t)sh[1]);
    rc = call.status();
    if (rc == ANNC_OK) rc = annc_reduce_mean_dev(o, v, sh[0], sh[1], call.stream());
    if (rc == ANNC_OK) rc = call.finish();
  }
  report("__reduce_mean", rc);
}

// in = {arg s64[m,k], mul_out f32[m,k,n], slice_starts s64[3], slice_limits s64[3],
//       info(arg), info(mul_out)}
void __pooling(void* out, void** in) {
  int64_t ia[2], im[3], ss[3], sl[3];
  int rc = read_info(in[4], 2, ia);
  if (rc == ANNC_OK) rc = read_info(in[5], 3, im);
  if (rc == ANNC_OK) rc = read_info(in[2], 3, ss);
  if (rc == ANNC_OK) rc = read_info(in[3], 3, sl);
  const int64_t m = ia[0], k = ia[1], n = im[2];
  if (rc == ANNC_OK && m * n > 0) {
    Call call;
    const int64_t* arg = call.in((const int64_t*)in[0], (size_t)(m * k));
    const float* mo = call.in((const float*)in[1], (size_t)(m * k * n));
    float* o = call.out((float*)out, (size_t)(m * n));
    rc = call.status();
    if (rc == ANNC_OK) rc = annc_pooling_dev(o, arg, mo, m, k, n, ss, sl, call.stream());
    if (rc == ANNC_OK) rc = call.finish();
  }
  report("__pooling", rc);
}

void __xla_cpu_runtime_XnnPackSoftMaxND(const void* /*run_options_ptr*/, void* in, void* out,
                                        int64_t batch_size, int64_t channels) {
  int rc = ANNC_OK;
  if (batch_size * channels > 0) {
    Call call;
    const float* x = call.in((const float*)in, (size_t)(batch_size * channels));
    float* y = call.out((float*)out, (size_t)(batch_size * channels));
    rc = call.status();
    if (rc == ANNC_OK) rc = annc_softmax_dev(x, y, batch_size, channels, call.stream());
    if (rc == ANNC_OK) rc = call.finish();
  }
  report("__xla_cpu_runtime_XnnPackSoftMaxND", rc);
}

#define ANNC_DEF_GEMM(name)                                                                  \
  void __xla_cpu_runtime_KernelSelectorGEMM##name(const void*, bool trA, bool trB,           \
                                                  const float* A, const float* B, int M,     \
                                                  int N, int K, float alpha, float beta,     \
                                                  float* C) {                                \
    report("KernelSelectorGEMM" #name,                                                       \
           gemm_host("KernelSelectorGEMM", C, A, B, nullptr, 1, M, N, K, trA, trB, alpha,    \
                     beta, ANNC_ACT_NONE, ANNC_B_PLAIN));                                    \
  }
ANNC_DEF_GEMM(Sequential)
ANNC_DEF_GEMM(Parallel)
ANNC_DEF_GEMM(MLIR)
#undef ANNC_DEF_GEMM
void __xla_cpu_runtime_KernelSelectorGEMMEmpty(const void*, bool, bool, const float*,
                                               const float*, int, int, int, float, float,
                                               float*) {}

#define ANNC_DEF_B3D(name)                                                                    \
  void __xla_cpu_runtime_KernelSelectorBatch3D##name(const void*, bool trA, bool trB,         \
                                                     const float* A, const float* B, int P,   \
                                                     int M, int N, int K, float* C) {         \
    report("KernelSelectorBatch3D" #name,                                                     \
           gemm_host("KernelSelectorBatch3D", C, A, B, nullptr, P, M, N, K, trA, trB, 1.0f,   \
                     0.0f, ANNC_ACT_NONE, ANNC_B_PLAIN));                                     \
  }
ANNC_DEF_B3D(Sequential)
ANNC_DEF_B3D(Parallel)
ANNC_DEF_B3D(MLIR)
#undef ANNC_DEF_B3D
void __xla_cpu_runtime_KernelSelectorBatch3DEmpty(const void*, bool, bool, const float*,
                                                  const float*, int, int, int, int, float*) {}

#define ANNC_DEF_B4D(name)                                                                    \
  void __xla_cpu_runtime_KernelSelectorBatch4D##name(const void*, bool trA, bool trB,         \
                                                     const float* A, const float* B, int Q,   \
                                                     int P, int M, int N, int K, float* C) {  \
    report("KernelSelectorBatch4D" #name,                                                     \
           gemm_host("KernelSelectorBatch4D", C, A, B, nullptr, (int64_t)Q * P, M, N, K, trA, \
                     trB, 1.0f, 0.0f, ANNC_ACT_NONE, ANNC_B_PLAIN));                          \
  }
ANNC_DEF_B4D(Sequential)
ANNC_DEF_B4D(Parallel)
ANNC_DEF_B4D(MLIR)
#undef ANNC_DEF_B4D
void __xla_cpu_runtime_KernelSelectorBatch4DEmpty(const void*, bool, bool, const float*,
                                                  const float*, int, int, int, int, int,
                                                  float*) {}

static void gemv_host(const char* who, bool trA, const float* A, const float* X, int M, int N,
                      float alpha, float beta, float* Y) {
  int rc = ANNC_OK;
  if (M > 0 && N > 0) {
    Call call;
    const int64_t ny = trA ? N : M, nx = trA ? M : N;
    const float* a = call.in(A, (size_t)M * N);
    const float* x = call.in(X, (size_t)nx);
    float* y = call.out(Y, (size_t)ny, beta != 0.0f);
    rc = call.status();
    if (rc == ANNC_OK) rc = annc_gemv_dev(trA, M, N, alpha, a, x, beta, y, call.stream());
    if (rc == ANNC_OK) rc = call.finish();
  }
  report(who, rc);
}

void __xla_cpu_runtime_KernelSelectorGEMV(const void*, bool trA, const float* A, const float* X,
                                          int M, int N, float alpha, float beta, float* Y) {
  gemv_host("KernelSelectorGEMV", trA, A, X, M, N, alpha, beta, Y);
}
void __xla_cpu_runtime_KernelSelectorGEMVMLIR(const void*, bool trA, const float* A,
                                              const float* X, int M, int N, float alpha,
                                              float beta, float* Y) {
  gemv_host("KernelSelectorGEMVMLIR", trA, A, X, M, N, alpha, beta, Y);
}
void __xla_cpu_runtime_KernelSelectorGEMVEmpty(const void*, bool, const float*, const float*, int,
                                               int, float, float, float*) {}

static void argmax_host(const char* who, int B, int M, int N, float* invals, int32_t* inidxs,
                        float init_value, int32_t init_idx, float* outvals, int32_t* outidxs) {
  int rc = ANNC_OK;
  const int64_t rows = (int64_t)B * M;
  if (rows > 0) {
    Call call;
    const float* v = call.in((const float*)invals, (size_t)(rows * N));
    const int32_t* ix = call.in((const int32_t*)inidxs, (size_t)(rows * N));
    float* ov = call.out(outvals, (size_t)rows);
    int32_t* oi = call.out(outidxs, (size_t)rows);
    rc = call.status();
    if (rc == ANNC_OK)
      rc = annc_argmax_dev(rows, N, v, ix, init_value, init_idx, ov, oi, call.stream());
    if (rc == ANNC_OK) rc = call.finish();
  }
  report(who, rc);
}

void __xla_cpu_runtime_ArgMax3DParallel(const void*, int B, int M, int N, float* invals,
                                        int32_t* inidxs, float init_value, int32_t init_idx,
                                        float* outvals, int32_t* outidxs) {
  argmax_host("ArgMax3DParallel", B, M, N, invals, inidxs, init_value, init_idx, outvals, outidxs);
}
void __xla_cpu_runtime_ArgMax3DSequential(const void*, int B, int M, int N, float* invals,
                                          int32_t* inidxs, float init_value, int32_t init_idx,
                                          float* outvals, int32_t* outidxs) {
  argmax_host("ArgMax3DSequential", B, M, N, invals, inidxs, init_value, init_idx, outvals,
              outidxs);
}
void __xla_cpu_runtime_ArgMax3DEmpty(const void*, int, int, int, float*, int32_t*, float, int32_t,
                                     float*, int32_t*) {}

}  // extern "C"

// C++-linkage twins: the names the reference's generated code and its MLIR lowering
// resolve (install/xla/matmul_lower.patch:65-68 calls _ZN3xla3cpu8__matmulEPvPPKv and
// _ZN3xla3cpu14__batch_matmulEPvPPKv; the kernel-selector functions are declared in
// namespace xla::cpu, annc/service/cpu/xla/kernel_selector.h:94-183).
namespace xla {
namespace cpu {

void __matmul(void* out, const void** in) { ::__matmul(out, in); }
void __layout_matmul(void* out, const void** in) { ::__layout_matmul(out, in); }
void __batch_matmul(void* out, const void** in) { ::__batch_matmul(out, in); }
void __matmul_add(void* out, const void** in) { ::__matmul_add(out, in); }
void __matmul_add_relu(void* out, const void** in) { ::__matmul_add_relu(out, in); }
void __reduce_mean(void* out, const void** in) { ::__reduce_mean(out, in); }
void __pooling(void* out, void** in) { ::__pooling(out, in); }

#define ANNC_CPP_GEMM(name)                                                                     \
  void __xla_cpu_runtime_KernelSelectorGEMM##name(const void* r, bool trA, bool trB,            \
                                                  const float* A, const float* B, int M, int N, \
                                                  int K, float alpha, float beta, float* C) {   \
    ::__xla_cpu_runtime_KernelSelectorGEMM##name(r, trA, trB, A, B, M, N, K, alpha, beta, C);   \
  }
ANNC_CPP_GEMM(Sequential) ANNC_CPP_GEMM(Parallel) ANNC_CPP_GEMM(MLIR) ANNC_CPP_GEMM(Empty)
#undef ANNC_CPP_GEMM
#define ANNC_CPP_B3D(name)                                                                      \
  void __xla_cpu_runtime_KernelSelectorBatch3D##name(const void* r, bool trA, bool trB,         \
                                                     const float* A, const float* B, int P,     \
                                                     int M, int N, int K, float* C) {           \
    ::__xla_cpu_runtime_KernelSelectorBatch3D##name(r, trA, trB, A, B, P, M, N, K, C);          \
  }
ANNC_CPP_B3D(Sequential) ANNC_CPP_B3D(Parallel) ANNC_CPP_B3D(MLIR) ANNC_CPP_B3D(Empty)
#undef ANNC_CPP_B3D
#define ANNC_CPP_B4D(name)                                                                      \
  void __xla_cpu_runtime_KernelSelectorBatch4D##name(const void* r, bool trA, bool trB,         \
                                                     const float* A, const float* B, int Q,     \
                                                     int P, int M, int N, int K, float* C) {    \
    ::__xla_cpu_runtime_KernelSelectorBatch4D##name(r, trA, trB, A, B, Q, P, M, N, K, C);       \
  }
ANNC_CPP_B4D(Sequential) ANNC_CPP_B4D(Parallel) ANNC_CPP_B4D(MLIR) ANNC_CPP_B4D(Empty)
#undef ANNC_CPP_B4D
#define ANNC_CPP_GEMV(name)                                                                     \
  void __xla_cpu_runtime_KernelSelectorGEMV##name(const void* r, bool trA, const float* A,      \
                                                  const float* X, int M, int N, float alpha,    \
                                                  float beta, float* Y) {                       \
    ::__xla_cpu_runtime_KernelSelectorGEMV##name(r, trA, A, X, M, N, alpha, beta, Y);           \
  }
ANNC_CPP_GEMV() ANNC_CPP_GEMV(MLIR) ANNC_CPP_GEMV(Empty)
#undef ANNC_CPP_GEMV
#define ANNC_CPP_ARGMAX(name)                                                                   \
  void __xla_cpu_runtime_ArgMax3D##name(const void* r, int B, int M, int N, float* invals,      \
                                        int32_t* inidxs, float init_value, int32_t init_idx,    \
                                        float* outvals, int32_t* outidxs) {                     \
    ::__xla_cpu_runtime_ArgMax3D##name(r, B, M, N, invals, inidxs, init_value, init_idx,        \
                                       outvals, outidxs);                                       \
  }
ANNC_CPP_ARGMAX(Parallel) ANNC_CPP_ARGMAX(Sequential) ANNC_CPP_ARGMAX(Empty)
#undef ANNC_CPP_ARGMAX

}  // namespace cpu
}  // namespace xla

// The small fused ops that sit next to the pooling ops in a KP-fused embedding subgraph:
// KPFusedEmbeddingPadding{,Fast}, KPFusedEmbeddingActionIdGather, KPFusedSparseReshape,
// KPFusedSparseSelect.  Keeping them on the device lets the whole subgraph stay in HBM.
// Validation order and messages follow the reference kernels.
#include <cstring>
#include <vector>

#include "common.h"

namespace annc {
namespace {

// out[row, col] = col < cols ? params[indices1[indices2[a, b], c], d] : 0 with the flat
// gather index row * cols + col = ((a * i2_1 + b) * i1_1 + c) * p1 + d.
struct ActionParams {
  const float* params;
  const void* idx1;
  const void* idx2;
  float* out;
  long long p0, p1, i1_0, i1_1, n2, cols, pack_size, pack_const;
  int idx1_64, idx2_64;
};

__global__ void action_id_gather_kernel(ActionParams g, int* err) {
  const long long width = g.cols + g.pack_const;
  const long long total = g.pack_size * width;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
    const long long row = e / width, col = e - row * width;
    float v = 0.f;
    if (col < g.cols) {
      const long long f = row * g.cols + col;
      const long long d = f % g.p1, r1 = f / g.p1;
      const long long c = r1 % g.i1_1, ab = r1 / g.i1_1;
      const long long i2 = g.idx2_64 ? ((const long long*)g.idx2)[ab] : (long long)((const int*)g.idx2)[ab];
      if (i2 < 0 || i2 >= g.i1_0) {
        atomicOr(err, 1);
      } else {
        const long long q = i2 * g.i1_1 + c;
        const long long i1 = g.idx1_64 ? ((const long long*)g.idx1)[q] : (long long)((const int*)g.idx1)[q];
        if (i1 < 0 || i1 >= g.p0) atomicOr(err, 1);
        else v = __ldg(g.params + i1 * g.p1 + d);
      }
    }
    g.out[e] = v;
  }
}

// The first gather of the reference runs over every entry of indices1, used later or not:
// an out-of-range entry anywhere fails the op.
__global__ void index_range_kernel(const void* idx, int is64, long long n, long long limit, int* err) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const long long v = is64 ? ((const long long*)idx)[i] : (long long)((const int*)idx)[i];
    if (v < 0 || v >= limit) atomicOr(err, 1);
  }
}

// indices (i, slice[i, col]) of a [rows, pack] sparse tensor re-expressed for shape [o0, o1].
__global__ void sparse_reshape_kernel(const long long* slice, long long rows, long long ncols, int col,
                                      long long in_stride0, long long out_stride0, int identity,
                                      long long* out) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < rows; i += stride) {
    const long long v = slice[i * ncols + col];
    if (identity) {
      out[2 * i] = i;
      out[2 * i + 1] = v;
    } else {
      long long id = i * in_stride0 + v;
      out[2 * i] = id / out_stride0;
      id %= out_stride0;
      out[2 * i + 1] = id;  // stride of the last dim is 1
    }
  }
}

__global__ void sparse_select_kernel(const int* a, const int* b, long long n, int greater, int eq1,
                                     int eq2, float* x, float* y, float* w) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float g = a[i] > greater ? 1.0f : 0.0f;
    const float r1 = b[i] == eq1 ? 1.0f : g;
    const float r2 = b[i] == eq2 ? 1.0f : r1;
    x[i] = (float)a[i];
    y[i] = r2;
    w[2 * i] = r2;
    w[2 * i + 1] = 1.0f;
  }
}

int grid_of(long long n) {
  long long g = (n + 255) / 256;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}

bool is_scalar(const annc_tensor* t) { return t->rank == 0; }
bool is_vector(const annc_tensor* t) { return t->rank == 1; }
bool is_matrix(const annc_tensor* t) { return t->rank == 2; }

// Writes a small host value to an output that may live on the device.
int put_small(Call& call, void* dst, const void* src, size_t bytes) {
  if (call.is_device(dst)) {
    ANNC_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, call.stream()));
    ANNC_CUDA(cudaStreamSynchronize(call.stream()));
  } else {
    if (call.status() != ANNC_OK) return call.status();
    memcpy(dst, src, bytes);
  }
  return ANNC_OK;
}

}  // namespace
}  // namespace annc

using namespace annc;

extern "C" {

int annc_KPFusedEmbeddingPadding(const annc_tensor* origin_shape, const annc_tensor* input,
                                 const annc_tensor* input_rows, const annc_tensor* reshape_sizes,
                                 const annc_tensor* pack, int fast, annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(origin_shape && input && input_rows && reshape_sizes && pack && alloc,
               ANNC_ERR_INVALID_ARGUMENT, "null argument");
  if (!is_vector(origin_shape))
    return fail(ANNC_ERR_INVALID_ARGUMENT, "origin_shape dims must 1D, not rank %d", origin_shape->rank);
  if (numel(*origin_shape) != 2)
    return fail(ANNC_ERR_INVALID_ARGUMENT, "origin_shape NumElements must == 2, not %lld",
                (long long)numel(*origin_shape));
  if (!is_matrix(input)) return fail(ANNC_ERR_INVALID_ARGUMENT, "input dims must 2D, not rank %d", input->rank);
  ANNC_REQUIRE(is_scalar(input_rows), ANNC_ERR_INVALID_ARGUMENT, "input_rows must be a scalar");
  if (!is_vector(reshape_sizes))
    return fail(ANNC_ERR_INVALID_ARGUMENT, "sizes input must be 1-D, not rank %d", reshape_sizes->rank);
  ANNC_REQUIRE(numel(*reshape_sizes) == 2, ANNC_ERR_INVALID_ARGUMENT, "reshape_sizes NumElements must == 2");
  Call call;
  int64_t oshape[2];
  int32_t rows_v, rs[2], pack_v;
  ANNC_TRY(call.read_host(origin_shape->data, sizeof(oshape), oshape));
  ANNC_TRY(call.read_host(input_rows->data, sizeof(rows_v), &rows_v));
  ANNC_TRY(call.read_host(reshape_sizes->data, sizeof(rs), rs));
  ANNC_TRY(call.read_host(pack->data, sizeof(pack_v), &pack_v));
  const int padding_rows = (int32_t)oshape[0] - rows_v;
  const int reshape_cols = rs[1];
  const int64_t output_rows = padding_rows + input->dims[0], output_cols = input->dims[1];
  if (padding_rows < 0)
    return fail(ANNC_ERR_INVALID_ARGUMENT, "Pooling size(%d) is greater than Input size(%d)", rows_v,
                (int32_t)oshape[0]);
  ANNC_REQUIRE(reshape_cols > 0, ANNC_ERR_INVALID_ARGUMENT, "reshape_cols must > 0");
  ANNC_REQUIRE(rs[0] == -1, ANNC_ERR_INVALID_ARGUMENT, "reshape[0] is not -1");
  if (pack_v != output_cols)
    return fail(ANNC_ERR_INVALID_ARGUMENT, "pack(%d) is not equal to embedding dims", pack_v);
  int32_t* out0 = static_cast<int32_t*>(alloc(ctx, 0, ANNC_I32, 0, nullptr));
  ANNC_REQUIRE(out0, ANNC_ERR_INTERNAL, "output allocation failed");
  const int32_t pad32 = padding_rows;
  ANNC_TRY(put_small(call, out0, &pad32, sizeof(pad32)));
  if (output_rows * output_cols % reshape_cols != 0)
    return fail(ANNC_ERR_INVALID_ARGUMENT, "padding cannot reshape to [-1, %d]", reshape_cols);
  const int32_t reshape_rows = (int32_t)(output_rows * output_cols / reshape_cols);
  if (fast) {
    int32_t* out1 = static_cast<int32_t*>(alloc(ctx, 1, ANNC_I32, 0, nullptr));
    ANNC_REQUIRE(out1, ANNC_ERR_INTERNAL, "output allocation failed");
    ANNC_TRY(put_small(call, out1, &reshape_rows, sizeof(reshape_rows)));
    return call.finish();
  }
  const int64_t dims[2] = {reshape_rows, reshape_cols};
  float* out1 = static_cast<float*>(alloc(ctx, 1, ANNC_F32, 2, dims));
  const int64_t total = (int64_t)reshape_rows * reshape_cols;
  ANNC_REQUIRE(out1 || total == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  if (total > 0) {
    // reference: memcpy of input_rows * cols floats, memset of the padding rows
    int64_t live = (int64_t)rows_v * output_cols;
    if (live > numel(*input)) live = numel(*input);
    if (live > total) live = total;
    const float* d_in = call.in((const float*)input->data, (size_t)numel(*input));
    float* d_out = call.out(out1, (size_t)total);
    if (call.status() != ANNC_OK) return call.status();
    if (live > 0)
      ANNC_CUDA(cudaMemcpyAsync(d_out, d_in, (size_t)live * 4, cudaMemcpyDeviceToDevice, call.stream()));
    if (total > live)
      ANNC_CUDA(cudaMemsetAsync(d_out + live, 0, (size_t)(total - live) * 4, call.stream()));
  }
  return call.finish();
}

int annc_KPFusedEmbeddingActionIdGather(const annc_tensor* indices1, const annc_tensor* params,
                                        const annc_tensor* indices2, const annc_tensor* pack_dim,
                                        const annc_tensor* pack, annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(indices1 && params && indices2 && pack_dim && pack && alloc, ANNC_ERR_INVALID_ARGUMENT,
               "null argument");
  ANNC_REQUIRE(is_matrix(indices1), ANNC_ERR_INVALID_ARGUMENT, "indices1 dims must = 2");
  ANNC_REQUIRE(is_matrix(indices2), ANNC_ERR_INVALID_ARGUMENT, "indices2 dims must = 2");
  ANNC_REQUIRE(is_matrix(params), ANNC_ERR_INVALID_ARGUMENT, "params dims must = 2");
  ANNC_REQUIRE(is_scalar(pack_dim), ANNC_ERR_INVALID_ARGUMENT, "pack_dim is scalar");
  ANNC_REQUIRE(is_scalar(pack), ANNC_ERR_INVALID_ARGUMENT, "pack const is scalar");
  Call call;
  cudaStream_t s = call.stream();
  int32_t pack_size = 0, pack_const = 0;
  ANNC_TRY(call.read_host(pack_dim->data, 4, &pack_size));
  ANNC_TRY(call.read_host(pack->data, 4, &pack_const));
  ActionParams g;
  memset(&g, 0, sizeof(g));
  g.p0 = params->dims[0];
  g.p1 = params->dims[1];
  g.i1_0 = indices1->dims[0];
  g.i1_1 = indices1->dims[1];
  g.n2 = numel(*indices2);
  g.idx1_64 = indices1->dtype == ANNC_I64;
  g.idx2_64 = indices2->dtype == ANNC_I64;
  // both gathers run (and range-check every index) before pack_size is looked at
  auto* d_err = static_cast<int*>(call.scratch(sizeof(int)));
  g.params = call.in_constant((const float*)params->data, (size_t)numel(*params));
  g.idx1 = call.in(indices1->data, (size_t)numel(*indices1) * dtype_size(indices1->dtype));
  g.idx2 = call.in(indices2->data, (size_t)g.n2 * dtype_size(indices2->dtype));
  if (call.status() != ANNC_OK) return call.status();
  ANNC_CUDA(cudaMemsetAsync(d_err, 0, sizeof(int), s));
  if (numel(*indices1) > 0)
    index_range_kernel<<<grid_of(numel(*indices1)), 256, 0, s>>>(g.idx1, g.idx1_64, numel(*indices1),
                                                                 g.p0, d_err);
  if (g.n2 > 0) index_range_kernel<<<grid_of(g.n2), 256, 0, s>>>(g.idx2, g.idx2_64, g.n2, g.i1_0, d_err);
  int bits = 0;
  ANNC_TRY(call.read_host(d_err, sizeof(int), &bits));
  ANNC_REQUIRE(bits == 0, ANNC_ERR_INVALID_ARGUMENT, "GatherV2 axis=0: index out of range");
  ANNC_REQUIRE(pack_size > 0, ANNC_ERR_INVALID_ARGUMENT, "pack_size must > 0");
  const int64_t gathered = g.n2 * g.i1_1 * g.p1;
  g.pack_size = pack_size;
  g.pack_const = pack_const;
  g.cols = gathered / pack_size;
  const int64_t dims[2] = {pack_size, g.cols + pack_const};
  float* out = static_cast<float*>(alloc(ctx, 0, ANNC_F32, 2, dims));
  const int64_t total = dims[0] * dims[1];
  ANNC_REQUIRE(out || total == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  if (total > 0) {
    g.out = call.out(out, (size_t)total);
    if (call.status() != ANNC_OK) return call.status();
    action_id_gather_kernel<<<grid_of(total), 256, 0, s>>>(g, d_err);
  }
  return call.finish();
}

int annc_KPFusedSparseReshape(const annc_tensor* slice_input, const annc_tensor* begin,
                              const annc_tensor* new_shape, const annc_tensor* pack_const,
                              annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(slice_input && begin && new_shape && pack_const && alloc, ANNC_ERR_INVALID_ARGUMENT,
               "null argument");
  ANNC_REQUIRE(slice_input->rank == 2, ANNC_ERR_INTERNAL, "slice_input dims must == 2");
  ANNC_REQUIRE(new_shape->rank >= 1 && new_shape->dims[0] == 2, ANNC_ERR_INTERNAL,
               "new_shape dim size must == 2");
  ANNC_REQUIRE(pack_const->rank == 0, ANNC_ERR_INVALID_ARGUMENT, "pack_const must be a scalar");
  ANNC_REQUIRE(begin->rank == 1 && begin->dims[0] == 2, ANNC_ERR_INVALID_ARGUMENT,
               "begin must be 1D with at least 2 elements");
  Call call;
  cudaStream_t s = call.stream();
  int32_t b[2];
  int64_t target[2], pack_v;
  ANNC_TRY(call.read_host(begin->data, sizeof(b), b));
  ANNC_TRY(call.read_host(new_shape->data, sizeof(target), target));
  ANNC_TRY(call.read_host(pack_const->data, sizeof(pack_v), &pack_v));
  const int32_t col = b[1];
  ANNC_REQUIRE(col < slice_input->dims[1] && col >= 0, ANNC_ERR_INTERNAL,
               "begin[1] must < slice_input.dim_size(1)");
  const int64_t rows = slice_input->dims[0], ncols = slice_input->dims[1];
  // ReshapeKp: sparse tensor of shape [rows, pack] to `target` (one -1 allowed)
  const int64_t in_shape[2] = {rows, pack_v};
  const int64_t dense = rows * pack_v;
  int64_t out_shape[2] = {1, 1}, product = 1;
  int unknown = -1;
  for (int d = 0; d < 2; ++d) {
    if (target[d] == -1) {
      if (unknown != -1)
        return fail(ANNC_ERR_INVALID_ARGUMENT, "only one output dimension may be -1, not both %d and %d",
                    unknown, d);
      unknown = d;
    } else {
      if (target[d] < 0)
        return fail(ANNC_ERR_INVALID_ARGUMENT, "size %d must be non-negative, not %lld", d,
                    (long long)target[d]);
      product *= target[d];
      out_shape[d] = target[d];
    }
  }
  if (unknown != -1) {
    ANNC_REQUIRE(product > 0, ANNC_ERR_INVALID_ARGUMENT,
                 "reshape cannot infer the missing input size for an empty tensor unless all "
                 "specified input sizes are non-zero");
    const int64_t missing = dense / product;
    if (product * missing != dense)
      return fail(ANNC_ERR_INVALID_ARGUMENT,
                  "Input to reshape is a SparseTensor with %lld dense values, but the requested shape "
                  "requires a multiple of %lld. input_shape=[%lld,%lld]",
                  (long long)dense, (long long)product, (long long)in_shape[0], (long long)in_shape[1]);
    out_shape[unknown] = missing;
  }
  if (out_shape[0] * out_shape[1] != dense)
    return fail(ANNC_ERR_INVALID_ARGUMENT,
                "Input to reshape is a tensor with %lld dense values, but the requested shape has %lld. "
                "input_shape=[%lld,%lld] output_shape=[%lld,%lld]",
                (long long)dense, (long long)(out_shape[0] * out_shape[1]), (long long)in_shape[0],
                (long long)in_shape[1], (long long)out_shape[0], (long long)out_shape[1]);
  const int identity = out_shape[0] == in_shape[0] && out_shape[1] == in_shape[1];
  const int64_t idims[2] = {rows, 2}, sdims[1] = {2};
  int64_t* out_idx = static_cast<int64_t*>(alloc(ctx, 0, ANNC_I64, 2, idims));
  int64_t* out_shp = static_cast<int64_t*>(alloc(ctx, 1, ANNC_I64, 1, sdims));
  ANNC_REQUIRE(out_shp && (out_idx || rows == 0), ANNC_ERR_INTERNAL, "output allocation failed");
  if (rows > 0) {
    const long long* d_slice = (const long long*)call.in((const int64_t*)slice_input->data, (size_t)(rows * ncols));
    long long* d_out = (long long*)call.out(out_idx, (size_t)(rows * 2));
    if (call.status() != ANNC_OK) return call.status();
    sparse_reshape_kernel<<<grid_of(rows), 256, 0, s>>>(d_slice, rows, ncols, col, pack_v,
                                                        out_shape[1] > 0 ? out_shape[1] : 1, identity,
                                                        d_out);
  }
  ANNC_TRY(put_small(call, out_shp, out_shape, sizeof(out_shape)));
  return call.finish();
}

int annc_KPFusedSparseSelect(const annc_tensor* a, const annc_tensor* b, const annc_tensor* c,
                             const annc_tensor* greater, const annc_tensor* equal1,
                             const annc_tensor* equal2, const annc_tensor* equal3,
                             annc_alloc_fn alloc, void* ctx) {
  ANNC_REQUIRE(a && b && c && greater && equal1 && equal2 && equal3 && alloc, ANNC_ERR_INVALID_ARGUMENT,
               "null argument");
  Call call;
  cudaStream_t s = call.stream();
  int32_t g = 0, e1 = 0, e2 = 0, e3 = 0;
  ANNC_TRY(call.read_host(equal1->data, 4, &e1));
  ANNC_TRY(call.read_host(equal2->data, 4, &e2));
  ANNC_TRY(call.read_host(equal3->data, 4, &e3));  // read and unused, as in the reference
  ANNC_TRY(call.read_host(greater->data, 4, &g));
  ANNC_REQUIRE(numel(*a) == numel(*b), ANNC_ERR_INVALID_ARGUMENT, "Input num elements of a and b must match");
  ANNC_REQUIRE(numel(*a) == numel(*c), ANNC_ERR_INVALID_ARGUMENT, "Input num elements of a and c must match");
  const int64_t n = numel(*a);
  const int64_t d1[2] = {n, 1}, d2[2] = {n, 2};
  float* ox = static_cast<float*>(alloc(ctx, 0, ANNC_F32, 2, d1));
  float* oy = static_cast<float*>(alloc(ctx, 1, ANNC_F32, 2, d1));
  float* ow = static_cast<float*>(alloc(ctx, 2, ANNC_F32, 2, d2));
  ANNC_REQUIRE((ox && oy && ow) || n == 0, ANNC_ERR_INTERNAL, "output allocation failed");
  if (n > 0) {
    const int* da = call.in((const int*)a->data, (size_t)n);
    const int* db = call.in((const int*)b->data, (size_t)n);
    float* dx = call.out(ox, (size_t)n);
    float* dy = call.out(oy, (size_t)n);
    float* dw = call.out(ow, (size_t)(2 * n));
    if (call.status() != ANNC_OK) return call.status();
    sparse_select_kernel<<<grid_of(n), 256, 0, s>>>(da, db, n, g, e1, e2, dx, dy, dw);
  }
  return call.finish();
}

}  // extern "C"

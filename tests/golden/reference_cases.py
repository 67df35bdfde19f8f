"""Known-answer cases transcribed from the reference's own unit tests
(annc/tensorflow/kernels/*_test.cc in the ANNC project).  Each entry cites the
test it comes from.  Used twice: to pin the CPU oracle (no GPU) and as parity
cases for the CUDA path (GPU)."""
import numpy as np

f32, i32, i64 = np.float32, np.int32, np.int64

_SLICE_3x4 = np.array([[1, 2, 2, 2], [1, 1, 2, 3], [2, 2, 3, 4]], i64)
_DATA_4x2 = np.arange(1, 9, dtype=f32).reshape(4, 2)

# embedding_fused_sparse_segment_reduce_test.cc:57-101
SEGMENT_REDUCE = [
    dict(name="TestReduceMean", combiner=1, data=_DATA_4x2, indices=np.array([0, 2, 1], i32),
         slice_input=_SLICE_3x4, begin=np.array([0, 2], i32), begin_1=np.array([1], i32),
         out=np.array([[0, 0], [0, 0], [3, 4], [3, 4]], f32), slice_out=2),
    dict(name="TestReduceSum", combiner=0, data=_DATA_4x2, indices=np.array([0, 2, 1], i32),
         slice_input=_SLICE_3x4, begin=np.array([0, 2], i32), begin_1=np.array([0], i32),
         out=np.array([[0, 0], [0, 0], [6, 8], [3, 4]], f32), slice_out=4),
]

# embedding_fused_sparse_segment_reduce_test.cc:103-202: (mutation, message substring)
SEGMENT_REDUCE_ERRORS = [
    ("begin", np.array([0, 5], i32), "Column index out of range"),
    ("indices", np.array([0, 2], i32), "indices and slice_input.dim_zie(0) should have same size"),
    ("data", _DATA_4x2.reshape(4, 2, 1), "input must be 2-D"),
    ("slice_input", _SLICE_3x4.reshape(3, 4, 1), "slice input must be 2-D"),
    ("begin", np.array([0, 2, 1], i32), "begin must have 2 elements"),
    ("begin_1", np.array([0, 1], i32), "begin_1 must have 1 element"),
]

_DATA_8 = np.arange(1, 9, dtype=f32)
_DATA_5x3 = np.array([[1, 2, 3], [4, 0, 6], [7, 8, 9], [0, 0, 0], [1, 1, 1]], f32)
_SLICE_5x4 = np.array([[1, 2, 2, 2], [1, 1, 2, 3], [2, 2, 3, 4], [1, 2, 3, 3], [2, 2, 4, 4]], i64)

# embedding_fused_sparse_segment_reduce_nonzero_test.cc:56-247
SEGMENT_REDUCE_NONZERO = [
    dict(name="TestReduceMean", combiner=1, data=_DATA_8, indices=np.array([0, 2, 1], i32),
         slice_input=_SLICE_3x4, begin=np.array([0, 2], i32),
         out_shape=np.array([4], i32), out_indices=np.array([[2], [3]], i32),
         out_values=np.array([2, 2], f32)),
    dict(name="TestReduceSum", combiner=0, data=_DATA_8, indices=np.array([0, 2, 1], i32),
         slice_input=_SLICE_3x4, begin=np.array([0, 2], i32),
         out_shape=np.array([4], i32), out_indices=np.array([[2], [3]], i32),
         out_values=np.array([4, 2], f32)),
    dict(name="Test2DReduceSum", combiner=0, data=_DATA_5x3, indices=np.array([0, 2, 1, 4, 3], i32),
         slice_input=_SLICE_5x4, begin=np.array([0, 2], i32),
         out_shape=np.array([5, 3], i32),
         out_indices=np.array([[2, 0], [2, 1], [2, 2], [3, 0], [3, 1], [3, 2]], i32),
         out_values=np.array([8, 10, 12, 5, 1, 7], f32)),
    dict(name="Test2DReduceMean", combiner=1, data=_DATA_5x3, indices=np.array([0, 2, 1, 4, 3], i32),
         slice_input=_SLICE_5x4, begin=np.array([0, 2], i32),
         out_shape=np.array([5, 3], i32),
         out_indices=np.array([[2, 0], [2, 1], [2, 2], [3, 0], [3, 1], [3, 2]], i32),
         out_values=np.array([4, 5, 6, 2.5, 0.5, 3.5], f32)),
    dict(name="Test2DElementWiseZeroFilter", combiner=0,
         data=np.array([[1, 0, 3], [0, 2, 0], [3, 0, 0], [0, 0, 4]], f32),
         indices=np.array([0, 1, 2, 3], i32),
         slice_input=np.array([[9, 0], [9, 0], [9, 1], [9, 1]], i64), begin=np.array([0, 1], i32),
         out_shape=np.array([2, 3], i32),
         out_indices=np.array([[0, 0], [0, 1], [0, 2], [1, 0], [1, 2]], i32),
         out_values=np.array([1, 2, 3, 3, 4], f32)),
]

# embedding_fused_sparse_segment_reduce_nonzero_test.cc:249-318
SEGMENT_REDUCE_NONZERO_ERRORS = [
    ("data", np.arange(1, 9, dtype=f32).reshape(2, 2, 2), "Input data must be a 1-D vector or 2-D matrix"),
    ("slice_input", _SLICE_3x4.reshape(3, 4, 1), "slice input must be 2-D"),
    ("begin", np.array([0, 2, 1], i32), "begin must have 2 elements"),
    ("begin", np.array([0, 4], i32), "Column index out of range"),
    ("indices", np.array([0, 2], i32), "indices and slice_input.dim_size(0) should have same size"),
]

_GATHER_DATA = np.arange(1, 25, dtype=f32).reshape(2, 12)

# embedding_fused_gather_test.cc:111-127
FUSED_GATHER = [
    dict(name="Valid_NormalInput", data=_GATHER_DATA,
         keys=np.array([[1, 1, 3], [0, 1, 5], [1, 0, 7], [0, 1, 9]], i64), begin=np.array([0, 1], i32),
         unique=np.array([1, 0], i64), indices=np.array([0, 0, 1, 0], i32),
         out=np.stack([_GATHER_DATA[1], _GATHER_DATA[0]])),
]

# embedding_fused_gather_test.cc:129-185: (data, keys, begin, message)
FUSED_GATHER_ERRORS = [
    (np.array([1, 2, 3, 4], f32), np.array([[0, 1], [2, 3]], i64), np.array([0, 0], i32),
     "Embedding table shape must be 2D"),
    (np.ones((2, 12), f32), np.array([0, 1, 2, 3], i64), np.array([0, 0], i32),
     "Input key must be 2D"),
    (np.ones((2, 12), f32), np.array([[0, 1], [2, 3]], i64), np.array([0, 2], i32),
     "slice cols out of keys range"),
    (np.ones((2, 12), f32), np.array([[0, 1], [2, 3]], i64), np.array([0, 0], i32),
     "idx out of table range"),
]

# embedding_fused_sparse_dynamic_stitch_test.cc:53-66
DYNAMIC_STITCH = [
    dict(name="TestTwoTables", x=np.array([0, 3, 2, 1], i64),
         tables=[np.array([[1, 2], [3, 4], [5, 6]], f32), np.array([[7, 8], [9, 10]], f32)],
         out=np.array([[1, 2], [9, 10], [3, 4], [7, 8]], f32)),
]

# embedding_fused_sparse_dynamic_stitch_test.cc:68-106: (x, tables, message)
DYNAMIC_STITCH_ERRORS = [
    (np.array([0, 3, 2, 1], i64),
     [np.array([[1, 2], [3, 4], [5, 6]], f32), np.array([[7, 8, 9, 10]], f32)],
     "All inputs must have same second dimension"),
    (np.array([0, 6, 2, 1], i64),
     [np.array([[1, 2], [3, 4], [5, 6]], f32), np.array([[7, 8], [9, 10]], f32)],
     "row_id out of range"),
    (np.array([0, 6, 2, 1], i64),
     [np.arange(1, 7, dtype=f32).reshape(3, 2, 1), np.arange(7, 11, dtype=f32).reshape(2, 2, 1)],
     "input dims must == 2"),
]


def make_range(size, start, step):
    """MakeRange of fused_batchmatmul_add_sigmoid_test.cc:33-39 (float32 arithmetic)."""
    return (f32(start) + f32(step) * np.arange(size, dtype=f32)).astype(f32)


# fused_batchmatmul_add_sigmoid_test.cc:140-204: shapes and MakeRange(start, step) triples;
# expected = the in-test scalar reference (:54-91), tolerance 1e-5 (:136).
BMM_ADD_SIGMOID = [
    dict(name="FastPathN16BiasVector", lhs=((2, 32, 64), -0.2, 0.001), rhs=((64, 16), 0.15, 0.002), bias=((16,), -0.3, 0.05)),
    dict(name="FastPathN12BiasVector", lhs=((2, 32, 12), -0.1, 0.003), rhs=((12, 12), 0.05, 0.004), bias=((12,), 0.2, -0.03)),
    dict(name="FastPathN8BiasVector", lhs=((2, 32, 16), -0.25, 0.01), rhs=((16, 8), 0.1, 0.02), bias=((8,), -0.4, 0.1)),
    dict(name="FastPathN4BiasVector", lhs=((1, 32, 8), -0.2, 0.015), rhs=((8, 4), -0.1, 0.03), bias=((4,), 0.05, -0.02)),
    dict(name="GenericFallbackWithOddOutputWidth", lhs=((2, 5, 7), -0.3, 0.02), rhs=((7, 3), 0.2, -0.015), bias=((3,), -0.25, 0.2)),
    dict(name="GenericFallbackWithBatchedRhs", lhs=((2, 3, 4), -0.2, 0.05), rhs=((2, 4, 2), 0.15, -0.04), bias=((2, 1, 2), 0.1, 0.2)),
    dict(name="GenericFallbackWithLargeM", lhs=((1, 33, 4), -0.15, 0.01), rhs=((4, 4), 0.2, -0.03), bias=((1, 4), -0.2, 0.07)),
]

# fused_batchmatmul_add_sigmoid_test.cc:206-252: (lhs shape, rhs shape, bias shape, message)
BMM_ADD_SIGMOID_ERRORS = [
    ((4, 8), (8, 4), (4,), "lhs must be rank 3"),
    ((1, 4, 8), (1, 2, 4, 4), (4,), "rhs must be rank 2 or 3"),
    ((1, 4, 8), (8, 4), (1, 1, 1, 4), "bias rank must be <= 3"),
    ((2, 3, 4), (3, 4, 2), (2,), "lhs/rhs batch mismatch"),
    ((1, 3, 5), (4, 2), (2,), "lhs/rhs contracting dim mismatch"),
    ((2, 3, 4), (4, 2), (2, 2, 2), "bias shape is not broadcast-compatible"),
]


def bmm_case_tensors(case):
    def mk(spec):
        shape, start, step = spec
        return make_range(int(np.prod(shape)), start, step).reshape(shape)
    return mk(case["lhs"]), mk(case["rhs"]), mk(case["bias"])


def bmm_reference(lhs, rhs, bias):
    """The reference test's own scalar oracle (fused_batchmatmul_add_sigmoid_test.cc:54-91),
    evaluated in float32 with sequential k order."""
    b, m, k = lhs.shape
    n = rhs.shape[-1]
    bias3 = bias.reshape((1,) * (3 - bias.ndim) + bias.shape)
    out = np.empty((b, m, n), f32)
    for bi in range(b):
        R = rhs[bi] if rhs.ndim == 3 else rhs
        for i in range(m):
            for j in range(n):
                acc = f32(bias3[bi if bias3.shape[0] > 1 else 0, i if bias3.shape[1] > 1 else 0,
                                j if bias3.shape[2] > 1 else 0])
                for kk in range(k):
                    acc = f32(acc + f32(lhs[bi, i, kk] * R[kk, j]))
                out[bi, i, j] = f32(1.0) / (f32(1.0) + np.exp(-acc, dtype=f32))
    return out


# embedding_fused_padding_test.cc:87-245: (embedding_dims, table_size, pooling_size, reshape_size);
# input = 1..pooling*dims row-major; expected = the input followed by zeros, reshaped.
PADDING = [(10, 151, 151, 1510), (10, 1510, 151, 1510), (12, 2, 2, 24), (12, 200, 2, 24)]
# :247-305: (dims, table, pooling, reshape_sizes, pack, message)
PADDING_ERRORS = [
    (12, 200, 2, [10, 24], 12, "reshape[0] is not -1"),
    (12, 200, 2, [-1, 24], 10, "pack(10) is not equal to embedding dims"),
    (12, 200, 201, [-1, 24], 12, "Pooling size(201) is greater than Input size(200)"),
]

# embedding_fused_action_id_gather_test.cc:71-145
ACTION_ID_GATHER = dict(indices1=np.array([[0], [2]]), params=np.array([[1, 2], [3, 4], [5, 6]], f32),
                        indices2=np.array([[1], [0]]), pack_dim=2, pack=1,
                        out=np.array([[5, 6, 0], [1, 2, 0]], f32))

# embedding_fused_sparse_select_test.cc:128-155: (shape, a, b, c, greater, equal1, equal2, y)
SPARSE_SELECT = [
    ((3,), [5, 3, 8], [1, 2, 1], [9, 8, 7], 4, 1, 3, [1, 0, 1]),
    ((2, 2), [6, 3, 8, 2], [2, 1, 3, 4], [0, 0, 0, 0], 5, 2, 3, [1, 0, 1, 0]),
]

# embedding_fused_sparse_reshape_test.cc:100-127: (slice, begin, new_shape, pack_const, out_shape)
SPARSE_RESHAPE = [
    (np.array([[0, 1], [1, 2], [2, 3], [3, 0]], i64), [0, 1], [2, 4], 2, [2, 4]),
    (np.array([[0, 1]], i64), [0, 1], [-1, 1], 1, [1, 1]),
]
# :129-277: (slice, begin, new_shape, message)
SPARSE_RESHAPE_ERRORS = [
    (np.zeros((4,), i64), [0, 1], [2, 2], "slice_input dims must == 2"),
    (np.zeros((4, 2), i64), [0, 1], [2, 2, 1], "new_shape dim size must == 2"),
    (np.zeros((4, 2), i64), [0, 2], [2, 4], "begin[1] must < slice_input.dim_size(1)"),
    (np.zeros((4, 2), i64), [0, 1], [-1, -1], "only one output dimension may be -1"),
    (np.array([[0, 0], [0, 1], [0, 2], [1, 0], [1, 1], [1, 2]], i64), [0, 0], [-1, 4],
     "Input to reshape is a SparseTensor with"),
    (np.zeros((4, 2), i64), [0, 1], [3, 3], "Input to reshape is a tensor with"),
    (np.zeros((4, 2), i64), [0, 1], [2, -2], "size 1 must be non-negative, not -2"),
    (np.zeros((4, 2), i64), [0, 1], [-1, 0], "reshape cannot infer the missing input size for an empty tensor"),
    (np.zeros((4, 2), i64), [0], [2, 4], "begin must be 1D with at least 2 elements"),
    (np.zeros((4, 2), i64), [0, 1, 2], [2, 4], "begin must be 1D with at least 2 elements"),
]

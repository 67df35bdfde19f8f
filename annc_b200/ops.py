"""Host-side mirror of the reference's operator interface.

One function per reference op, same operand order and meaning, calling the C ABI
of libannc_b200.so.  Operands may be numpy arrays (host memory: staged by the
library) or torch CUDA tensors (used in place); outputs come back in the same
kind.  Failures raise AnncError carrying the reference's message.

``xla_*`` helpers play the XLA:CPU caller: they build the ``in[]`` operand array of
a custom call the way KDnnRewriter does, fusion operands followed by one s64
shape-info vector [dims..., minor_to_major...] per operand
(annc/service/hlo_util.h:14-33, annc/service/cpu/kdnn_rewriter.cc:59-66).
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import ALLOC_FN, ANNC_BOOL, ANNC_F32, ANNC_I32, ANNC_I64, ANNC_U64, Tensor, check, lib

try:  # torch is plumbing for device memory only
    import torch
except Exception:  # pragma: no cover
    torch = None

_NP_DTYPE = {ANNC_F32: np.float32, ANNC_I32: np.int32, ANNC_I64: np.int64, ANNC_BOOL: np.bool_,
             ANNC_U64: np.uint64}


def _is_torch(x) -> bool:
    return torch is not None and isinstance(x, torch.Tensor)


def _code(x) -> int:
    if _is_torch(x):
        return {torch.float32: ANNC_F32, torch.int32: ANNC_I32, torch.int64: ANNC_I64,
                torch.bool: ANNC_BOOL, torch.uint8: ANNC_BOOL, torch.uint64: ANNC_U64}[x.dtype]
    return {np.dtype(np.float32): ANNC_F32, np.dtype(np.int32): ANNC_I32,
            np.dtype(np.int64): ANNC_I64, np.dtype(np.bool_): ANNC_BOOL,
            np.dtype(np.uint8): ANNC_BOOL, np.dtype(np.uint64): ANNC_U64}[x.dtype]


def _ptr(x) -> int:
    if x is None:
        return 0
    return x.data_ptr() if _is_torch(x) else x.ctypes.data


def _contig(x):
    if x is None:
        return None
    if _is_torch(x):
        return x.contiguous()
    return np.ascontiguousarray(x)


def as_tensor(x, dtype_code: Optional[int] = None) -> Tensor:
    t = Tensor()
    t.data = _ptr(x)
    t.dtype = _code(x) if dtype_code is None else dtype_code
    shape = tuple(x.shape)
    if len(shape) > 4:
        raise ValueError("rank > 4 not supported")
    t.rank = len(shape)
    for i, d in enumerate(shape):
        t.dims[i] = int(d)
    return t


class _Outputs:
    """allocate_output stand-in: numpy on the host, torch on the device."""

    def __init__(self, on_device: bool, device=None):
        self.on_device = on_device
        self.device = device
        self.arrays = {}
        self.fn = ALLOC_FN(self._alloc)

    def _alloc(self, _ctx, index, dtype, rank, dims):
        shape = tuple(int(dims[i]) for i in range(rank))
        if self.on_device:
            td = {ANNC_F32: torch.float32, ANNC_I32: torch.int32, ANNC_I64: torch.int64,
                  ANNC_BOOL: torch.bool}[dtype]
            a = torch.empty(shape, dtype=td, device=self.device)
            self.arrays[index] = a
            return a.data_ptr() if a.numel() else 1  # non-null for empty outputs
        a = np.empty(shape, _NP_DTYPE[dtype])
        self.arrays[index] = a
        return a.ctypes.data if a.size else 1

    def __getitem__(self, i):
        return self.arrays[i]


def _outputs_for(x) -> _Outputs:
    if _is_torch(x) and x.is_cuda:
        lib.annc_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
        return _Outputs(True, x.device)
    return _Outputs(False)


def _small_i32(x):
    return np.ascontiguousarray(x.cpu().numpy() if _is_torch(x) else x, dtype=np.int32)


# ---------------------------------------------------------------- TF fused-op twins

def kp_fused_sparse_segment_reduce(data, indices, slice_input, begin, begin_1, combiner):
    """KPFusedSparseSegmentReduce -> (output f32[batch, D], slice_out int32 scalar)."""
    data, indices, slice_input = _contig(data), _contig(indices), _contig(slice_input)
    begin, begin_1 = _small_i32(begin), _small_i32(begin_1)
    outs = _outputs_for(data)
    check(lib.annc_KPFusedSparseSegmentReduce(
        C.byref(as_tensor(data)), C.byref(as_tensor(indices)), C.byref(as_tensor(slice_input)),
        C.byref(as_tensor(begin)), C.byref(as_tensor(begin_1)), C.c_int(combiner), outs.fn, None))
    return outs[0], outs[1]


def kp_fused_sparse_segment_reduce_nonzero(data, indices, slice_input, begin, combiner):
    """KPFusedSparseSegmentReduceNonzero -> (shape i32[r], indices i32[nz, r], values f32[nz])."""
    data, indices, slice_input = _contig(data), _contig(indices), _contig(slice_input)
    begin = _small_i32(begin)
    outs = _outputs_for(data)
    check(lib.annc_KPFusedSparseSegmentReduceNonzero(
        C.byref(as_tensor(data)), C.byref(as_tensor(indices)), C.byref(as_tensor(slice_input)),
        C.byref(as_tensor(begin)), C.c_int(combiner), outs.fn, None))
    return outs[0], outs[1], outs[2]


def kp_fused_gather(data, keys, begin):
    """KPFusedGather -> (unique keys i64[U], inverse map i32[nnz], rows f32[U, D])."""
    data, keys = _contig(data), _contig(keys)
    begin = _small_i32(begin)
    outs = _outputs_for(data)
    check(lib.annc_KPFusedGather(C.byref(as_tensor(data)), C.byref(as_tensor(keys)),
                                 C.byref(as_tensor(begin)), outs.fn, None))
    return outs[0], outs[1], outs[2]


def kp_fused_sparse_dynamic_stitch(x, tables: Sequence):
    """KPFusedSparseDynamicStitch -> f32[numel(x), D]."""
    x = _contig(x)
    tabs = [_contig(t) for t in tables]
    arr = (Tensor * len(tabs))(*[as_tensor(t) for t in tabs])
    outs = _outputs_for(tabs[0])
    check(lib.annc_KPFusedSparseDynamicStitch(C.byref(as_tensor(x)), arr, C.c_int(len(tabs)),
                                              outs.fn, None))
    return outs[0]


def kp_fused_embedding_with_hash_bucket(fingerprints, variable, num_buckets, empty=None,
                                        bounded=False):
    """KPFusedEmbeddingWithHashBucket on 64-bit fingerprints -> f32[batch, D]; ``bounded``
    gives the KPFusedDnn/Linear...WithHashBucket / RecEmbeddingV2 behaviour."""
    fingerprints, variable, empty = _contig(fingerprints), _contig(variable), _contig(empty)
    outs = _outputs_for(variable)
    e = C.byref(as_tensor(empty, ANNC_BOOL)) if empty is not None else None
    check(lib.annc_KPFusedEmbeddingWithHashBucket(
        C.byref(as_tensor(fingerprints, ANNC_U64)), e, C.byref(as_tensor(variable)),
        C.c_int64(num_buckets), C.c_int(int(bounded)), outs.fn, None))
    return outs[0]


def kp_fused_sparse_embedding(fingerprints, num_buckets, empty=None):
    """KPFusedSparseEmbedding / RecEmbeddingV1 -> (indices, values, empty_row_indicator, dense_shape)."""
    fingerprints, empty = _contig(fingerprints), _contig(empty)
    outs = _outputs_for(fingerprints)
    e = C.byref(as_tensor(empty, ANNC_BOOL)) if empty is not None else None
    check(lib.annc_KPFusedSparseEmbedding(C.byref(as_tensor(fingerprints, ANNC_U64)), e,
                                          C.c_int64(num_buckets), outs.fn, None))
    return outs[0], outs[1], outs[2], outs[3]


def kp_fused_batch_matmul_add_sigmoid(lhs, rhs, bias):
    """KPFusedBatchMatMulAddSigmoid -> f32[B, m, n]."""
    lhs, rhs, bias = _contig(lhs), _contig(rhs), _contig(bias)
    outs = _outputs_for(lhs)
    check(lib.annc_KPFusedBatchMatMulAddSigmoid(C.byref(as_tensor(lhs)), C.byref(as_tensor(rhs)),
                                                C.byref(as_tensor(bias)), outs.fn, None))
    return outs[0]


def sparse_embedding2(ids, table, lo, hi, dflt):
    """sparse_embedding2 fusion -> f32[n, D]."""
    ids, table = _contig(ids), _contig(table)
    n = int(np.prod(ids.shape))
    if _is_torch(table) and table.is_cuda:
        lib.annc_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
        out = torch.empty((n, table.shape[1]), dtype=torch.float32, device=table.device)
    else:
        out = np.empty((n, table.shape[1]), np.float32)
    check(lib.annc_sparse_embedding2(C.byref(as_tensor(ids)), C.byref(as_tensor(table)),
                                     C.c_int64(lo), C.c_int64(hi), C.c_int64(dflt),
                                     C.c_void_p(_ptr(out))))
    return out


# ---------------------------------------------------------------- XLA custom calls (mock caller)

def shape_info(x) -> np.ndarray:
    """get_param_info: [dims..., minor_to_major...] for a default row-major layout."""
    r = len(x.shape)
    return np.array(list(x.shape) + list(range(r - 1, -1, -1)), np.int64)


def _call_custom(target: str, out, operands: List):
    fn_addr = lib.annc_lookup_custom_call(target.encode())
    if not fn_addr:
        raise _lib.AnncError(102, f"custom-call target {target} is not registered "
                                  "(flag annc-pass off?)")
    fn = C.CFUNCTYPE(None, C.c_void_p, C.POINTER(C.c_void_p))(fn_addr)
    arr = (C.c_void_p * len(operands))(*[_ptr(o) for o in operands])
    if any(_is_torch(o) and o.is_cuda for o in operands):
        lib.annc_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    fn(C.c_void_p(_ptr(out)), arr)
    return out


def _new_like(x, shape):
    if _is_torch(x):
        return torch.empty(shape, dtype=torch.float32, device=x.device)
    return np.empty(shape, np.float32)


def xla_matmul(lhs, rhs):
    """custom-call "__matmul": in = {lhs, rhs, info(lhs), info(rhs)}."""
    lhs, rhs = _contig(lhs), _contig(rhs)
    out = _new_like(lhs, (lhs.shape[0], rhs.shape[1]))
    return _call_custom("__matmul", out, [lhs, rhs, shape_info(lhs), shape_info(rhs)])


def xla_layout_matmul(lhs, rhs_packed):
    """custom-call "__layout_matmul": rhs buffer is kn4-packed, declared shape [k, n]."""
    lhs, rhs_packed = _contig(lhs), _contig(rhs_packed)
    out = _new_like(lhs, (lhs.shape[0], rhs_packed.shape[1]))
    return _call_custom("__layout_matmul", out,
                        [lhs, rhs_packed, shape_info(lhs), shape_info(rhs_packed)])


def xla_batch_matmul(lhs, rhs):
    lhs, rhs = _contig(lhs), _contig(rhs)
    out = _new_like(lhs, (lhs.shape[0], lhs.shape[1], rhs.shape[2]))
    return _call_custom("__batch_matmul", out, [lhs, rhs, shape_info(lhs), shape_info(rhs)])


def xla_matmul_add(addend, lhs, rhs):
    """in = {addend, lhs, rhs, info(addend), info(lhs), info(rhs)}."""
    addend, lhs, rhs = _contig(addend), _contig(lhs), _contig(rhs)
    out = _new_like(lhs, (lhs.shape[0], rhs.shape[1]))
    return _call_custom("__matmul_add", out, [addend, lhs, rhs, shape_info(addend),
                                              shape_info(lhs), shape_info(rhs)])


def xla_matmul_add_relu(max_operand, addend, lhs, rhs):
    """in = {max operand, addend, lhs, rhs, 4 x info}."""
    max_operand, addend, lhs, rhs = (_contig(v) for v in (max_operand, addend, lhs, rhs))
    out = _new_like(lhs, (lhs.shape[0], rhs.shape[1]))
    return _call_custom("__matmul_add_relu", out,
                        [max_operand, addend, lhs, rhs, shape_info(max_operand),
                         shape_info(addend), shape_info(lhs), shape_info(rhs)])


def xla_pooling(arg, mul_out, slice_starts, slice_limits):
    """custom-call "__pooling": in = {arg, mul_out, slice_starts, slice_limits, info, info}."""
    arg, mul_out = _contig(arg), _contig(mul_out)
    ss = np.ascontiguousarray(slice_starts, np.int64)
    sl = np.ascontiguousarray(slice_limits, np.int64)
    out = _new_like(mul_out, (arg.shape[0], mul_out.shape[2]))
    return _call_custom("__pooling", out, [arg, mul_out, ss, sl, shape_info(arg),
                                           shape_info(mul_out)])


def xla_reduce_mean(value, m, n):
    """custom-call "__reduce_mean": in = {axis, value, unused, shape}."""
    value = _contig(value)
    out = _new_like(value, (n,))
    axis = np.zeros(1, np.float32)
    shape = np.array([m, n], np.int64)
    return _call_custom("__reduce_mean", out, [axis, value, axis, shape])


def xla_softmax(x):
    """__xla_cpu_runtime_XnnPackSoftMaxND on the [batch, channels] view of x."""
    x = _contig(x)
    ch = x.shape[-1]
    out = _new_like(x, tuple(x.shape))
    if _is_torch(x) and x.is_cuda:
        lib.annc_set_stream(C.c_void_p(torch.cuda.current_stream().cuda_stream))
    n = int(np.prod(x.shape))
    lib.__xla_cpu_runtime_XnnPackSoftMaxND(None, C.c_void_p(_ptr(x)), C.c_void_p(_ptr(out)),
                                           C.c_int64(n // ch), C.c_int64(ch))
    return out


def selector_gemm(variant, trA, trB, A, B, M, N, K, alpha=1.0, beta=0.0, Cin=None):
    """__xla_cpu_runtime_KernelSelectorGEMM{Sequential,Parallel,MLIR,Empty}."""
    A, B = _contig(A), _contig(B)
    if Cin is None:
        out = _new_like(A, (M, N))
        if beta != 0.0:
            out[...] = 0
    else:
        out = Cin.clone() if _is_torch(Cin) else np.array(Cin, np.float32, copy=True)
    fn = getattr(lib, f"__xla_cpu_runtime_KernelSelectorGEMM{variant}")
    fn(None, C.c_bool(trA), C.c_bool(trB), C.c_void_p(_ptr(A)), C.c_void_p(_ptr(B)), C.c_int(M),
       C.c_int(N), C.c_int(K), C.c_float(alpha), C.c_float(beta), C.c_void_p(_ptr(out)))
    return out


def selector_batch3d(variant, trA, trB, A, B, P, M, N, K):
    A, B = _contig(A), _contig(B)
    out = _new_like(A, (P, M, N))
    fn = getattr(lib, f"__xla_cpu_runtime_KernelSelectorBatch3D{variant}")
    fn(None, C.c_bool(trA), C.c_bool(trB), C.c_void_p(_ptr(A)), C.c_void_p(_ptr(B)), C.c_int(P),
       C.c_int(M), C.c_int(N), C.c_int(K), C.c_void_p(_ptr(out)))
    return out


def selector_batch4d(variant, trA, trB, A, B, Q, P, M, N, K):
    A, B = _contig(A), _contig(B)
    out = _new_like(A, (Q, P, M, N))
    fn = getattr(lib, f"__xla_cpu_runtime_KernelSelectorBatch4D{variant}")
    fn(None, C.c_bool(trA), C.c_bool(trB), C.c_void_p(_ptr(A)), C.c_void_p(_ptr(B)), C.c_int(Q),
       C.c_int(P), C.c_int(M), C.c_int(N), C.c_int(K), C.c_void_p(_ptr(out)))
    return out


def selector_gemv(variant, trA, A, X, M, N, alpha=1.0, beta=0.0, Yin=None):
    A, X = _contig(A), _contig(X)
    ny = N if trA else M
    if Yin is None:
        out = _new_like(A, (ny,))
        out[...] = 0
    else:
        out = Yin.clone() if _is_torch(Yin) else np.array(Yin, np.float32, copy=True)
    fn = getattr(lib, f"__xla_cpu_runtime_KernelSelectorGEMV{variant}")
    fn(None, C.c_bool(trA), C.c_void_p(_ptr(A)), C.c_void_p(_ptr(X)), C.c_int(M), C.c_int(N),
       C.c_float(alpha), C.c_float(beta), C.c_void_p(_ptr(out)))
    return out


def selector_argmax3d(variant, invals, inidxs, init_value, init_idx):
    invals, inidxs = _contig(invals), _contig(inidxs)
    B, M, N = invals.shape
    if _is_torch(invals):
        ov = torch.zeros((B, M), dtype=torch.float32, device=invals.device)
        oi = torch.zeros((B, M), dtype=torch.int32, device=invals.device)
    else:
        ov, oi = np.zeros((B, M), np.float32), np.zeros((B, M), np.int32)
    fn = getattr(lib, f"__xla_cpu_runtime_ArgMax3D{variant}")
    fn(None, C.c_int(B), C.c_int(M), C.c_int(N), C.c_void_p(_ptr(invals)), C.c_void_p(_ptr(inidxs)),
       C.c_float(init_value), C.c_int32(init_idx), C.c_void_p(_ptr(ov)), C.c_void_p(_ptr(oi)))
    return ov, oi


# ---------------------------------------------------------------- adjacent fused ops

def _scalar(v, dtype):
    return np.asarray(v, dtype=dtype).reshape(())


def kp_fused_embedding_padding(origin_shape, input, input_rows, reshape_sizes, pack, fast=False):
    """KPFusedEmbeddingPadding{,Fast} -> (padding rows, padded+reshaped input | its row count)."""
    input = _contig(input)
    outs = _outputs_for(input)
    os_ = np.array(origin_shape, dtype=np.int64)
    ir = np.array(input_rows, dtype=np.int32)
    rs = np.array(reshape_sizes, dtype=np.int32)
    pk = np.array(pack, dtype=np.int32)
    check(lib.annc_KPFusedEmbeddingPadding(C.byref(as_tensor(os_)), C.byref(as_tensor(input)),
                                           C.byref(as_tensor(ir)), C.byref(as_tensor(rs)),
                                           C.byref(as_tensor(pk)), C.c_int(int(fast)), outs.fn, None))
    return outs[0], outs[1]


def kp_fused_embedding_action_id_gather(indices1, params, indices2, pack_dim, pack):
    """KPFusedEmbeddingActionIdGather -> f32[pack_dim, cols + pack]."""
    indices1, params, indices2 = _contig(indices1), _contig(params), _contig(indices2)
    outs = _outputs_for(params)
    pd = np.array(pack_dim, dtype=np.int32)
    pk = np.array(pack, dtype=np.int32)
    check(lib.annc_KPFusedEmbeddingActionIdGather(
        C.byref(as_tensor(indices1)), C.byref(as_tensor(params)), C.byref(as_tensor(indices2)),
        C.byref(as_tensor(pd)), C.byref(as_tensor(pk)), outs.fn, None))
    return outs[0]


def kp_fused_sparse_reshape(slice_input, begin, new_shape, pack_const):
    """KPFusedSparseReshape -> (indices i64[rows, 2], shape i64[2])."""
    slice_input = _contig(slice_input)
    outs = _outputs_for(slice_input)
    bg = np.array(begin, dtype=np.int32)
    ns = np.array(new_shape, dtype=np.int64)
    pc = np.array(pack_const, dtype=np.int64)
    check(lib.annc_KPFusedSparseReshape(C.byref(as_tensor(slice_input)), C.byref(as_tensor(bg)),
                                        C.byref(as_tensor(ns)), C.byref(as_tensor(pc)), outs.fn, None))
    return outs[0], outs[1]


def kp_fused_sparse_select(a, b, c, greater, equal1, equal2, equal3=0):
    """KPFusedSparseSelect -> (x f32[n,1], y f32[n,1], w f32[n,2])."""
    a, b, c = _contig(a), _contig(b), _contig(c)
    outs = _outputs_for(a)
    sc = [_scalar(v, np.int32) for v in (greater, equal1, equal2, equal3)]
    check(lib.annc_KPFusedSparseSelect(C.byref(as_tensor(a)), C.byref(as_tensor(b)),
                                       C.byref(as_tensor(c)), *[C.byref(as_tensor(v)) for v in sc],
                                       outs.fn, None))
    return outs[0], outs[1], outs[2]

"""CPU oracle, Python side.  TEST INFRASTRUCTURE ONLY.

ctypes wrappers over ``oracle/_ref/libannc_oracle.so`` (the plain-C restatement
in ``annc_oracle.c``), numpy/OpenBLAS restatements of the GEMM custom calls, and
a restatement of the ``kn4`` prepacked-weight layout.  Only ``tests/``, the smoke
test and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may
import this module; the product package never does.

Reference citations are paths inside the ANNC project.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import List, Sequence, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_ref", "libannc_oracle.so")
_FLAGS_REF_PATH = os.path.join(_HERE, "_ref", "libannc_flags_ref.so")

i64p = C.POINTER(C.c_int64)
i32p = C.POINTER(C.c_int32)
f32p = C.POINTER(C.c_float)
u8p = C.POINTER(C.c_uint8)


def reference_root() -> str | None:
    """The ANNC checkout named by ANNC_REFERENCE_ROOT, or None when unset / not a directory."""
    root = os.environ.get("ANNC_REFERENCE_ROOT")
    return root if root and os.path.isdir(root) else None


def build(reference_root_dir: str | None = None) -> None:
    """Compile the C oracle, and where an ANNC checkout is given (argument, else the
    ANNC_REFERENCE_ROOT environment variable) the pieces of the reference that compile
    from their own sources."""
    root = reference_root_dir or reference_root()
    cmd = ["make", "-C", _HERE, "all"]
    if root:
        cmd += [f"REFERENCE_ROOT={root}", "ref"]
    subprocess.run(cmd, check=True, stdout=subprocess.DEVNULL)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_segment_batch.restype = C.c_int64
        _lib.oracle_sparse_segment_reduce_nonzero.restype = C.c_int64
        _lib.oracle_fused_gather.restype = C.c_int64
    return _lib


def _p(a: np.ndarray, t):
    return a.ctypes.data_as(t)


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---------------------------------------------------------------- embedding family

def segment_batch(slice_input: np.ndarray, col: int) -> int:
    s = _c(slice_input, np.int64)
    return int(lib().oracle_segment_batch(_p(s, i64p), C.c_int64(s.shape[0]),
                                          C.c_int64(s.shape[1]), C.c_int32(col)))


def sparse_segment_reduce(data, indices, slice_input, begin, begin_1, combiner
                          ) -> Tuple[np.ndarray, np.int32]:
    """KPFusedSparseSegmentReduce
    (annc/tensorflow/kernels/embedding_fused_sparse_segment_reduce.cc:38-152)."""
    data = _c(data, np.float32)
    s = _c(slice_input, np.int64)
    idx = np.ascontiguousarray(indices)
    idx64 = idx.dtype == np.int64
    if not idx64:
        idx = idx.astype(np.int32)
    col = int(begin[1])
    batch = segment_batch(s, col)
    out = np.empty((batch, data.shape[1]), np.float32)
    so = C.c_int32(0)
    lib().oracle_sparse_segment_reduce(
        _p(data, f32p), C.c_int64(data.shape[1]), idx.ctypes.data_as(C.c_void_p),
        C.c_int(int(idx64)), C.c_int64(idx.shape[0]), _p(s, i64p), C.c_int64(s.shape[1]),
        C.c_int32(col), C.c_int32(int(begin_1[0])), C.c_int(combiner), _p(out, f32p),
        C.c_int64(batch), C.byref(so))
    return out, np.int32(so.value)


def sparse_segment_reduce_nonzero(data, indices, slice_input, begin, combiner):
    """KPFusedSparseSegmentReduceNonzero
    (annc/tensorflow/kernels/embedding_fused_sparse_segment_reduce_nonzero.cc:39-374)."""
    data = _c(data, np.float32)
    rank = data.ndim
    dim = data.shape[1] if rank == 2 else 1
    s = _c(slice_input, np.int64)
    idx = np.ascontiguousarray(indices)
    idx64 = idx.dtype == np.int64
    if not idx64:
        idx = idx.astype(np.int32)
    nnz = idx.shape[0]
    cap = max(1, nnz * dim)
    out_shape = np.zeros(rank, np.int32)
    out_idx = np.zeros((cap, rank), np.int32)
    out_val = np.zeros(cap, np.float32)
    nz = lib().oracle_sparse_segment_reduce_nonzero(
        _p(data, f32p), C.c_int(rank), C.c_int64(dim), idx.ctypes.data_as(C.c_void_p),
        C.c_int(int(idx64)), C.c_int64(nnz), _p(s, i64p), C.c_int64(s.shape[1]),
        C.c_int32(int(begin[1])), C.c_int(combiner), _p(out_shape, i32p), _p(out_idx, i32p),
        _p(out_val, f32p))
    return out_shape, out_idx[:nz].copy(), out_val[:nz].copy()


def fused_gather(data, keys, begin):
    """KPFusedGather (annc/tensorflow/kernels/embedding_fused_gather.cc:26-86).
    Returns (unique_keys, inverse_indices, rows) or raises ValueError with the
    reference's message."""
    data = _c(data, np.float32)
    keys = _c(keys, np.int64)
    nnz, ncols = keys.shape
    uniq = np.zeros(max(nnz, 1), np.int64)
    inv = np.zeros(max(nnz, 1), np.int32)
    rows = np.zeros((max(nnz, 1), data.shape[1]), np.float32)
    nu = lib().oracle_fused_gather(
        _p(data, f32p), C.c_int64(data.shape[0]), C.c_int64(data.shape[1]), _p(keys, i64p),
        C.c_int64(nnz), C.c_int64(ncols), C.c_int32(int(begin[1])), _p(uniq, i64p),
        _p(inv, i32p), _p(rows, f32p))
    if nu < 0:
        raise ValueError("idx out of table range")
    return uniq[:nu].copy(), inv[:nnz].copy(), rows[:nu].copy()


def sparse_dynamic_stitch(x, tables: Sequence[np.ndarray]) -> np.ndarray:
    """KPFusedSparseDynamicStitch
    (annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:31-83)."""
    x = _c(x, np.int64).reshape(-1)
    tabs = [_c(t, np.float32) for t in tables]
    dim = tabs[0].shape[1]
    ptrs = (f32p * len(tabs))(*[_p(t, f32p) for t in tabs])
    rows = np.array([t.shape[0] for t in tabs], np.int64)
    out = np.zeros((x.shape[0], dim), np.float32)
    rc = lib().oracle_sparse_dynamic_stitch(_p(x, i64p), C.c_int64(x.shape[0]), ptrs,
                                            _p(rows, i64p), C.c_int(len(tabs)),
                                            C.c_int64(dim), _p(out, f32p))
    if rc != 0:
        raise ValueError("row_id out of range.")
    return out


def hash_bucket(hashes, num_buckets) -> np.ndarray:
    """uint64 fingerprint % num_buckets
    (python/tensorflow/kernels/fused_embedding_with_hash_bucket.cc:63-64)."""
    h = _c(hashes, np.uint64)
    out = np.zeros(h.shape, np.int64)
    lib().oracle_hash_bucket(h.ctypes.data_as(C.POINTER(C.c_uint64)), C.c_int64(h.size),
                             C.c_int64(num_buckets), _p(out, i64p))
    return out


def embedding_with_hash_bucket(hashes, empty, weight, num_buckets, bounded=False):
    """KPFusedEmbeddingWithHashBucket (fused_embedding_with_hash_bucket.cc:29-77); with
    ``bounded`` the Dnn/Linear/RecEmbeddingV2 variant that leaves out-of-table buckets
    zero (fused_dnn_embedding_with_hash_bucket.cc:32-47)."""
    h = _c(hashes, np.uint64)
    w = _c(weight, np.float32)
    e = None if empty is None else _c(empty, np.uint8)
    out = np.empty((h.shape[0], w.shape[1]), np.float32)
    hp = h.ctypes.data_as(C.POINTER(C.c_uint64))
    ep = _p(e, u8p) if e is not None else None
    if bounded:
        lib().oracle_dnn_embedding_with_hash_bucket(
            hp, ep, C.c_int64(h.shape[0]), _p(w, f32p), C.c_int64(w.shape[0]),
            C.c_int64(w.shape[1]), C.c_int64(num_buckets), _p(out, f32p))
    else:
        lib().oracle_embedding_with_hash_bucket(
            hp, ep, C.c_int64(h.shape[0]), _p(w, f32p), C.c_int64(w.shape[1]),
            C.c_int64(num_buckets), _p(out, f32p))
    return out


def sparse_embedding(hashes, empty, num_buckets):
    """KPFusedSparseEmbedding / RecEmbeddingV1
    (python/tensorflow/kernels/fused_sparse_embedding.cc:25-80)."""
    h = _c(hashes, np.uint64)
    e = _c(empty, np.uint8)
    n = h.shape[0]
    idx = np.zeros((n, 2), np.int64)
    val = np.zeros(n, np.int64)
    emp = np.zeros(n, np.uint8)
    shp = np.zeros(2, np.int64)
    ni, nv = C.c_int64(0), C.c_int64(0)
    lib().oracle_sparse_embedding(h.ctypes.data_as(C.POINTER(C.c_uint64)), _p(e, u8p),
                                  C.c_int64(n), C.c_int64(num_buckets), _p(idx, i64p),
                                  _p(val, i64p), _p(emp, u8p), _p(shp, i64p),
                                  C.byref(ni), C.byref(nv))
    return idx[:ni.value], val[:nv.value], emp[:nv.value].astype(bool), shp


def sparse_embedding2(ids, table, lo, hi, dflt) -> np.ndarray:
    """sparse_embedding2 fusion (annc/service/cpu/graph_opt.cc:8-41)."""
    ids = _c(ids, np.int64).reshape(-1)
    t = _c(table, np.float32)
    out = np.empty((ids.shape[0], t.shape[1]), np.float32)
    lib().oracle_sparse_embedding2(_p(ids, i64p), C.c_int64(ids.shape[0]), _p(t, f32p),
                                   C.c_int64(t.shape[1]), C.c_int64(lo), C.c_int64(hi),
                                   C.c_int64(dflt), _p(out, f32p))
    return out


def pooling(arg, mul_out, slice_starts, slice_limits) -> np.ndarray:
    """__pooling (annc/service/cpu/graph_opt.cc:131-176)."""
    arg = _c(arg, np.int64)
    mo = _c(mul_out, np.float32)
    m, k = arg.shape
    n = mo.shape[2]
    out = np.empty((m, n), np.float32)
    ss = _c(slice_starts, np.int64)
    sl = _c(slice_limits, np.int64)
    a_info = np.array([m, k, 1, 0], np.int64)
    m_info = np.array([m, k, n, 2, 1, 0], np.int64)
    lib().oracle_pooling(_p(out, f32p), _p(arg, i64p), _p(mo, f32p), _p(ss, i64p),
                         _p(sl, i64p), _p(a_info, i64p), _p(m_info, i64p))
    return out


def softmax(x) -> np.ndarray:
    """__xla_cpu_runtime_XnnPackSoftMaxND (annc/service/cpu/xla/xnnpack_ops.cc:30-74)."""
    x = _c(x, np.float32)
    ch = x.shape[-1]
    out = np.empty_like(x)
    lib().oracle_softmax(_p(x, f32p), _p(out, f32p), C.c_int64(x.size // ch), C.c_int64(ch))
    return out


def reduce_mean(value, m, n) -> np.ndarray:
    """__reduce_mean (annc/service/cpu/reduce_rewriter.cc:31-46)."""
    v = _c(value, np.float32)
    out = np.empty(n, np.float32)
    lib().oracle_reduce_mean(_p(out, f32p), _p(v, f32p), C.c_int64(m), C.c_int64(n))
    return out


def argmax3d(invals, inidxs, init_value, init_idx):
    """ArgMax3D (annc/service/cpu/xla/kernel_selector.cc:317-394)."""
    v = _c(invals, np.float32)
    ix = _c(inidxs, np.int32)
    n = v.shape[-1]
    rows = v.size // n
    ov = np.empty(v.shape[:-1], np.float32)
    oi = np.empty(v.shape[:-1], np.int32)
    lib().oracle_argmax3d(C.c_int64(rows), C.c_int64(n), _p(v, f32p), _p(ix, i32p),
                          C.c_float(init_value), C.c_int32(init_idx), _p(ov, f32p), _p(oi, i32p))
    return ov, oi


# ---------------------------------------------------------------- GEMM family

_blas = None


def openblas() -> C.CDLL:
    """scipy's bundled OpenBLAS (LP64 `scipy_cblas_*` names): the library family the reference
    links (OpenBLAS 0.3.29, third_party/repo.bzl:3-12).  Threads are set to the affinity count."""
    global _blas
    if _blas is None:
        import glob
        import scipy
        cand = glob.glob(os.path.join(os.path.dirname(scipy.__file__), os.pardir, "scipy.libs",
                                      "libscipy_openblas*.so"))
        if not cand:
            raise RuntimeError("scipy's bundled OpenBLAS was not found")
        _blas = C.CDLL(cand[0])
        _blas.scipy_cblas_sasum.restype = C.c_float
        _blas.scipy_openblas_set_num_threads(C.c_int(max(1, host_threads())))
    return _blas


def set_blas_threads(n: int) -> None:
    openblas().scipy_openblas_set_num_threads(C.c_int(max(1, int(n))))


_ROW, _NOTR, _TR = 101, 111, 112


def cblas_sgemm(trA, trB, M, N, K, alpha, A, lda, B, ldb, beta, Cbuf, ldc) -> None:
    """cblas_sgemm(CblasRowMajor, ...) on contiguous float32 arrays; Cbuf is updated in place."""
    openblas().scipy_cblas_sgemm(C.c_int(_ROW), C.c_int(_TR if trA else _NOTR),
                                 C.c_int(_TR if trB else _NOTR), C.c_int(M), C.c_int(N), C.c_int(K),
                                 C.c_float(alpha), _p(A, f32p), C.c_int(lda), _p(B, f32p),
                                 C.c_int(ldb), C.c_float(beta), _p(Cbuf, f32p), C.c_int(ldc))


def sgemm(trA, trB, A, B, M, N, K, alpha=1.0, beta=0.0, Cin=None, blas=True) -> np.ndarray:
    """Row-major sgemm with the leading dimensions of
    annc/service/cpu/xla/kernel_selector.cc:31-43 (lda = trA ? M : K, ldb = trB ? K : N).
    ``blas=True`` calls OpenBLAS cblas_sgemm like the reference, else the scalar C loop."""
    A = _c(A, np.float32).reshape((M, K) if not trA else (K, M))
    B = _c(B, np.float32).reshape((K, N) if not trB else (N, K))
    out = np.zeros((M, N), np.float32) if Cin is None else _c(Cin, np.float32).reshape(M, N).copy()
    if M * N == 0:
        return out
    if blas:
        if K == 0:
            return (np.float32(beta) * out).astype(np.float32)
        cblas_sgemm(trA, trB, M, N, K, alpha, A, M if trA else K, B, K if trB else N, beta, out, N)
        return out
    lib().oracle_sgemm(C.c_int(int(trA)), C.c_int(int(trB)), C.c_int64(M), C.c_int64(N),
                       C.c_int64(K), C.c_float(alpha), _p(A, f32p), _p(B, f32p),
                       C.c_float(beta), _p(out, f32p))
    return out


def matmul(A, B):
    """__matmul (annc/service/cpu/gemm_rewriter.cc:161-185): one row-major sgemm, alpha 1 beta 0."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    (M, K), N = A.shape, B.shape[1]
    return sgemm(False, False, A, B, M, N, K)


def batch_matmul(A, B):
    """__batch_matmul (annc/service/cpu/gemm_rewriter.cc:187-216): one sgemm per batch slab."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    lead = A.shape[:-2]
    A3, B3 = A.reshape((-1,) + A.shape[-2:]), B.reshape((-1,) + B.shape[-2:])
    out = np.empty((A3.shape[0], A3.shape[1], B3.shape[2]), np.float32)
    for i in range(A3.shape[0]):
        out[i] = sgemm(False, False, A3[i], B3[i], A3.shape[1], B3.shape[2], A3.shape[2])
    return out.reshape(lead + out.shape[-2:])


def matmul_add(addend, A, B):
    """__matmul_add (annc/service/cpu/gemm_rewriter.cc:218-247): memcpy of the addend into the
    output, then sgemm with beta = 1."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    (M, K), N = A.shape, B.shape[1]
    return sgemm(False, False, A, B, M, N, K, 1.0, 1.0, np.broadcast_to(_c(addend, np.float32), (M, N)))


def matmul_add_relu(addend, A, B):
    """__matmul_add_relu (annc/service/cpu/gemm_rewriter.cc:249-281); the max operand is
    ignored by the reference, a literal 0 is used (:279)."""
    return np.maximum(matmul_add(addend, A, B), np.float32(0.0))


def sgemv(trA, A, X, M, N, alpha=1.0, beta=0.0, Y=None):
    """KernelSelectorGEMV (annc/service/cpu/xla/kernel_selector.cc:168-178)."""
    A = _c(A, np.float32).reshape(M, N)
    X = _c(X, np.float32)
    out = np.zeros(N if trA else M, np.float32) if Y is None else _c(Y, np.float32).copy()
    lib().oracle_sgemv(C.c_int(int(trA)), C.c_int64(M), C.c_int64(N), C.c_float(alpha),
                       _p(A, f32p), _p(X, f32p), C.c_float(beta), _p(out, f32p))
    return out


def batch_matmul_add_sigmoid(lhs, rhs, bias) -> np.ndarray:
    """KPFusedBatchMatMulAddSigmoid, generic path
    (annc/tensorflow/kernels/fused_batchmatmul_add_sigmoid.cc:216-255)."""
    lhs = _c(lhs, np.float32)
    rhs = _c(rhs, np.float32)
    bias = _c(bias, np.float32)
    b, m, k = lhs.shape
    n = rhs.shape[-1]
    bd = np.ones(3, np.int64)
    for i, d in enumerate(bias.shape):
        bd[3 - bias.ndim + i] = d
    out = np.empty((b, m, n), np.float32)
    lib().oracle_batch_matmul_add_sigmoid(_p(lhs, f32p), _p(rhs, f32p), _p(bias, f32p),
                                          _p(bd, i64p), C.c_int64(b), C.c_int64(m),
                                          C.c_int64(k), C.c_int64(n), C.c_int(int(rhs.ndim == 3)),
                                          _p(out, f32p))
    return out


# ---------------------------------------------------------------- kn4 prepacked layout

def _split_axis(dim: int, tile: int, vec: int) -> List[Tuple[int, int]]:
    """Chunk boundaries of one axis (python/annc/optimize/data_pack.py:43-92): chunks of
    ``tile``; when ``dim`` is not a multiple the last two chunks share the remainder,
    the first of them rounded to a multiple of ``vec``."""
    if dim < tile:
        return [(0, dim)]
    num = dim // tile + (1 if dim % tile else 0)
    out = []
    for i in range(num):
        start, end = i * tile, (i + 1) * tile
        if dim % tile:
            if i == num - 2 or i == num - 1:
                res = dim - (num - 2) * tile
                first = (res // 2) // vec * vec
                if res - first > first + 1:
                    first += vec
                if i == num - 2:
                    end = start + first
                else:
                    start, end = dim - res + first, dim
        out.append((start, end))
    return out


def _panel_widths(n: int, vec: int) -> List[int]:
    """Panel widths inside one block (data_pack.py:129-149)."""
    w = [vec] * (n // vec)
    rest = n % vec
    small = 4 if vec == 12 else vec // 2
    while small:
        if vec == 12:
            while rest >= small:
                w.append(small)
                rest -= small
        elif rest >= small:
            w.append(small)
            rest -= small
        small //= 2
    return w


def kn4_offsets(K: int, N: int, vec: int = 12, k_tile: int = 352, n_tile: int = 128) -> np.ndarray:
    """int64[K,N] map: position of B[k,n] inside the kn4-packed buffer written by
    ``FormageChange(12).run(B, kn, kn4, [(0,352),(1,128)])``
    (python/annc/optimize/constant_folding.py:77-88, data_pack.py:36-41,118-127)."""
    off = np.empty((K, N), np.int64)
    pos = 0
    for k0, k1 in _split_axis(K, k_tile, vec):
        for n0, n1 in _split_axis(N, n_tile, vec):
            nloc = n0
            for w in _panel_widths(n1 - n0, vec):
                cnt = (k1 - k0) * w
                off[k0:k1, nloc:nloc + w] = pos + np.arange(cnt, dtype=np.int64).reshape(k1 - k0, w)
                pos += cnt
                nloc += w
    assert pos == K * N
    return off


def kn4_pack(B: np.ndarray) -> np.ndarray:
    B = _c(B, np.float32)
    out = np.empty(B.size, np.float32)
    out[kn4_offsets(*B.shape).reshape(-1)] = B.reshape(-1)
    return out.reshape(B.shape)


def kn4_unpack(packed: np.ndarray, K: int, N: int) -> np.ndarray:
    return _c(packed, np.float32).reshape(-1)[kn4_offsets(K, N)]


def layout_matmul(A, Bpacked):
    """__layout_matmul (annc/service/cpu/gemm_rewriter.cc:136-159): C = A . unpack(Bpacked)."""
    A = _c(A, np.float32)
    K = A.shape[1]
    N = Bpacked.size // K
    return (A @ kn4_unpack(Bpacked, K, N)).astype(np.float32)


# ---------------------------------------------------------------- custom-call bodies (real reference)

_XLA_REF_PATH = os.path.join(_HERE, "_ref", "libannc_xla_ref.so")
_xla_ref = None


def xla_ref_available() -> bool:
    return os.path.exists(_XLA_REF_PATH)


def xla_ref() -> C.CDLL:
    """The reference's own bodies of __matmul, __batch_matmul, __matmul_add, __matmul_add_relu,
    __pooling and __reduce_mean (oracle/xla_ref_shim.cc, built by `make ref`), with their CBLAS
    calls pointed at the same OpenBLAS the restatements above call."""
    global _xla_ref
    if _xla_ref is None:
        l = C.CDLL(_XLA_REF_PATH)
        b = openblas()
        l.annc_xla_ref_set_blas(C.cast(b.scipy_cblas_sgemm, C.c_void_p), C.cast(b.scipy_cblas_sasum, C.c_void_p))
        if hasattr(l, "annc_xla_ref_set_sgemv"):
            l.annc_xla_ref_set_sgemv(C.cast(b.scipy_cblas_sgemv, C.c_void_p))
        _xla_ref = l
    return _xla_ref


def shape_info(a: np.ndarray) -> np.ndarray:
    """The s64 operand XLA appends per tensor: [dims..., minor_to_major...]
    (annc/service/hlo_util.h:14-21); row-major, so minor_to_major = rank-1 .. 0."""
    return np.array(list(a.shape) + list(range(a.ndim - 1, -1, -1)), np.int64)


def xla_ref_call(name: str, out: np.ndarray, operands) -> np.ndarray:
    """Calls annc_ref_<name>(out, in) with `operands` (contiguous numpy arrays) as in[]."""
    keep = [np.ascontiguousarray(o) for o in operands]
    arr = (C.c_void_p * len(keep))(*[C.c_void_p(o.ctypes.data) for o in keep])
    getattr(xla_ref(), "annc_ref_" + name)(C.c_void_p(out.ctypes.data), arr)
    return out


def xla_ref_kernel_selector_available() -> bool:
    return xla_ref_available() and hasattr(xla_ref(), "annc_ref_ks_gemm")


def ks_ref_gemm(trA, trB, A, B, M, N, K, alpha=1.0, beta=0.0, Cin=None) -> np.ndarray:
    """The reference's own __xla_cpu_runtime_KernelSelectorGEMMSequential
    (annc/service/cpu/xla/kernel_selector.cc:31-43)."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    out = np.zeros((M, N), np.float32) if Cin is None else _c(Cin, np.float32).reshape(M, N).copy()
    xla_ref().annc_ref_ks_gemm(C.c_int(int(trA)), C.c_int(int(trB)), _p(A, f32p), _p(B, f32p), C.c_int(M),
                               C.c_int(N), C.c_int(K), C.c_float(alpha), C.c_float(beta), _p(out, f32p))
    return out


def ks_ref_batch(trA, trB, A, B, lead, M, N, K) -> np.ndarray:
    """...KernelSelectorBatch3DSequential (lead = (P,)) or ...Batch4DSequential (lead = (Q, P))
    (kernel_selector.cc:99-116, 234-251)."""
    A, B = _c(A, np.float32), _c(B, np.float32)
    out = np.empty(tuple(lead) + (M, N), np.float32)
    if len(lead) == 1:
        xla_ref().annc_ref_ks_batch3d(C.c_int(int(trA)), C.c_int(int(trB)), _p(A, f32p), _p(B, f32p),
                                      C.c_int(lead[0]), C.c_int(M), C.c_int(N), C.c_int(K), _p(out, f32p))
    else:
        xla_ref().annc_ref_ks_batch4d(C.c_int(int(trA)), C.c_int(int(trB)), _p(A, f32p), _p(B, f32p),
                                      C.c_int(lead[0]), C.c_int(lead[1]), C.c_int(M), C.c_int(N), C.c_int(K),
                                      _p(out, f32p))
    return out


def ks_ref_gemv(trA, A, X, M, N, alpha=1.0, beta=0.0, Y=None) -> np.ndarray:
    """...KernelSelectorGEMV (kernel_selector.cc:168-178): cblas_sgemv with lda = trA ? M : N."""
    A, X = _c(A, np.float32), _c(X, np.float32)
    out = np.zeros(N if trA else M, np.float32) if Y is None else _c(Y, np.float32).copy()
    xla_ref().annc_ref_ks_gemv(C.c_int(int(trA)), _p(A, f32p), _p(X, f32p), C.c_int(M), C.c_int(N),
                               C.c_float(alpha), C.c_float(beta), _p(out, f32p))
    return out


def ks_ref_argmax3d(invals, inidxs, init_value, init_idx):
    """...ArgMax3DSequential over f32/i32 [B, M, N] (kernel_selector.cc:317-339, 376-389)."""
    v, ix = _c(invals, np.float32), _c(inidxs, np.int32)
    Bn, M, N = v.shape
    ov, oi = np.empty((Bn, M), np.float32), np.empty((Bn, M), np.int32)
    xla_ref().annc_ref_ks_argmax3d(C.c_int(Bn), C.c_int(M), C.c_int(N), _p(v, f32p), _p(ix, i32p),
                                   C.c_float(init_value), C.c_int32(init_idx), _p(ov, f32p), _p(oi, i32p))
    return ov, oi


# ---------------------------------------------------------------- ANNC_FLAGS (real reference)

def flags_ref_available() -> bool:
    return os.path.exists(_FLAGS_REF_PATH)


def flag_enabled_ref(flags_env: str | None, name: str) -> bool:
    """Runs the reference's own parser (annc/service/cpu/annc_flags.cc) compiled into
    oracle/_ref/libannc_flags_ref.so."""
    l = C.CDLL(_FLAGS_REF_PATH)
    return bool(l.annc_ref_flag_enabled(None if flags_env is None else flags_env.encode(),
                                        name.encode()))


# ---------------------------------------------------------------- DLRM-style model on the CPU

def embed_bags_tables(tables, table_rows, raw_ids, slice_inputs, batch, dim, out, out_slots,
                      out_first, combiner=0, col=0, threads=1) -> None:
    """Hash-bucket mapping (E1) + segment reduce (E3) of every table into
    out[batch, out_slots, dim] starting at slot out_first; one table per thread."""
    n = len(tables)
    tabs = [_c(t, np.float32) for t in tables]
    ids = [_c(i, np.int64) for i in raw_ids]
    segs = [_c(s, np.int64) for s in slice_inputs]
    tp = (f32p * n)(*[_p(t, f32p) for t in tabs])
    ip = (i64p * n)(*[_p(i, i64p) for i in ids])
    sp = (i64p * n)(*[_p(s, i64p) for s in segs])
    rows = np.asarray(table_rows, np.int64)
    nnz = np.array([i.shape[0] for i in ids], np.int64)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    lib().oracle_embed_bags_tables(C.c_int(n), tp, _p(rows, i64p), C.c_int64(dim), ip, sp,
                                   _p(nnz, i64p), C.c_int64(segs[0].shape[1]), C.c_int32(col),
                                   C.c_int(combiner), C.c_int64(batch), _p(out, f32p),
                                   C.c_int64(out_slots), C.c_int64(out_first), C.c_int(threads))


def host_threads() -> int:
    return int(lib().oracle_num_threads())


def dlrm_forward(model, sample: int | None = None, threads: int = 1) -> np.ndarray:
    """CPU forward of the DLRM-style model the way the reference's operators would run it:
    bottom MLP as __matmul_add_relu calls (OpenBLAS sgemm + bias add + max, gemm_rewriter.cc
    :249-281), per-table hash-bucket + KPFusedSparseSegmentReduce sum pooling, dot interaction
    as __batch_matmul of Z by its transpose and the strict lower triangle, top MLP with a final
    sigmoid.  ``sample`` limits the pass to the first `sample` samples of the batch."""
    emb = model.emb
    B = emb.batch if sample is None else min(sample, emb.batch)
    x = _c(model.dense[:B], np.float32)
    for w, b in model.bottom:
        x = np.maximum(x @ w + b, np.float32(0))
    T = len(emb.tables)
    F = T + 1
    z = np.empty((B, F, emb.dim), np.float32)
    z[:, 0, :] = x
    ids, segs = [], []
    for bag in emb.bags:
        n = int(np.searchsorted(bag.slice_input[:, 0], B, side="left"))
        ids.append(bag.raw_ids[:n])
        segs.append(bag.slice_input[:n])
    embed_bags_tables(emb.tables, [t.shape[0] for t in emb.tables], ids, segs, B, emb.dim, z, F, 1,
                      threads=threads)
    g = np.matmul(z, np.swapaxes(z, 1, 2))
    li, lj = np.tril_indices(F, -1)
    h = np.concatenate([z[:, 0, :], g[:, li, lj]], axis=1)
    for i, (w, b) in enumerate(model.top):
        h = h @ w + b
        if i + 1 < len(model.top):
            h = np.maximum(h, np.float32(0))
    return (np.float32(1) / (np.float32(1) + np.exp(-h, dtype=np.float32))).astype(np.float32)


# ---------------------------------------------------------------- adjacent fused ops (numpy)

def embedding_padding(origin_shape, x, input_rows, reshape_sizes, fast=False):
    """KPFusedEmbeddingPadding{,Fast} (annc/tensorflow/kernels/embedding_fused_padding.cc:35-113)."""
    x = _c(x, np.float32)
    pad = int(origin_shape[0]) - int(input_rows)
    cols = int(reshape_sizes[1])
    out_rows = pad + x.shape[0]
    rr = out_rows * x.shape[1] // cols
    if fast:
        return np.int32(pad), np.int32(rr)
    flat = np.zeros(out_rows * x.shape[1], np.float32)
    live = int(input_rows) * x.shape[1]
    flat[:live] = x.reshape(-1)[:live]
    return np.int32(pad), flat.reshape(rr, cols)


def action_id_gather(indices1, params, indices2, pack_dim, pack):
    """KPFusedEmbeddingActionIdGather
    (annc/tensorflow/kernels/embedding_fused_action_id_gather.cc:59-129)."""
    t1 = _c(params, np.float32)[np.asarray(indices1)]
    t2 = t1[np.asarray(indices2)]
    a = t2.reshape(int(pack_dim), -1)
    return np.concatenate([a, np.zeros((int(pack_dim), int(pack)), np.float32)], axis=1)


def sparse_reshape(slice_input, begin, new_shape, pack_const):
    """KPFusedSparseReshape (annc/tensorflow/kernels/embedding_fused_sparse_reshape.cc:28-190)."""
    s = _c(slice_input, np.int64)
    rows = s.shape[0]
    in_shape = [rows, int(pack_const)]
    tgt = [int(v) for v in new_shape]
    dense = in_shape[0] * in_shape[1]
    out_shape = list(tgt)
    if -1 in tgt:
        k = tgt.index(-1)
        other = tgt[1 - k]
        out_shape[k] = dense // other
    ids = np.arange(rows, dtype=np.int64) * in_shape[1] + s[:, int(begin[1])]
    if out_shape == in_shape:
        idx = np.stack([np.arange(rows, dtype=np.int64), s[:, int(begin[1])]], 1)
    else:
        idx = np.stack([ids // out_shape[1], ids % out_shape[1]], 1)
    return idx, np.array(out_shape, np.int64)


def sparse_select(a, b, greater, equal1, equal2):
    """KPFusedSparseSelect (annc/tensorflow/kernels/embedding_fused_sparse_select.cc:32-107)."""
    a = np.asarray(a, np.int32).reshape(-1)
    b = np.asarray(b, np.int32).reshape(-1)
    g = (a > greater).astype(np.float32)
    r1 = np.where(b == equal1, np.float32(1), g)
    r2 = np.where(b == equal2, np.float32(1), r1).astype(np.float32)
    return a.astype(np.float32).reshape(-1, 1), r2.reshape(-1, 1), np.stack([r2, np.ones_like(r2)], 1)


# ---------------------------------------------------------------- KERNEL_MAP_FILE
# Restatement of the kernel selector's map parser and lookup
# (annc/service/cpu/xla/kernel_selector_ops_rewriter.cc:50-104 IntervalMap, :124-195 parseInt /
# parseRange / parseLine, :201-259 fill_map_from_file).

_KMAP_TYPES = {"gemv": (0, 2), "gemm": (1, 3), "batch3d": (2, 4), "batch4d": (3, 5), "argmax": (4, 3)}
_KMAP_ANY = (0, 2 ** 31 - 1)


def kernel_map_parse(text: str):
    """Returns (entries, bad_lines); entries is a dict {(type_index, ranges): symbol}."""
    import re
    elem = r"(?:\d+|\*|\d+:(?:\d+|\*))"
    pat = re.compile(r"^\[(.+)\]\(((?:" + elem + r",)*" + elem + r")\)->(.+)$", re.S)
    entries, bad = {}, 0
    for line in text.split("\n")[:-1] if text.endswith("\n") else text.split("\n"):
        if line.endswith("\r"):
            line = line[:-1]
        t = "".join(ch for ch in line if ch not in " \t\n\v\f\r")
        m = pat.match(t)
        if not m:
            bad += 1
            continue

        def num(s):
            if s == "*":
                return _KMAP_ANY[1]
            v = int(s)
            return v if v <= _KMAP_ANY[1] else -1

        ranges, ok = [], True
        for tok in m.group(2).split(","):
            if tok == "*":
                r = _KMAP_ANY
            elif ":" in tok:
                a, b = tok.split(":")
                r = (num(a), num(b))
            else:
                r = (num(tok), num(tok))
            if r[0] == -1 or r[1] == -1:
                ok = False
                break
            ranges.append(r)
        if not ok:
            bad += 1
            continue
        if m.group(1) not in _KMAP_TYPES:
            bad += 1
            break
        ty, rank = _KMAP_TYPES[m.group(1)]
        if len(ranges) == 1 and ranges[0] == _KMAP_ANY:
            ranges = [_KMAP_ANY] * rank
        if len(ranges) != rank:
            bad += 1
            continue
        entries[(ty, tuple(ranges))] = m.group(3)
    return entries, bad


def kernel_map_lookup(entries, kernel: str, sizes):
    """First entry, in std::map key order, whose ranges contain the sizes; None otherwise."""
    if kernel not in _KMAP_TYPES:
        return None
    ty = _KMAP_TYPES[kernel][0]
    for key in sorted(entries):
        if key[0] != ty or len(key[1]) != len(sizes):
            continue
        if all(lo <= s <= hi for s, (lo, hi) in zip(sizes, key[1])):
            return entries[key]
    return None

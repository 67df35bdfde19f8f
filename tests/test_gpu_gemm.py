"""Parity of the GEMM custom calls, kernel-selector entry points and the
KPFusedBatchMatMulAddSigmoid twin with the CPU oracle, through the C ABI.
Error measure: normwise max|y - ref| / max|ref| against the fp32 OpenBLAS result;
bound 2e-3 for the TF32 tensor-core route, 1e-2 for BF16, 2e-5 for the fp32 route."""
import numpy as np
import pytest

from oracle import oracle
from tests.golden import reference_cases as rc

pytestmark = pytest.mark.gpu

import torch
from annc_b200 import ops  # noqa: E402  (no fallback: a missing library fails the collection)
from annc_b200 import AnncError, _lib, device, synth  # noqa: E402

TOL = {"simt_fp32": 2e-5, "tcgen05_tf32": 2e-3, "tcgen05_pair_tf32": 2e-3, "tcgen05_pair_bf16": 1e-2}


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def nerr(got, want):
    got = got.cpu().numpy() if hasattr(got, "cpu") else got
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def _tol_for(m, n, k, **kw):
    d = _lib.GemmDesc()
    d.m, d.n, d.k, d.batch = m, n, k, kw.get("batch", 1)
    d.lda, d.ldb, d.ldc = k, n, n
    d.stride_a, d.stride_b, d.stride_c = m * k, k * n, m * n
    d.a = d.b = d.c = 256  # alignment probe only
    d.trans_a, d.trans_b = int(kw.get("trA", False)), int(kw.get("trB", False))
    d.b_format = kw.get("b_format", 0)
    return TOL[_lib.lib.annc_gemm_kernel_name(__import__("ctypes").byref(d)).decode()]


@pytest.mark.parametrize("shape", [(12, 12, 12), (13, 17, 19), (64, 64, 64), (100, 130, 77),
                                   (128, 128, 128), (256, 512, 384), (512, 1024, 1024),
                                   (1000, 520, 264), (129, 257, 100)])
@pytest.mark.parametrize("where", ["host", "device"])
def test_matmul_custom_call(shape, where):
    m, n, k = shape
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    want = oracle.matmul(a, b)
    got = ops.xla_matmul(_dev(a), _dev(b)) if where == "device" else ops.xla_matmul(a, b)
    assert nerr(got, want) <= _tol_for(m, n, k)


def test_matmul_add_relu_config():
    """BASELINE config: X[512,1024] ~ U(-1,1), W[1024,1024] ~ N(0,1/32), bias ~ N(0,0.1)."""
    x, w, bias, addend, maxop = synth.matmul_add_relu_case(0)
    want = oracle.matmul_add_relu(addend, x, w)
    got = ops.xla_matmul_add_relu(_dev(maxop), _dev(addend), _dev(x), _dev(w))
    assert nerr(got, want) <= _tol_for(512, 1024, 1024)
    assert (got.cpu().numpy() >= 0).all()
    got_add = ops.xla_matmul_add(addend, x, w)
    assert nerr(got_add, oracle.matmul_add(addend, x, w)) <= _tol_for(512, 1024, 1024)


@pytest.mark.parametrize("shape", [(4, 16, 8, 24), (64, 256, 64, 256), (3, 27, 64, 27), (70000, 8, 8, 8)])
def test_batch_matmul_custom_call(shape):
    b, m, k, n = shape
    rng = np.random.default_rng(b)
    A = rng.standard_normal((b, m, k)).astype(np.float32)
    B = rng.standard_normal((b, k, n)).astype(np.float32)
    got = ops.xla_batch_matmul(_dev(A), _dev(B))
    assert nerr(got, oracle.batch_matmul(A, B)) <= _tol_for(m, n, k, batch=b)


@pytest.mark.parametrize("shape", [(12, 12, 12), (40, 30, 20), (64, 353, 129), (128, 400, 140),
                                   (256, 705, 257), (512, 1024, 1024)])
def test_layout_matmul_custom_call(shape):
    m, k, n = shape
    rng = np.random.default_rng(k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    packed = oracle.kn4_pack(w)  # pinned to the reference packer in the CPU tests
    want = oracle.layout_matmul(a, packed)
    got = ops.xla_layout_matmul(_dev(a), _dev(packed))
    assert nerr(got, want) <= _tol_for(m, n, k, b_format=1)


def test_kn4_device_pack_unpack_bit_exact():
    for K, N in [(12, 12), (353, 129), (705, 257), (2048, 4096)]:
        w = np.arange(K * N, dtype=np.float32).reshape(K, N)
        packed = device.kn4_pack(_dev(w))
        if K * N < 1_000_000:
            np.testing.assert_array_equal(packed.cpu().numpy(), oracle.kn4_pack(w))
        assert torch.equal(device.kn4_unpack(packed), _dev(w))
    offs = oracle.kn4_offsets(705, 257)
    for k, n in [(0, 0), (704, 256), (352, 128), (351, 127), (500, 200)]:
        assert _lib.lib.annc_kn4_offset(705, 257, k, n) == offs[k, n]


@pytest.mark.parametrize("variant", ["Sequential", "Parallel", "MLIR"])
@pytest.mark.parametrize("trA,trB", [(False, False), (True, False), (False, True), (True, True)])
def test_selector_gemm(variant, trA, trB):
    M, N, K = 70, 50, 90
    rng = np.random.default_rng(1)
    A = rng.standard_normal((K, M) if trA else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if trB else (K, N)).astype(np.float32)
    C0 = rng.standard_normal((M, N)).astype(np.float32)
    for alpha, beta in [(1.0, 0.0), (0.5, 1.0), (2.0, -0.25)]:
        want = oracle.sgemm(trA, trB, A, B, M, N, K, alpha, beta, C0)
        got = ops.selector_gemm(variant, trA, trB, A, B, M, N, K, alpha, beta, C0)
        assert nerr(got, want) <= 2e-5


def test_selector_empty_variants_are_noops():
    A = np.ones((4, 4), np.float32)
    C0 = np.full((4, 4), 3.0, np.float32)
    got = ops.selector_gemm("Empty", False, False, A, A, 4, 4, 4, 1.0, 0.0, C0)
    np.testing.assert_array_equal(got, C0)


@pytest.mark.parametrize("trB", [False, True])
def test_selector_batch3d_4d(trB):
    rng = np.random.default_rng(4)
    P, Q, M, N, K = 6, 2, 26, 4, 26
    A = rng.standard_normal((Q, P, M, K)).astype(np.float32)
    B = rng.standard_normal((Q, P, N, K) if trB else (Q, P, K, N)).astype(np.float32)
    Bm = np.swapaxes(B, -1, -2) if trB else B
    want = np.matmul(A, Bm)
    got4 = ops.selector_batch4d("Sequential", False, trB, A, B, Q, P, M, N, K)
    assert nerr(got4, want) <= 2e-5
    got3 = ops.selector_batch3d("Parallel", False, trB, A[0], B[0], P, M, N, K)
    assert nerr(got3, want[0]) <= 2e-5


@pytest.mark.parametrize("trA", [False, True])
def test_selector_gemv(trA):
    rng = np.random.default_rng(8)
    M, N = 300, 77
    A = rng.standard_normal((M, N)).astype(np.float32)
    X = rng.standard_normal(M if trA else N).astype(np.float32)
    Y0 = rng.standard_normal(N if trA else M).astype(np.float32)
    for alpha, beta in [(1.0, 0.0), (0.5, 2.0)]:
        want = oracle.sgemv(trA, A, X, M, N, alpha, beta, Y0)
        got = ops.selector_gemv("", trA, A, X, M, N, alpha, beta, Y0)
        assert nerr(got, want) <= 2e-5


@pytest.mark.parametrize("case", rc.BMM_ADD_SIGMOID, ids=lambda c: c["name"])
def test_bmm_add_sigmoid_golden(case):
    lhs, rhs, bias = rc.bmm_case_tensors(case)
    want = rc.bmm_reference(lhs, rhs, bias)
    got = ops.kp_fused_batch_matmul_add_sigmoid(lhs, rhs, bias)
    np.testing.assert_allclose(got, want, atol=1e-5, rtol=0)  # tolerance of the reference test
    got_d = ops.kp_fused_batch_matmul_add_sigmoid(_dev(lhs), _dev(rhs), _dev(bias))
    np.testing.assert_allclose(got_d.cpu().numpy(), want, atol=1e-5, rtol=0)


@pytest.mark.parametrize("err", rc.BMM_ADD_SIGMOID_ERRORS, ids=lambda e: e[3][:20])
def test_bmm_add_sigmoid_errors(err):
    ls, rs, bs, msg = err
    with pytest.raises(AnncError) as e:
        ops.kp_fused_batch_matmul_add_sigmoid(np.zeros(ls, np.float32), np.zeros(rs, np.float32),
                                              np.zeros(bs, np.float32))
    assert msg in e.value.message


@pytest.mark.parametrize("m,n,k", [(4096, 512, 13), (1500, 64, 16), (1024, 8, 1)])
def test_small_k_route(m, n, k):
    """First DLRM layer shape class: k <= 16, bias + ReLU, fp32 exact route."""
    rng = np.random.default_rng(k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    b = rng.standard_normal((k, n)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    c = torch.empty((m, n), device="cuda")
    name = device.gemm(_dev(a), _dev(b), c, m=m, n=n, k=k, bias=_dev(bias), activation=1)
    want = np.maximum(a @ b + bias, 0)
    assert name == "simt_fp32"
    assert nerr(c, want) <= 2e-5


@pytest.mark.parametrize("shared_b", [False, True])
@pytest.mark.parametrize("trans_b", [False, True])
def test_strided_batch_on_tensor_cores(shared_b, trans_b):
    """Strided-batch GEMM through rank-3 tensor maps (tails in m, n and k inside every batch)."""
    b, m, n, k = 5, 200, 136, 100
    rng = np.random.default_rng(7)
    A = rng.standard_normal((b, m, k)).astype(np.float32)
    B = rng.standard_normal((1 if shared_b else b, k, n)).astype(np.float32)
    want = np.matmul(A, B)
    Bd = _dev(np.swapaxes(B, 1, 2)) if trans_b else _dev(B)
    c = torch.full((b, m, n), float("nan"), device="cuda")
    name = device.gemm(_dev(A), Bd, c, m=m, n=n, k=k, batch=b, trans_b=trans_b, stride_a=m * k,
                       stride_b=0 if shared_b else k * n, stride_c=m * n)
    assert name in ("tcgen05_tf32", "tcgen05_pair_tf32") and not device.gemm_timed_out()
    assert nerr(c, want) <= 2e-3

"""Pins the oracle's restatements of the XLA custom-call bodies to the reference's own
bodies, compiled here from the reference sources (oracle/xla_ref_shim.cc, `make ref`):
__matmul, __batch_matmul, __matmul_add, __matmul_add_relu (annc/service/cpu/gemm_rewriter.cc
:161-281), __pooling (annc/service/cpu/graph_opt.cc:131-176) and __reduce_mean
(annc/service/cpu/reduce_rewriter.cc:31-46), and the sequential KernelSelector GEMM / Batch3D /
Batch4D / GEMV / ArgMax3D runtime symbols (annc/service/cpu/xla/kernel_selector.cc:31-43, 99-116,
168-178, 234-251, 317-339, 376-389).  Both sides call the same OpenBLAS, so the comparison is
bit for bit.  Skipped where the reference tree was not available at build time."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.skipif(not oracle.xla_ref_available(),
                                reason="reference custom-call bodies not compiled here")


def _rng(seed):
    return np.random.default_rng(seed)


@pytest.mark.parametrize("m,k,n", [(512, 1024, 1024), (128, 416, 1024), (12, 12, 12), (33, 70, 17)])
def test_matmul_family_bit_exact(m, k, n):
    r = _rng(m + k + n)
    a = r.uniform(-1, 1, (m, k)).astype(np.float32)
    b = (r.standard_normal((k, n)) / 32).astype(np.float32)
    addend = np.ascontiguousarray(np.broadcast_to((r.standard_normal(n) * 0.1).astype(np.float32), (m, n)))
    zeros = np.zeros((m, n), np.float32)
    ia, ib, ic = oracle.shape_info(a), oracle.shape_info(b), oracle.shape_info(addend)

    want = oracle.xla_ref_call("matmul", np.empty((m, n), np.float32), [a, b, ia, ib])
    assert np.array_equal(oracle.matmul(a, b), want)

    want = oracle.xla_ref_call("matmul_add", np.empty((m, n), np.float32), [addend, a, b, ic, ia, ib])
    assert np.array_equal(oracle.matmul_add(addend, a, b), want)

    # in = {max operand, addend, lhs, rhs, 4 x info}; the max operand is never read (:279)
    want = oracle.xla_ref_call("matmul_add_relu", np.empty((m, n), np.float32),
                               [zeros, addend, a, b, ic, ic, ia, ib])
    got = oracle.matmul_add_relu(addend, a, b)
    assert np.array_equal(got, want)
    assert (got >= 0).all() and (got == 0).any()


@pytest.mark.parametrize("bt,m,k,n", [(64, 256, 64, 256), (5, 27, 64, 27), (3, 8, 9, 8)])
def test_batch_matmul_bit_exact(bt, m, k, n):
    r = _rng(bt * m + n)
    a = (r.standard_normal((bt, m, k)) / 8).astype(np.float32)
    b = (r.standard_normal((bt, k, n)) / 8).astype(np.float32)
    want = oracle.xla_ref_call("batch_matmul", np.empty((bt, m, n), np.float32),
                               [a, b, oracle.shape_info(a), oracle.shape_info(b)])
    assert np.array_equal(oracle.batch_matmul(a, b), want)


@pytest.mark.parametrize("m,k,n", [(128, 30, 16), (7, 5, 4), (16, 1, 3)])
def test_pooling_bit_exact(m, k, n):
    r = _rng(m * k + n)
    arg = r.integers(-2, 3, (m, k)).astype(np.int64)
    arg[0] = 0          # a row without a positive entry: the output row is zero
    mul_out = r.standard_normal((m, k, n)).astype(np.float32)
    for ss, sl in [((0, 0, 0), (m, k, n)), ((0, 0, 0), (m, max(1, k - 1), n)), ((1 if m > 1 else 0, 0, 0), (m, k, max(1, n - 1)))]:
        ss, sl = np.array(ss, np.int64), np.array(sl, np.int64)
        a_info = np.array([m, k, 1, 0], np.int64)
        m_info = np.array([m, k, n, 2, 1, 0], np.int64)
        want = oracle.xla_ref_call("pooling", np.empty((m, n), np.float32),
                                   [arg, mul_out, ss, sl, a_info, m_info])
        assert np.array_equal(oracle.pooling(arg, mul_out, ss, sl), want)


@pytest.mark.parametrize("m,n", [(64, 37), (1, 5), (1000, 3)])
def test_reduce_mean_bit_exact(m, n):
    r = _rng(m + n)
    value = r.standard_normal(m * n).astype(np.float32)
    shape = np.array([m, n], np.int64)
    axis = np.array([1.0], np.float32)
    want = oracle.xla_ref_call("reduce_mean", np.empty(n, np.float32), [axis, value, axis, shape])
    got = oracle.reduce_mean(value, m, n)
    # the reference divides OpenBLAS' sasum by m; the C restatement adds |x| in index order, so
    # this one is a 1e-6 relative check, not a bit-for-bit one
    np.testing.assert_allclose(got, want, rtol=2e-6, atol=0)


# ---- the sequential KernelSelector runtime symbols (annc/service/cpu/xla/kernel_selector.cc) ----
ks = pytest.mark.skipif(not (oracle.xla_ref_available() and oracle.xla_ref_kernel_selector_available()),
                        reason="reference KernelSelector bodies not compiled here")


@ks
@pytest.mark.parametrize("trA", [False, True])
@pytest.mark.parametrize("trB", [False, True])
@pytest.mark.parametrize("m,n,k,alpha,beta", [(64, 48, 80, 1.0, 0.0), (33, 17, 70, 0.5, 2.0), (8, 128, 1, 2.0, 1.0)])
def test_kernel_selector_gemm_bit_exact(trA, trB, m, n, k, alpha, beta):
    """oracle.sgemm (what the GPU tests of KernelSelectorGEMM* compare with) against the reference's
    own KernelSelectorGEMMSequential: same leading dimensions, same OpenBLAS call."""
    r = _rng(m * n + k + 2 * trA + trB)
    a = r.standard_normal((k, m) if trA else (m, k)).astype(np.float32)
    b = r.standard_normal((n, k) if trB else (k, n)).astype(np.float32)
    c = r.standard_normal((m, n)).astype(np.float32)
    want = oracle.ks_ref_gemm(trA, trB, a, b, m, n, k, alpha, beta, c)
    got = oracle.sgemm(trA, trB, a, b, m, n, k, alpha, beta, c)
    assert np.array_equal(got, want)


@ks
@pytest.mark.parametrize("lead", [(5,), (2, 3)])
@pytest.mark.parametrize("trA,trB", [(False, False), (False, True), (True, False)])
def test_kernel_selector_batch_bit_exact(lead, trA, trB):
    """Batch3D / Batch4D Sequential: one sgemm per slab, alpha 1, beta 0."""
    m, n, k = 12, 20, 9
    r = _rng(len(lead) * 7 + 2 * trA + trB)
    a = r.standard_normal(lead + ((k, m) if trA else (m, k))).astype(np.float32)
    b = r.standard_normal(lead + ((n, k) if trB else (k, n))).astype(np.float32)
    want = oracle.ks_ref_batch(trA, trB, a, b, lead, m, n, k)
    a3, b3 = a.reshape((-1,) + a.shape[-2:]), b.reshape((-1,) + b.shape[-2:])
    got = np.stack([oracle.sgemm(trA, trB, a3[i], b3[i], m, n, k) for i in range(a3.shape[0])])
    assert np.array_equal(got.reshape(lead + (m, n)), want)


@ks
@pytest.mark.parametrize("trA,m,n", [(False, 37, 53), (False, 128, 16), (True, 40, 40), (True, 7, 7)])
def test_kernel_selector_gemv_matches_reference(trA, m, n):
    """The oracle's scalar GEMV against the reference's cblas_sgemv call.  The transposed form is
    compared on square matrices only: the reference passes lda = M there, which is the row pitch
    of the M x N row-major matrix only when M == N (with M < N OpenBLAS rejects the call)."""
    r = _rng(m + 3 * n + trA)
    a = r.standard_normal((m, n)).astype(np.float32)
    x = r.standard_normal(m if trA else n).astype(np.float32)
    y = r.standard_normal(n if trA else m).astype(np.float32)
    for alpha, beta in ((1.0, 0.0), (0.5, 2.0)):
        want = oracle.ks_ref_gemv(trA, a, x, m, n, alpha, beta, y)
        got = oracle.sgemv(trA, a, x, m, n, alpha, beta, y)
        scale = np.abs(want).max() + 1e-30
        assert np.abs(got - want).max() <= 2e-6 * scale  # OpenBLAS' dot-product order differs from the scalar loop


@ks
def test_argmax3d_bit_exact():
    r = _rng(99)
    v = r.integers(-3, 4, (4, 6, 19)).astype(np.float32)   # many ties: the last of equal values wins (>=)
    ix = r.integers(0, 1000, (4, 6, 19)).astype(np.int32)
    for init_v, init_i in ((-np.inf, -1), (2.0, 7), (100.0, 5)):
        wv, wi = oracle.ks_ref_argmax3d(v, ix, init_v, init_i)
        gv, gi = oracle.argmax3d(v, ix, init_v, init_i)
        assert np.array_equal(gv, wv) and np.array_equal(gi, wi)

"""Pins the oracle's restatements of the XLA custom-call bodies to the reference's own
bodies, compiled here from the reference sources (oracle/xla_ref_shim.cc, `make ref`):
__matmul, __batch_matmul, __matmul_add, __matmul_add_relu (annc/service/cpu/gemm_rewriter.cc
:161-281), __pooling (annc/service/cpu/graph_opt.cc:131-176) and __reduce_mean
(annc/service/cpu/reduce_rewriter.cc:31-46).  Both sides call the same OpenBLAS, so the
comparison is bit for bit.  Skipped where the reference tree was not available at build time."""
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

"""The host-pointer side of the ABI: device mirrors of host operands keyed by (pointer, bytes),
uploads skipped when the sampled fingerprint of the host contents is unchanged (weights upload
once; an output that comes back as the next call's input is not uploaded), the re-laid kn4
weight kept with its mirror, and the report of a tensor-core wait that ran out.  The staging
counters of the library (annc_staging_counters) are the evidence."""
import ctypes as C

import numpy as np
import pytest
import torch

from annc_b200 import ops
from annc_b200._lib import lib
from oracle import oracle

pytestmark = pytest.mark.gpu


def counters():
    a, b, c = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
    lib.annc_staging_counters(C.byref(a), C.byref(b), C.byref(c))
    return a.value, b.value, c.value


def nerr(got, want):
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


@pytest.fixture(autouse=True)
def _default_mode():
    lib.annc_set_operand_cache(2, 0)
    yield
    lib.annc_set_operand_cache(2, 0)


def test_second_call_with_the_same_weight_uploads_nothing():
    rng = np.random.default_rng(0)
    m, k, n = 256, 384, 512
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = rng.standard_normal((k, n)).astype(np.float32)
    addend = np.ascontiguousarray(np.broadcast_to(rng.standard_normal(n).astype(np.float32), (m, n)))
    zeros = np.zeros((m, n), np.float32)
    out = np.empty((m, n), np.float32)
    info = [ops.shape_info(addend), ops.shape_info(addend), ops.shape_info(x), ops.shape_info(w)]
    operands = [zeros, addend, x, w] + info
    want = oracle.matmul_add_relu(addend, x, w)

    h0, d0, s0 = counters()
    ops._call_custom("__matmul_add_relu", out, operands)
    h1, d1, s1 = counters()
    assert h1 - h0 == x.nbytes + w.nbytes + addend.nbytes  # the max operand is never read
    assert d1 - d0 == out.nbytes
    assert nerr(out, want) <= 2e-3

    out[:] = -1
    ops._call_custom("__matmul_add_relu", out, operands)
    h2, d2, s2 = counters()
    assert h2 - h1 == 0, "weight, addend and activation are unchanged: nothing to upload"
    assert s2 - s1 == x.nbytes + w.nbytes + addend.nbytes
    assert nerr(out, want) <= 2e-3

    # a new batch in the same buffer: only the activation travels
    x[:] = rng.standard_normal((m, k)).astype(np.float32)
    ops._call_custom("__matmul_add_relu", out, operands)
    h3, _, _ = counters()
    assert h3 - h2 == x.nbytes
    assert nerr(out, oracle.matmul_add_relu(addend, x, w)) <= 2e-3

    # mode 1: constants (weight, addend) are reused, activations always travel
    lib.annc_set_operand_cache(1, 0)
    ops._call_custom("__matmul_add_relu", out, operands)
    h4, _, _ = counters()
    assert h4 - h3 == x.nbytes
    # mode 0: everything travels every time
    lib.annc_set_operand_cache(0, 0)
    ops._call_custom("__matmul_add_relu", out, operands)
    h5, _, _ = counters()
    assert h5 - h4 == x.nbytes + w.nbytes + addend.nbytes
    assert nerr(out, oracle.matmul_add_relu(addend, x, w)) <= 2e-3


def test_output_of_one_call_is_not_uploaded_for_the_next():
    rng = np.random.default_rng(1)
    m, k, n, n2 = 200, 128, 256, 64
    x = rng.standard_normal((m, k)).astype(np.float32)
    w1 = (rng.standard_normal((k, n)) / 8).astype(np.float32)
    w2 = (rng.standard_normal((n, n2)) / 8).astype(np.float32)
    y1 = np.empty((m, n), np.float32)
    y2 = np.empty((m, n2), np.float32)
    for it in range(2):
        ops._call_custom("__matmul", y1, [x, w1, ops.shape_info(x), ops.shape_info(w1)])
        h0, _, s0 = counters()
        ops._call_custom("__matmul", y2, [y1, w2, ops.shape_info(y1), ops.shape_info(w2)])
        h1, _, s1 = counters()
        # y1 sits on the device already; w2 travels on the first round only
        assert h1 - h0 == (w2.nbytes if it == 0 else 0)
        assert s1 - s0 >= y1.nbytes
        want = oracle.matmul(oracle.matmul(x, w1), w2)
        assert nerr(y2, want) <= 4e-3
        # the host touches y1: it must travel again
        y1[3, 5] += 1.0
        y1[:] = y1 * 1.0
    y1[:] = rng.standard_normal((m, n)).astype(np.float32)
    h0, _, _ = counters()
    ops._call_custom("__matmul", y2, [y1, w2, ops.shape_info(y1), ops.shape_info(w2)])
    h1, _, _ = counters()
    assert h1 - h0 == y1.nbytes
    assert nerr(y2, oracle.matmul(y1, w2)) <= 2e-3


def test_layout_matmul_keeps_the_relaid_weight():
    rng = np.random.default_rng(2)
    m, k, n = 256, 704, 384
    x = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((k, n)) / 16).astype(np.float32)
    packed = oracle.kn4_pack(w) if hasattr(oracle, "kn4_pack") else None
    if packed is None:
        offs = oracle.kn4_offsets(k, n)
        packed = np.empty(k * n, np.float32)
        packed[offs] = w.reshape(-1)
        packed = packed.reshape(k, n)
    out = np.empty((m, n), np.float32)
    operands = [x, packed, ops.shape_info(x), ops.shape_info(packed)]
    want = oracle.layout_matmul(x, packed)
    ops._call_custom("__layout_matmul", out, operands)
    assert nerr(out, want) <= 2e-3
    h0, _, _ = counters()
    for _ in range(3):
        out[:] = 0
        ops._call_custom("__layout_matmul", out, operands)
        assert nerr(out, want) <= 2e-3
    h1, _, _ = counters()
    assert h1 - h0 == 0
    # device activations, host weight: the call has nothing to stage and does not wait
    xd = torch.from_numpy(x).cuda()
    od = torch.empty((m, n), device="cuda")
    ops._call_custom("__layout_matmul", od, [xd, packed, ops.shape_info(x), ops.shape_info(packed)])
    torch.cuda.synchronize()
    assert nerr(od.cpu().numpy(), want) <= 2e-3
    assert counters()[0] - h1 == 0


def test_a_wait_that_ran_out_is_reported(capfd):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((256, 256)).astype(np.float32)
    b = rng.standard_normal((256, 256)).astype(np.float32)
    out = np.empty((256, 256), np.float32)
    try:
        assert lib.annc_gemm_debug_set_error_word(1) == 0
        ops._call_custom("__matmul", out, [a, b, ops.shape_info(a), ops.shape_info(b)])
        assert "wait ran out" in lib.annc_last_error().decode()
        assert "__matmul failed" in capfd.readouterr().err
    finally:
        assert lib.annc_gemm_debug_set_error_word(0) == 0
    ops._call_custom("__matmul", out, [a, b, ops.shape_info(a), ops.shape_info(b)])
    assert nerr(out, oracle.matmul(a, b)) <= 2e-3

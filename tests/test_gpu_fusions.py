"""Parity of the softmax, pooling, reduce-mean, arg-max and dot-interaction kernels
with the CPU oracle, through the C ABI."""
import numpy as np
import pytest

from oracle import oracle

pytestmark = pytest.mark.gpu

import torch
from annc_b200 import ops  # noqa: E402  (no fallback: a missing library fails the collection)
from annc_b200 import device, synth  # noqa: E402


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("shape", [(1, 2), (7, 33), (64, 128), (16384, 256), (100, 1000), (5, 1024), (3, 4100)])
def test_softmax(shape):
    rng = np.random.default_rng(shape[1])
    x = (rng.standard_normal(shape) * 3).astype(np.float32)
    want = oracle.softmax(x)
    got = ops.xla_softmax(_dev(x)).cpu().numpy()
    assert np.abs(got - want).max() <= 1e-5  # absolute, on probabilities
    np.testing.assert_allclose(got.sum(-1), 1.0, atol=1e-5)
    if x.size < 100000:
        assert np.abs(ops.xla_softmax(x) - want).max() <= 1e-5


def test_bmm_then_softmax_config():
    """batch_matmul Q[64,256,64] . K^T[64,64,256] then row softmax over the [16384,256] view."""
    q, kt = synth.batch_matmul_softmax_case(0)
    s = ops.xla_batch_matmul(_dev(q), _dev(kt))
    p = ops.xla_softmax(s.view(64 * 256, 256))
    want = oracle.softmax(oracle.batch_matmul(q, kt).reshape(-1, 256))
    assert np.abs(p.cpu().numpy() - want).max() <= 2e-3  # scores may come from the TF32 route


@pytest.mark.parametrize("m,k,n", [(128, 30, 16), (5, 6, 4), (1, 1, 1), (33, 7, 50)])
def test_pooling(m, k, n):
    rng = np.random.default_rng(m)
    arg = rng.integers(-1, 3, (m, k)).astype(np.int64)
    arg[0] = 0  # a row with no positive entry -> zeros
    mo = rng.standard_normal((m, k, n)).astype(np.float32)
    for ss, sl in [([0, 0, 0], [m, k, n]), ([0, 1, 0], [m, k, max(1, n - 1)])]:
        want = oracle.pooling(arg, mo, ss, sl)
        np.testing.assert_array_equal(ops.xla_pooling(arg, mo, ss, sl), want)
        np.testing.assert_array_equal(ops.xla_pooling(_dev(arg), _dev(mo), ss, sl).cpu().numpy(), want)


def test_reduce_mean():
    rng = np.random.default_rng(0)
    m, n = 37, 19
    v = rng.standard_normal(m * n).astype(np.float32)
    want = oracle.reduce_mean(v, m, n)
    np.testing.assert_allclose(ops.xla_reduce_mean(v, m, n), want, rtol=1e-5)


@pytest.mark.parametrize("variant", ["Sequential", "Parallel"])
def test_argmax_last_wins(variant):
    rng = np.random.default_rng(1)
    vals = rng.integers(0, 5, (3, 7, 100)).astype(np.float32)  # many ties
    vals[0, 0, :] = -5.0  # all below init -> init pair survives
    idxs = rng.integers(0, 1000, vals.shape).astype(np.int32)
    wv, wi = oracle.argmax3d(vals, idxs, -1.0, 77)
    gv, gi = ops.selector_argmax3d(variant, vals, idxs, -1.0, 77)
    np.testing.assert_array_equal(gv, wv)
    np.testing.assert_array_equal(gi, wi)


@pytest.mark.parametrize("F,D,math,tol", [(27, 64, 1, 2e-5), (4, 16, 1, 2e-5), (32, 32, 1, 2e-5),
                                          (9, 128, 1, 2e-5), (27, 64, 2, 2e-3), (32, 64, 2, 2e-3),
                                          (2, 64, 2, 2e-3), (9, 64, 0, 2e-3), (5, 64, 2, 2e-3)])
def test_dot_interaction(F, D, math, tol):
    rng = np.random.default_rng(F)
    batch = 333
    z = rng.standard_normal((batch, F, D)).astype(np.float32)
    tri = F * (F - 1) // 2
    width = (D + tri + 3) // 4 * 4
    out = torch.full((batch, width), 9.0, device="cuda")
    device.dot_interaction(_dev(z), out, math)
    assert not device.gemm_timed_out()
    g = oracle.batch_matmul(z, np.swapaxes(z, 1, 2))
    li, lj = np.tril_indices(F, -1)
    want = np.concatenate([z[:, 0, :], g[:, li, lj], np.zeros((batch, width - D - tri), np.float32)], 1)
    got = out.cpu().numpy()
    np.testing.assert_array_equal(got[:, :D], z[:, 0, :])  # the copied row is never rounded
    assert np.abs(got - want).max() <= tol * np.abs(want).max()


@pytest.mark.parametrize("use_map,bf16", [(False, False), (True, False), (True, True)])
def test_masked_sum_of_slot_major_parts_with_output_slots(use_map, bf16):
    """annc_sum_partials_masked_slot_major_dev: parts laid out [slots, rows, width] (a part's place
    follows its key), summed in ascending part order where the mask names them, written to
    out[r, out_slots[slot], :]; the slots of the output that no table maps to stay untouched."""
    import ctypes as C
    from annc_b200._lib import check, lib
    lib.annc_sum_partials_masked_slot_major_dev.argtypes = [
        C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64, C.c_int, C.c_int64, C.c_void_p, C.c_void_p,
        C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
    rng = np.random.default_rng(12)
    parts, rows, slots, width, out_slots_n = 5, 300, 3, 16, 6
    src = rng.standard_normal((parts, slots, rows, width)).astype(np.float32)
    mask = rng.integers(0, 1 << parts, (slots, rows)).astype(np.uint32)
    mask[0, :10] = 0                                   # bags nobody contributes to: zeros
    slot_map = np.array([4, 0, 2], np.int32) if use_map else np.arange(slots, dtype=np.int32)
    width_out = out_slots_n if use_map else slots
    want = np.full((rows, width_out, width), 7.0, np.float32)
    for s in range(slots):
        for r in range(rows):
            acc = None
            for p in range(parts):                     # ascending part order, fp32 adds
                if (mask[s, r] >> p) & 1:
                    acc = src[p, s, r].copy() if acc is None else (acc + src[p, s, r]).astype(np.float32)
            want[r, slot_map[s]] = 0.0 if acc is None else acc
    dsrc = torch.from_numpy(src).cuda()
    dmask = torch.from_numpy(mask.view(np.int32)).cuda()
    dmap = torch.from_numpy(slot_map).cuda()
    out = torch.full((rows, width_out, width), 7.0, device="cuda",
                     dtype=torch.bfloat16 if bf16 else torch.float32)
    check(lib.annc_sum_partials_masked_slot_major_dev(
        C.c_void_p(dsrc.data_ptr()), C.c_void_p(dmask.data_ptr()), C.c_int(parts),
        C.c_int64(slots * rows * width), C.c_int64(rows), C.c_int(slots), C.c_int64(width), None,
        C.c_void_p(dmap.data_ptr()) if use_map else None, C.c_void_p(out.data_ptr()),
        C.c_int64(width_out * width), C.c_int(int(bf16)), None))
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    if bf16:
        ref = torch.from_numpy(want).to(torch.bfloat16).float().numpy()
        assert np.array_equal(got, ref)
    else:
        assert np.array_equal(got, want)

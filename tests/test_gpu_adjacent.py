"""The fused ops next to the pooling ops (padding, action-id gather, sparse reshape, sparse
select): the reference's known-answer tests and error strings, and random parity with the
numpy oracle, through the C ABI.  All results are bit-exact (copies and integer work)."""
import numpy as np
import pytest

from oracle import oracle
from tests.golden import reference_cases as rc

pytestmark = pytest.mark.gpu
import torch
from annc_b200 import ops  # noqa: E402  (no fallback: a missing library fails the collection)
from annc_b200 import AnncError  # noqa: E402


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _np(x):
    return x.cpu().numpy() if hasattr(x, "cpu") else np.asarray(x)


@pytest.mark.parametrize("dims,table,pool,resh", rc.PADDING)
@pytest.mark.parametrize("where", ["host", "device"])
def test_padding_golden(dims, table, pool, resh, where):
    x = np.arange(1, pool * dims + 1, dtype=np.float32).reshape(pool, dims)
    xin = _dev(x) if where == "device" else x
    pad, out = ops.kp_fused_embedding_padding([table, dims], xin, pool, [-1, resh], dims)
    want = np.zeros(table * dims, np.float32)
    want[:pool * dims] = x.reshape(-1)
    assert int(_np(pad)) == table - pool
    np.testing.assert_array_equal(_np(out), want.reshape(table * dims // resh, resh))
    pad, rows = ops.kp_fused_embedding_padding([table, dims], xin, pool, [-1, resh], dims, fast=True)
    assert int(_np(pad)) == table - pool and int(_np(rows)) == table * dims // resh
    wp, wo = oracle.embedding_padding([table, dims], x, pool, [-1, resh])
    np.testing.assert_array_equal(_np(out), wo)


@pytest.mark.parametrize("dims,table,pool,rs,pack,msg", rc.PADDING_ERRORS)
def test_padding_errors(dims, table, pool, rs, pack, msg):
    x = np.ones((pool, dims), np.float32)
    with pytest.raises(AnncError) as e:
        ops.kp_fused_embedding_padding([table, dims], x, pool, rs, pack)
    assert msg in e.value.message


@pytest.mark.parametrize("t1,t2", [(np.int64, np.int32), (np.int32, np.int32), (np.int64, np.int64),
                                   (np.int32, np.int64)])
def test_action_id_gather_golden(t1, t2):
    c = rc.ACTION_ID_GATHER
    out = ops.kp_fused_embedding_action_id_gather(c["indices1"].astype(t1), c["params"],
                                                  c["indices2"].astype(t2), c["pack_dim"], c["pack"])
    np.testing.assert_array_equal(out, c["out"])


def test_action_id_gather_random_and_errors():
    rng = np.random.default_rng(0)
    params = rng.standard_normal((50, 12)).astype(np.float32)
    i1 = rng.integers(0, 50, (30, 4)).astype(np.int64)
    i2 = rng.integers(0, 30, (16, 5)).astype(np.int32)
    want = oracle.action_id_gather(i1, params, i2, 16, 3)
    got = ops.kp_fused_embedding_action_id_gather(_dev(i1), _dev(params), _dev(i2), 16, 3)
    np.testing.assert_array_equal(_np(got), want)
    bad = i1.copy()
    bad[7, 2] = 50
    for args, msg in [((bad, params, i2, 16, 3), "GatherV2 axis=0: index out of range"),
                      ((i1, params, i2, 0, 3), "pack_size must > 0"),
                      ((i1[0], params, i2, 16, 3), "indices1 dims must = 2"),
                      ((i1, params, i2[0], 16, 3), "indices2 dims must = 2"),
                      ((i1, params[0], i2, 16, 3), "params dims must = 2"),
                      ((i1, params, i2, [16], 3), "pack_dim is scalar"),
                      ((i1, params, i2, 16, [3]), "pack const is scalar")]:
        with pytest.raises(AnncError) as e:
            ops.kp_fused_embedding_action_id_gather(*args)
        assert msg in e.value.message


@pytest.mark.parametrize("shape,a,b,c,g,e1,e2,y", rc.SPARSE_SELECT)
def test_sparse_select_golden(shape, a, b, c, g, e1, e2, y):
    A = np.array(a, np.int32).reshape(shape)
    B = np.array(b, np.int32).reshape(shape)
    Cc = np.array(c, np.int32).reshape(shape)
    x, yy, w = ops.kp_fused_sparse_select(A, B, Cc, g, e1, e2)
    np.testing.assert_array_equal(x, np.array(a, np.float32).reshape(-1, 1))
    np.testing.assert_array_equal(yy, np.array(y, np.float32).reshape(-1, 1))
    np.testing.assert_array_equal(w, np.stack([np.array(y, np.float32), np.ones(len(y), np.float32)], 1))
    for bad in ((A, B.reshape(-1)[:-1], Cc, "a and b must match"), (A, B, Cc.reshape(-1)[:-1], "a and c must match")):
        with pytest.raises(AnncError) as e:
            ops.kp_fused_sparse_select(bad[0], bad[1], bad[2], g, e1, e2)
        assert bad[3] in e.value.message


def test_sparse_select_random():
    rng = np.random.default_rng(1)
    a = rng.integers(0, 10, 5000).astype(np.int32)
    b = rng.integers(0, 5, 5000).astype(np.int32)
    wx, wy, ww = oracle.sparse_select(a, b, 4, 1, 3)
    x, y, w = ops.kp_fused_sparse_select(_dev(a), _dev(b), _dev(a), 4, 1, 3)
    np.testing.assert_array_equal(_np(x), wx)
    np.testing.assert_array_equal(_np(y), wy)
    np.testing.assert_array_equal(_np(w), ww)


@pytest.mark.parametrize("sl,begin,new_shape,pack,out_shape", rc.SPARSE_RESHAPE)
def test_sparse_reshape_golden(sl, begin, new_shape, pack, out_shape):
    idx, shp = ops.kp_fused_sparse_reshape(sl, begin, new_shape, pack)
    assert idx.shape == (sl.shape[0], 2)
    np.testing.assert_array_equal(shp, out_shape)
    wi, ws = oracle.sparse_reshape(sl, begin, new_shape, pack)
    np.testing.assert_array_equal(idx, wi)


@pytest.mark.parametrize("sl,begin,new_shape,msg", rc.SPARSE_RESHAPE_ERRORS)
def test_sparse_reshape_errors(sl, begin, new_shape, msg):
    with pytest.raises(AnncError) as e:
        ops.kp_fused_sparse_reshape(sl, begin, new_shape, 1 if "SparseTensor" in msg else 2)
    assert msg in e.value.message
    with pytest.raises(AnncError) as e:
        ops.kp_fused_sparse_reshape(np.zeros((4, 2), np.int64), [0, 1], [2, 4], [2])
    assert "pack_const must be a scalar" in e.value.message


def test_sparse_reshape_random():
    rng = np.random.default_rng(2)
    rows, pack = 6000, 20
    sl = np.stack([rng.integers(0, 9, rows), rng.integers(0, pack, rows)], 1).astype(np.int64)
    for new_shape in ([-1, 8], [rows * pack // 100, 100], [rows, pack], [1, -1]):
        wi, ws = oracle.sparse_reshape(sl, [0, 1], new_shape, pack)
        gi, gs = ops.kp_fused_sparse_reshape(_dev(sl), [0, 1], new_shape, pack)
        np.testing.assert_array_equal(_np(gi), wi)
        np.testing.assert_array_equal(_np(gs), ws)

"""Parity of the CUDA embedding path with the CPU oracle and with the reference's
known-answer tests, through the C ABI.  Bit-exact for ids, rows, COO indices and
for sums over sorted segment ids; 1e-5 relative for the atomic (unsorted) route."""
import numpy as np
import pytest

from oracle import oracle
from tests.golden import reference_cases as rc

pytestmark = pytest.mark.gpu

import torch
from annc_b200 import ops  # noqa: E402  (no fallback: a missing library fails the collection)
from annc_b200 import AnncError, synth  # noqa: E402
from annc_b200.device import BagPlan  # noqa: E402


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("case", rc.SEGMENT_REDUCE, ids=lambda c: c["name"])
@pytest.mark.parametrize("where", ["host", "device"])
def test_segment_reduce_golden(case, where):
    args = [case["data"], case["indices"], case["slice_input"]]
    if where == "device":
        args = [_dev(a) for a in args]
    out, so = ops.kp_fused_sparse_segment_reduce(*args, case["begin"], case["begin_1"], case["combiner"])
    if where == "device":
        out, so = out.cpu().numpy(), so.cpu().numpy()
    np.testing.assert_array_equal(out, case["out"])
    assert int(so) == case["slice_out"]


@pytest.mark.parametrize("mut", rc.SEGMENT_REDUCE_ERRORS, ids=lambda m: m[2][:24])
def test_segment_reduce_errors(mut):
    base = dict(rc.SEGMENT_REDUCE[1])
    base[mut[0]] = mut[1]
    with pytest.raises(AnncError) as e:
        ops.kp_fused_sparse_segment_reduce(base["data"], base["indices"], base["slice_input"],
                                           base["begin"], base["begin_1"], 0)
    assert mut[2] in e.value.message


@pytest.mark.parametrize("dim", [1, 3, 4, 8, 12, 16, 32, 64, 100, 128, 130, 256, 512])
@pytest.mark.parametrize("combiner", [0, 1])
@pytest.mark.parametrize("idx_dtype", [np.int32, np.int64])
def test_segment_reduce_sorted_bit_exact(dim, combiner, idx_dtype):
    rng = np.random.default_rng(dim * 7 + combiner)
    rows, batch = 997, 301
    data = rng.standard_normal((rows, dim)).astype(np.float32)
    lens = rng.integers(0, 7, batch)  # empty bags included
    lens[-1] = max(lens[-1], 1)
    nnz = int(lens.sum())
    seg = np.repeat(np.arange(batch), lens)
    slice_input = np.stack([rng.integers(0, 9, nnz), seg, rng.integers(0, 9, nnz)], 1).astype(np.int64)
    idx = rng.integers(0, rows, nnz).astype(idx_dtype)
    begin, begin_1 = np.array([0, 1], np.int32), np.array([0], np.int32)
    want, want_so = oracle.sparse_segment_reduce(data, idx, slice_input, begin, begin_1, combiner)
    got, so = ops.kp_fused_sparse_segment_reduce(_dev(data), _dev(idx), _dev(slice_input), begin, begin_1, combiner)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert int(so.cpu()) == int(want_so)


@pytest.mark.parametrize("combiner", [0, 1])
def test_segment_reduce_unsorted(combiner):
    rng = np.random.default_rng(5)
    rows, batch, dim, nnz = 500, 64, 64, 3000
    data = rng.standard_normal((rows, dim)).astype(np.float32)
    seg = rng.integers(0, batch, nnz)
    slice_input = np.stack([seg, np.zeros(nnz, np.int64)], 1).astype(np.int64)
    idx = rng.integers(0, rows, nnz).astype(np.int64)
    begin, begin_1 = np.array([0, 0], np.int32), np.array([1], np.int32)
    want, want_so = oracle.sparse_segment_reduce(data, idx, slice_input, begin, begin_1, combiner)
    got, so = ops.kp_fused_sparse_segment_reduce(data, idx, slice_input, begin, begin_1, combiner)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-5 * scale  # fp32 pooling tolerance, order not fixed
    assert int(so) == int(want_so)


def test_segment_reduce_empty_and_single():
    data = np.arange(12, dtype=np.float32).reshape(3, 4)
    begin, b1 = np.array([0, 0], np.int32), np.array([0], np.int32)
    out, so = ops.kp_fused_sparse_segment_reduce(data, np.zeros(0, np.int32), np.zeros((0, 2), np.int64), begin, b1, 0)
    np.testing.assert_array_equal(out, np.zeros((1, 4), np.float32))  # max starts at 0 -> batch 1
    assert int(so) == 1
    out, _ = ops.kp_fused_sparse_segment_reduce(data, np.array([2], np.int32), np.array([[5, 0]], np.int64), begin, b1, 1)
    want = np.zeros((6, 4), np.float32)
    want[5] = data[2]
    np.testing.assert_array_equal(out, want)


def test_segment_reduce_row_out_of_range_is_reported():
    data = np.ones((4, 8), np.float32)
    with pytest.raises(AnncError):
        ops.kp_fused_sparse_segment_reduce(data, np.array([0, 9], np.int32), np.array([[0, 0], [1, 0]], np.int64),
                                           np.array([0, 0], np.int32), np.array([0], np.int32), 0)


@pytest.mark.parametrize("case", rc.SEGMENT_REDUCE_NONZERO, ids=lambda c: c["name"])
def test_segment_reduce_nonzero_golden(case):
    shp, idx, val = ops.kp_fused_sparse_segment_reduce_nonzero(
        case["data"], case["indices"], case["slice_input"], case["begin"], case["combiner"])
    np.testing.assert_array_equal(shp, case["out_shape"])
    np.testing.assert_array_equal(idx, case["out_indices"])
    np.testing.assert_array_equal(val, case["out_values"])


@pytest.mark.parametrize("mut", rc.SEGMENT_REDUCE_NONZERO_ERRORS, ids=lambda m: m[2][:24])
def test_segment_reduce_nonzero_errors(mut):
    base = dict(rc.SEGMENT_REDUCE_NONZERO[1])
    base[mut[0]] = mut[1]
    with pytest.raises(AnncError) as e:
        ops.kp_fused_sparse_segment_reduce_nonzero(base["data"], base["indices"], base["slice_input"], base["begin"], 0)
    assert mut[2] in e.value.message


@pytest.mark.parametrize("rank,combiner", [(1, 0), (1, 1), (2, 0), (2, 1)])
def test_segment_reduce_nonzero_random(rank, combiner):
    rng = np.random.default_rng(rank * 2 + combiner)
    rows, dim, nnz = 211, 12, 5000
    data = rng.integers(-2, 3, (rows, dim)).astype(np.float32)  # many exact zeros in the sums
    if rank == 1:
        data = data[:, 0].copy()
    seg = np.sort(rng.integers(0, 400, nnz))
    seg = seg + 1000  # sparse, large segment ids: first-appearance ranks differ from ids
    slice_input = np.stack([np.zeros(nnz, np.int64), seg], 1).astype(np.int64)
    idx = rng.integers(0, rows, nnz).astype(np.int32)
    begin = np.array([0, 1], np.int32)
    w_shp, w_idx, w_val = oracle.sparse_segment_reduce_nonzero(data, idx, slice_input, begin, combiner)
    shp, gi, gv = ops.kp_fused_sparse_segment_reduce_nonzero(_dev(data), _dev(idx), _dev(slice_input), begin, combiner)
    np.testing.assert_array_equal(shp.cpu().numpy(), w_shp)
    np.testing.assert_array_equal(gi.cpu().numpy(), w_idx)
    np.testing.assert_array_equal(gv.cpu().numpy(), w_val)


@pytest.mark.parametrize("case", rc.FUSED_GATHER, ids=lambda c: c["name"])
def test_fused_gather_golden(case):
    u, inv, rows = ops.kp_fused_gather(case["data"], case["keys"], case["begin"])
    np.testing.assert_array_equal(u, case["unique"])
    np.testing.assert_array_equal(inv, case["indices"])
    np.testing.assert_array_equal(rows, case["out"])


@pytest.mark.parametrize("err", rc.FUSED_GATHER_ERRORS, ids=lambda e: e[3][:20])
def test_fused_gather_errors(err):
    data, keys, begin, msg = err
    with pytest.raises(AnncError) as e:
        ops.kp_fused_gather(data, keys, begin)
    assert msg in e.value.message


def test_fused_gather_random_first_appearance():
    rng = np.random.default_rng(11)
    rows, dim, nnz = 5000, 24, 40000
    data = rng.standard_normal((rows, dim)).astype(np.float32)
    keys = np.stack([rng.integers(0, 7, nnz), rng.zipf(1.3, nnz) % rows], 1).astype(np.int64)
    begin = np.array([0, 1], np.int32)
    wu, wi, wr = oracle.fused_gather(data, keys, begin)
    u, inv, r = ops.kp_fused_gather(_dev(data), _dev(keys), begin)
    np.testing.assert_array_equal(u.cpu().numpy(), wu)
    np.testing.assert_array_equal(inv.cpu().numpy(), wi)
    np.testing.assert_array_equal(r.cpu().numpy(), wr)


@pytest.mark.parametrize("case", rc.DYNAMIC_STITCH, ids=lambda c: c["name"])
def test_dynamic_stitch_golden(case):
    np.testing.assert_array_equal(ops.kp_fused_sparse_dynamic_stitch(case["x"], case["tables"]), case["out"])


@pytest.mark.parametrize("err", rc.DYNAMIC_STITCH_ERRORS, ids=lambda e: e[2][:20])
def test_dynamic_stitch_errors(err):
    x, tables, msg = err
    with pytest.raises(AnncError) as e:
        ops.kp_fused_sparse_dynamic_stitch(x, tables)
    assert msg in e.value.message


def test_dynamic_stitch_random():
    rng = np.random.default_rng(3)
    n_part, dim = 5, 64
    tabs = [rng.standard_normal((int(r), dim)).astype(np.float32) for r in rng.integers(100, 400, n_part)]
    limit = min(t.shape[0] for t in tabs) * n_part
    x = rng.integers(0, limit, (37, 41)).astype(np.int64)
    want = oracle.sparse_dynamic_stitch(x, tabs)
    got = ops.kp_fused_sparse_dynamic_stitch(_dev(x), [_dev(t) for t in tabs])
    np.testing.assert_array_equal(got.cpu().numpy(), want)


EDGE_IDS = np.array([0, 1, 999_999, 1_000_000, 1_000_001, (1 << 62) - 1, (1 << 63) - 1, (1 << 63),
                     (1 << 64) - 1, 0x9E3779B97F4A7C15], np.uint64)


@pytest.mark.parametrize("num_buckets", [1, 2, 7, 1000, 1_000_000])
@pytest.mark.parametrize("bounded", [False, True])
def test_hash_bucket_gather_bit_exact(num_buckets, bounded):
    rng = np.random.default_rng(num_buckets)
    rows = num_buckets if not bounded else max(1, num_buckets // 2)
    rows = min(rows, 50_000)
    nb = num_buckets if bounded else rows
    w = rng.standard_normal((rows, 64)).astype(np.float32)
    fp = np.concatenate([EDGE_IDS, rng.integers(0, 1 << 63, 5000, dtype=np.uint64) * np.uint64(2) + np.uint64(1)])
    empty = rng.random(fp.shape[0]) < 0.1
    want = oracle.embedding_with_hash_bucket(fp, empty, w, nb, bounded=bounded)
    got = ops.kp_fused_embedding_with_hash_bucket(_dev(fp.view(np.int64)).view(torch.int64), _dev(w), nb,
                                                  empty=_dev(empty), bounded=bounded)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    got_h = ops.kp_fused_embedding_with_hash_bucket(fp, w, nb, empty=empty, bounded=bounded)
    np.testing.assert_array_equal(got_h, want)


def test_sparse_embedding_matches_reference_quirk():
    rng = np.random.default_rng(9)
    fp = rng.integers(0, 1 << 63, 300, dtype=np.uint64)
    fp[::7] = np.uint64(50) * fp[::7]  # multiples of num_buckets -> bucket 0 -> value dropped
    empty = rng.random(300) < 0.2
    wi, wv, we, ws = oracle.sparse_embedding(fp, empty, 50)
    gi, gv, ge, gs = ops.kp_fused_sparse_embedding(fp, 50, empty=empty)
    np.testing.assert_array_equal(gi, wi)
    np.testing.assert_array_equal(gv, wv)
    np.testing.assert_array_equal(ge, we)
    np.testing.assert_array_equal(gs, ws)
    assert len(gv) < len(gi)


@pytest.mark.parametrize("dtype", [np.int32, np.int64])
def test_sparse_embedding2(dtype):
    rng = np.random.default_rng(2)
    table = rng.standard_normal((100, 16)).astype(np.float32)
    ids = rng.integers(-20, 140, 1000).astype(dtype)
    want = oracle.sparse_embedding2(ids, table, 0, 100, 0)
    got = ops.sparse_embedding2(_dev(ids), _dev(table), 0, 100, 0)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    np.testing.assert_array_equal(ops.sparse_embedding2(ids, table, 0, 100, 0), want)


@pytest.mark.parametrize("combiner", [0, 1])
def test_grouped_hash_bags_bit_exact(combiner):
    """embed_hash_bucket + segment pooling for several tables in one launch, output
    interleaved as [batch, slots, dim] the way the DLRM pipeline consumes it."""
    rows = [1000, 37, 250_000, 5]
    w = synth.embedding_workload(4, rows, 64, 2048, 20, 1.05)
    slots = len(rows) + 1
    out = torch.full((2048, slots, 64), 7.0, device="cuda")
    plan = BagPlan([_dev(t) for t in w.tables], [_dev(b.raw_ids) for b in w.bags],
                   [_dev(b.slice_input) for b in w.bags], out, 1, 2048, id_kind=2, col=0, combiner=combiner)
    plan.run()
    assert plan.error_bits() == 0
    got = out.cpu().numpy()
    assert (got[:, 0, :] == 7.0).all()  # slot 0 untouched
    for t, (tab, bag) in enumerate(zip(w.tables, w.bags)):
        idx = oracle.hash_bucket(bag.raw_ids.view(np.uint64), rows[t])
        want, _ = oracle.sparse_segment_reduce(tab, idx, bag.slice_input, np.array([0, 0], np.int32),
                                               np.array([0], np.int32), combiner)
        np.testing.assert_array_equal(got[:, t + 1, :], want)


def test_hash_bags_full_size_properties():
    """Config-sized run (26 tables x 1M x 64, batch 16384) checked through properties that
    need no full CPU pass: linearity in the table values and an exact check on a slice."""
    w = synth.hash_bucket_bag_case(seed=0, tables=26, rows=1_000_000, batch=16384)
    tabs = [_dev(t) for t in w.tables]
    ids = [_dev(b.raw_ids) for b in w.bags]
    segs = [_dev(b.slice_input) for b in w.bags]
    out = torch.empty((16384, 26, 64), device="cuda")
    plan = BagPlan(tabs, ids, segs, out, 0, 16384, id_kind=2, col=0, combiner=0)
    plan.run()
    assert plan.error_bits() == 0
    base = out.clone()
    for t in (0, 13, 25):
        idx = oracle.hash_bucket(w.bags[t].raw_ids.view(np.uint64), 1_000_000)
        want, _ = oracle.sparse_segment_reduce(w.tables[t], idx, w.bags[t].slice_input,
                                               np.array([0, 0], np.int32), np.array([0], np.int32), 0)
        np.testing.assert_array_equal(base[:, t, :].cpu().numpy(), want)
    # scaling every table by 2 (exact in fp32) must scale every pooled vector by 2
    for t in tabs:
        t.mul_(2.0)
    plan.run()
    assert torch.equal(out, base * 2.0)


@pytest.mark.parametrize("shards,combiner", [(2, 0), (3, 1), (8, 0)])
def test_row_sharded_exchange_on_one_gpu(shards, combiner):
    """The fused pooling + exchange step with its ranks run one after the other on one GPU:
    each rank pools the lookups it owns (mod partition) into its part of a receive buffer and
    leaves bags it does not contribute to unwritten (the buffer is poisoned with NaN first);
    the owner mask, computed from the ids alone, must name exactly the written parts, and the
    masked rank-order sum must match the unsharded oracle within the fp32 pooling tolerance."""
    from annc_b200.device import BagLaunch, BagPrepass, OwnerMask, sum_partials_masked
    rows = [1000, 37, 50_000, 5, 3]
    B, D = 1024, 64
    T = len(rows)
    w = synth.embedding_workload(11, rows, D, B, 12, 1.05)
    dev = torch.device("cuda")
    ids = [_dev(b.raw_ids) for b in w.bags]
    segs = [_dev(b.slice_input) for b in w.bags]
    pre = BagPrepass(segs, B)
    ws = torch.zeros(pre.ws_bytes, dtype=torch.uint8, device=dev)
    pre.run(ws)
    off_ptr = lambda t: ws.data_ptr() + 512 + t * (B + 1) * 4
    recv = torch.full((shards, B, T, D), float("nan"), device=dev)
    keep = []
    for g in range(shards):
        shard_tabs = [_dev(np.ascontiguousarray(t[g::shards]) if t[g::shards].shape[0] else
                           np.zeros((1, D), np.float32)) for t in w.tables]
        keep.append(shard_tabs)
        entries = [(shard_tabs[t].data_ptr(), len(range(g, rows[t], shards)), rows[t],
                    ids[t].data_ptr(), None, ids[t].shape[0],
                    recv.data_ptr() + ((g * B) * T + t) * D * 4, off_ptr(t)) for t in range(T)]
        launch = BagLaunch(entries, D, B, 2, T * D, dev, combiner=combiner, shard_count=shards,
                           shard_rank=g, exchange=True)
        launch.run()
        assert launch.error_bits() == 0
    owners = OwnerMask([(ids[t].data_ptr(), ids[t].shape[0], rows[t], off_ptr(t)) for t in range(T)],
                       B, shards, dev)
    owners.run()
    mask = owners.mask.cpu().numpy().reshape(T, B)
    written = ~torch.isnan(recv[:, :, :, 0]).cpu().numpy()  # [shards, B, T]
    for t, bag in enumerate(w.bags):
        bucket = bag.raw_ids.view(np.uint64) % np.uint64(rows[t])
        want_mask = np.zeros(B, np.int64)
        np.bitwise_or.at(want_mask, bag.slice_input[:, 0], 1 << (bucket % np.uint64(shards)).astype(np.int64))
        np.testing.assert_array_equal(mask[t], want_mask)
        for g in range(shards):
            np.testing.assert_array_equal(written[g, :, t], (want_mask >> g) & 1 == 1)
    out = torch.full((B, T, D), 3.0, device=dev)
    sum_partials_masked(recv.data_ptr(), owners.mask, shards, B * T * D, B, T, D, out.data_ptr(), T * D)
    got = out.cpu().numpy()
    for t, (tab, bag) in enumerate(zip(w.tables, w.bags)):
        idx = oracle.hash_bucket(bag.raw_ids.view(np.uint64), rows[t])
        want, _ = oracle.sparse_segment_reduce(tab, idx, bag.slice_input, np.array([0, 0], np.int32),
                                               np.array([0], np.int32), combiner)
        scale = max(float(np.abs(want).max()), 1e-30)
        assert float(np.abs(got[:, t, :] - want).max()) / scale <= 1e-5


@pytest.mark.parametrize("num_buckets", [1, 2, 3, 7, 10**6, 2**31 - 1, 2**32 + 1, 2**62 + 3, 2**63 - 1])
def test_division_free_modulo_is_exact(num_buckets):
    """The kernels compute `fingerprint % num_buckets` with a reciprocal multiply and a
    correction step.  The owner-mask kernel exposes (id % num_buckets) % G without needing a
    table of num_buckets rows; three coprime G pin the bucket on edge and random ids."""
    from annc_b200.device import OwnerMask
    rng = np.random.default_rng(3)
    d = num_buckets
    edge = [0, 1, d - 1, d, d + 1, 2 * d - 1, 2 * d, 2**62 - 1, 2**63 - 1, 2**63, 2**64 - 1,
            2**64 - d, (2**64 - 1) // d * d, (2**64 - 1) // d * d - 1]
    ids = np.array([e % 2**64 for e in edge if e >= 0], dtype=np.uint64)
    ids = np.concatenate([ids, rng.integers(0, 2**64, 4096, dtype=np.uint64)])
    n = ids.shape[0]
    ids_d = _dev(ids.view(np.int64))
    off = _dev(np.arange(n + 1, dtype=np.int32))  # one lookup per bag
    want_bucket = np.array([int(x) % d for x in ids.tolist()], dtype=object)
    for g in (32, 31, 29):
        m = OwnerMask([(ids_d.data_ptr(), n, d, off.data_ptr())], n, g, torch.device("cuda"))
        m.run()
        got = m.mask.cpu().numpy().view(np.uint32)
        want = np.array([1 << (int(b) % g) for b in want_bucket], dtype=np.uint32)
        np.testing.assert_array_equal(got, want)

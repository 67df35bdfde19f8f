"""annc_embed_bags_static_dev: the embedding-bag entry point for callers that cannot
hand the library a workspace (no device allocation allowed where they run, e.g. inside
an allocator or stream callback of a host framework, or under a fixed memory budget).
It must give exactly what annc_embed_bags_dev gives, call after call, although every
call reuses the same built-in scratch array.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

import torch
import annc_b200  # noqa: F401,E402  (no fallback: a missing library fails the collection)
from annc_b200 import AnncError, synth  # noqa: E402
from annc_b200._lib import BagTable, check, lib  # noqa: E402
from annc_b200.device import BagPlan  # noqa: E402


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run_static(plan: BagPlan, out: torch.Tensor, slot0: int, err: torch.Tensor):
    desc = (BagTable * plan.n)()
    for t in range(plan.n):
        for f, _ in BagTable._fields_:
            setattr(desc[t], f, getattr(plan.desc[t], f))
        desc[t].out = out.data_ptr() + (slot0 + t) * plan.dim * 4
    check(lib.annc_embed_bags_static_dev(
        desc, C.c_int(plan.n), C.c_int64(plan.dim), C.c_int(plan.id_kind), C.c_int64(plan.ncols),
        C.c_int32(plan.col), C.c_int(plan.combiner), C.c_int64(plan.batch),
        C.c_int64(plan.out_stride), C.c_void_p(err.data_ptr()),
        C.c_void_p(torch.cuda.current_stream().cuda_stream)))


def test_static_scratch_matches_workspace_entry_twice():
    batch = 4096
    outs = []
    for call, (seed, combiner) in enumerate([(21, 0), (22, 1)]):
        # the second call has other bag lengths, another combiner and one unsorted table,
        # so stale offsets or marks left in the shared array by the first call would show
        w = synth.embedding_workload(seed, [5000, 64, 120_000], 64, batch, 20, 1.05)
        segs = [b.slice_input.copy() for b in w.bags]
        if call == 1:
            segs[1] = segs[1][::-1].copy()
        tabs = [_dev(t) for t in w.tables]
        ids = [_dev(b.raw_ids if i != 1 or call == 0 else b.raw_ids[::-1].copy())
               for i, b in enumerate(w.bags)]
        dsegs = [_dev(s) for s in segs]
        want = torch.zeros((batch, 4, 64), device="cuda")
        plan = BagPlan(tabs, ids, dsegs, want, 1, batch, id_kind=2, col=0, combiner=combiner)
        plan.run()
        assert plan.error_bits() == 0
        got = torch.zeros((batch, 4, 64), device="cuda")
        err = torch.full((1,), -1, dtype=torch.int32, device="cuda")
        _run_static(plan, got, 1, err)
        torch.cuda.synchronize()
        assert int(err.item()) == 0
        if call == 0:
            assert torch.equal(got, want)  # sorted ids: bit-exact
        else:
            # table 1 took the atomic route (order of adds not fixed): fp32 pooling tolerance
            assert torch.equal(got[:, [1, 3]], want[:, [1, 3]])
            scale = want[:, 2].abs().max().item()
            assert (got[:, 2] - want[:, 2]).abs().max().item() <= 1e-5 * scale
        outs.append(got)
    assert not torch.equal(outs[0], outs[1])


def test_static_scratch_rejects_oversize():
    d = (BagTable * 1)()
    with pytest.raises(AnncError) as e:
        check(lib.annc_embed_bags_static_dev(d, C.c_int(64), C.c_int64(64), C.c_int(2), C.c_int64(2),
                                             C.c_int32(0), C.c_int(0), C.c_int64(131072),
                                             C.c_int64(64), None, None))
    assert e.value.code == 102 and "exceeds the built-in scratch" in e.value.message


def test_static_scratch_allocates_nothing_and_reports_bad_rows():
    """The property the entry point exists for: once the library is warm, calls leave the
    device's free memory where it was.  Also: a row outside its table is reported through
    error_bits_dev, and a sorted call right after an unsorted one on the shared array is exact."""
    batch = 2048
    w = synth.embedding_workload(31, [3000, 50], 64, batch, 12, 1.05)
    tabs = [_dev(t) for t in w.tables]
    ids = [_dev(b.raw_ids) for b in w.bags]
    segs = [_dev(b.slice_input) for b in w.bags]
    want = torch.zeros((batch, 2, 64), device="cuda")
    plan = BagPlan(tabs, ids, segs, want, 0, batch, id_kind=2, col=0, combiner=0)
    plan.run()
    got = torch.zeros_like(want)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    # an unsorted call first, so that the shared array holds counters, not offsets
    rsegs = [_dev(b.slice_input[::-1].copy()) for b in w.bags]
    rids = [_dev(b.raw_ids[::-1].copy()) for b in w.bags]
    rplan = BagPlan(tabs, rids, rsegs, want.clone(), 0, batch, id_kind=2, col=0, combiner=0)
    _run_static(rplan, torch.zeros_like(want), 0, err)
    _run_static(plan, got, 0, err)  # warm: symbol address looked up, kernels loaded
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        _run_static(plan, got, 0, err)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "annc_embed_bags_static_dev changed the device's free memory"
    assert torch.equal(got, want) and int(err.item()) == 0
    # row ids instead of fingerprints, one of them outside its table
    rows = [_dev((b.raw_ids.view(np.uint64) % np.uint64(t.shape[0])).astype(np.int64)) for b, t in zip(w.bags, w.tables)]
    rows[1][7] = 50
    bad = BagPlan(tabs, rows, segs, torch.zeros_like(want), 0, batch, id_kind=1, col=0, combiner=0)
    _run_static(bad, torch.zeros_like(want), 0, err)
    torch.cuda.synchronize()
    assert int(err.item()) & 1


def test_static_scratch_more_tables_than_one_launch_takes():
    """More than 120 tables (the limit of one grouped launch) inside the scratch limit: the entry
    point walks them in groups on the shared array."""
    n, batch, dim = 130, 64, 16
    rng = np.random.default_rng(5)
    tabs = [_dev(rng.standard_normal((40, dim)).astype(np.float32)) for _ in range(n)]
    lens = rng.integers(0, 4, (n, batch))
    ids, segs = [], []
    for t in range(n):
        seg = np.repeat(np.arange(batch, dtype=np.int64), lens[t])
        ids.append(_dev(rng.integers(0, 1 << 40, seg.shape[0]).astype(np.int64)))
        segs.append(_dev(np.stack([seg, np.zeros_like(seg)], axis=1).reshape(-1, 2)))
    want = torch.full((batch, n, dim), 5.0, device="cuda")
    plan = BagPlan(tabs, ids, segs, want, 0, batch, id_kind=2, col=0, combiner=0)
    plan.run()
    got = torch.full((batch, n, dim), -5.0, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    _run_static(plan, got, 0, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0 and torch.equal(got, want)

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

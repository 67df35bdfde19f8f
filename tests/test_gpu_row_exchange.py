"""The row-sharded exchange (annc_row_exchange_*) with its ranks emulated on one GPU: every
rank is an object of its own with its own "peer" buffer (plain device memory here), and the
three phases of a step are run rank by rank — begin on all, pool on all, finish on all — so
every flag a rank waits for has been stored before the wait is launched.  Pooled vectors are
checked against the unsharded CPU oracle (fp32 pooling tolerance 1e-5 relative) and the record
lists against a numpy statement of the partition."""
import numpy as np
import pytest
import torch

from annc_b200 import row_exchange as rx
from annc_b200 import synth
from oracle import oracle

pytestmark = pytest.mark.gpu


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _oracle_pooled(w, rows, combiner):
    out = []
    for t, (tab, bag) in enumerate(zip(w.tables, w.bags)):
        idx = oracle.hash_bucket(bag.raw_ids.view(np.uint64), rows[t])
        want, _ = oracle.sparse_segment_reduce(tab, idx, bag.slice_input, np.array([0, 0], np.int32),
                                               np.array([0], np.int32), combiner)
        out.append(want)
    return out


class Emulated:
    """`world` ranks of one exchange on the current device.  works[r] is rank r's batch."""

    def __init__(self, world, rows, dim, batch, works, hot_k, combiner, tables_np, also=()):
        self.world, self.T, self.B, self.D = world, len(rows), batch, dim
        self.keep = []
        sized = list(works) + list(also)  # every batch the exchange will be given
        nnz_max = max(int(sum(b.raw_ids.shape[0] for b in w.bags)) for w in sized)
        per_table = max(int(b.raw_ids.shape[0]) for w in sized for b in w.bags)
        hot_rows = [works[0].bags[t].popular_rows(hot_k[t], rows[t]) for t in range(self.T)]
        self.hot_rows = hot_rows
        cfgs = []
        for r in range(world):
            tabs = []
            for t in range(self.T):
                held = np.concatenate([tables_np[t][r::world], tables_np[t][hot_rows[t]]])  # shard, then hot rows
                shard = _dev(held) if held.shape[0] else None
                full = hot_rows[t].shape[0] == rows[t]
                hr = _dev(hot_rows[t]) if (hot_rows[t].shape[0] and not full) else None
                self.keep += [shard, hr]
                tabs.append(dict(shard=shard.data_ptr() if shard is not None else 0,
                                 local_rows=len(range(r, rows[t], world)), rows=rows[t],
                                 hot_rows=hr.data_ptr() if hr is not None else 0,
                                 hot_count=int(hot_rows[t].shape[0])))
            cfgs.append(rx.make_config(world, r, tabs, dim, batch, nnz_max, per_table, combiner=combiner))
        nbytes = rx.peer_bytes(cfgs[0][0])
        self.bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
        ptrs = [b.data_ptr() for b in self.bufs]
        self.ex = [rx.RowExchange(c, k, ptrs) for c, k in cfgs]
        self.inputs = []
        for w in works:
            ids = [_dev(b.raw_ids) for b in w.bags]
            segs = [_dev(b.slice_input) for b in w.bags]
            self.keep += ids + segs
            self.inputs.append(rx.StepInputs([i.data_ptr() for i in ids], [s.data_ptr() for s in segs],
                                             [int(i.shape[0]) for i in ids]))

    def step(self, outs, bf16=False):
        for r in range(self.world):
            self.ex[r].begin(self.inputs[r])
        for r in range(self.world):
            self.ex[r].pool()
        for r in range(self.world):
            self.ex[r].finish(outs[r].data_ptr(), self.T * self.D, bf16)

    def close(self):
        torch.cuda.synchronize()
        for e in self.ex:
            e.destroy()


@pytest.mark.parametrize("world,combiner,hot,dim", [(1, 0, 0, 64), (2, 0, 0, 64), (3, 1, 0, 64), (8, 0, 0, 64),
                                                    (8, 1, 64, 64), (4, 0, 1 << 30, 64), (8, 0, 300, 128),
                                                    (2, 1, 16, 32), (5, 0, 100, 16), (4, 1, 50, 256)])
def test_emulated_ranks_match_oracle(world, combiner, hot, dim):
    rows = [1000, 37, 50_000, 5, 3]
    B = 512
    T = len(rows)
    works = [synth.embedding_workload(21, rows, dim, B, 40, 1.05, input_seed=300 + r) for r in range(world)]
    hot_k = [hot, 0, hot, hot, 0][:T]
    em = Emulated(world, rows, dim, B, works, hot_k, combiner, works[0].tables)
    outs = [torch.full((B, T, dim), 7.0, device="cuda") for _ in range(world)]
    for it in range(2):  # a second step reuses lists, masks and slabs
        em.step(outs)
        for r in range(world):
            assert em.ex[r].error_bits() == 0
            got = outs[r].cpu().numpy()
            want = _oracle_pooled(works[r], rows, combiner)
            for t in range(T):
                scale = max(float(np.abs(want[t]).max()), 1e-30)
                err = float(np.abs(got[:, t, :] - want[t]).max()) / scale
                assert err <= 1e-5, (it, r, t, err)
            if world == 1:  # one rank: lookup order, hence the reference's sums bit for bit
                for t in range(T):
                    if combiner == 0:
                        assert np.array_equal(got[:, t, :], want[t])
    # list sizes against numpy: records pooled per source, parts per owner
    recs, parts = em.ex[0].stats()
    for q in range(world):
        n = 0
        for t, bag in enumerate(works[q].bags):
            bucket = (bag.raw_ids.view(np.uint64) % np.uint64(rows[t])).astype(np.int64)
            is_hot = np.isin(bucket, em.hot_rows[t])
            owner = np.where(is_hot, q, bucket % world)
            n += int((owner == 0).sum())
        assert recs[q] == n
    want_parts = [0] * world
    for t, bag in enumerate(works[0].bags):
        bucket = (bag.raw_ids.view(np.uint64) % np.uint64(rows[t])).astype(np.int64)
        owner = np.where(np.isin(bucket, em.hot_rows[t]), 0, bucket % world)
        for g in range(world):
            want_parts[g] += int(np.unique(bag.slice_input[owner == g, 0]).shape[0])
    assert parts == want_parts
    em.close()


def test_one_step_of_lookahead():
    """begin() of step i + 1 before pool() and finish() of step i (the split of the next batch
    runs under the pooling of this one): lists, bounds, masks and receive slabs alternate
    between two sets, so every step must still match the oracle although its successor's lists
    were already published.  Two different batches alternate; mean pooling exercises the bag
    offsets too."""
    rows = [3000, 41, 20_000]
    B, D, world, T = 256, 64, 4, 3
    batches = [[synth.embedding_workload(8, rows, D, B, 30, 1.05, input_seed=500 + 10 * v + r) for r in range(world)]
               for v in range(2)]
    em = Emulated(world, rows, D, B, batches[0], [50, 0, 500], 1, batches[0][0].tables, also=batches[1])
    inputs = [em.inputs]
    ids2 = [[_dev(b.raw_ids) for b in w.bags] for w in batches[1]]
    segs2 = [[_dev(b.slice_input) for b in w.bags] for w in batches[1]]
    inputs.append([rx.StepInputs([i.data_ptr() for i in ids], [s.data_ptr() for s in segs],
                                 [int(i.shape[0]) for i in ids]) for ids, segs in zip(ids2, segs2)])
    want = [[_oracle_pooled(batches[v][r], rows, 1) for r in range(world)] for v in range(2)]
    outs = [torch.zeros((B, T, D), device="cuda") for _ in range(world)]
    steps = 5
    for r in range(world):
        em.ex[r].begin(inputs[0][r])
    for k in range(steps):
        if k + 1 < steps:
            for r in range(world):
                em.ex[r].begin(inputs[(k + 1) % 2][r])
        for r in range(world):
            em.ex[r].pool()
        for r in range(world):
            em.ex[r].finish(outs[r].data_ptr(), T * D)
        for r in range(world):
            assert em.ex[r].error_bits() == 0
            got = outs[r].cpu().numpy()
            for t in range(T):
                w = want[k % 2][r][t]
                assert float(np.abs(got[:, t, :] - w).max()) / max(float(np.abs(w).max()), 1e-30) <= 1e-5, (k, r, t)
    # a third begin before the oldest step has finished is refused
    for r in range(world):
        em.ex[r].begin(inputs[0][r])
        em.ex[r].begin(inputs[1][r])
    with pytest.raises(Exception) as e:
        em.ex[0].begin(inputs[0][0])
    assert "one step ahead" in str(e.value)
    for _ in range(2):
        for r in range(world):
            em.ex[r].pool()
        for r in range(world):
            em.ex[r].finish(outs[r].data_ptr(), T * D)
    em.close()


def test_bf16_output_and_full_size_bags():
    """bf16 output (the input of a BF16 MLP) and bags far longer than a chunk of records."""
    rows = [20_000, 64]
    B, D, world = 256, 128, 4
    works = [synth.embedding_workload(5, rows, D, B, 300, 1.2, input_seed=40 + r) for r in range(world)]
    em = Emulated(world, rows, D, B, works, [128, 0], 1, works[0].tables)
    outs = [torch.zeros((B, 2, D), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    em.step(outs, bf16=True)
    for r in range(world):
        assert em.ex[r].error_bits() == 0
        want = _oracle_pooled(works[r], rows, 1)
        got = outs[r].float().cpu().numpy()
        for t in range(2):
            ref = torch.from_numpy(want[t]).to(torch.bfloat16).float().numpy()
            assert np.abs(got[:, t, :] - ref).max() <= 2 ** -8 * max(np.abs(ref).max(), 1e-30)
    em.close()


def test_errors_are_reported():
    rows = [100, 50]
    B, D = 64, 64
    w = synth.embedding_workload(9, rows, D, B, 5, 1.05)
    em = Emulated(1, rows, D, B, [w], [0, 0], 0, w.tables)
    out = [torch.zeros((B, 2, D), device="cuda")]
    # unsorted segment ids
    seg = w.bags[0].slice_input.copy()
    seg[[0, -1]] = seg[[-1, 0]]
    bad = _dev(seg)
    good = em.inputs[0]
    ids = [_dev(b.raw_ids) for b in w.bags]
    segs = [bad, _dev(w.bags[1].slice_input)]
    em.inputs[0] = rx.StepInputs([i.data_ptr() for i in ids], [s.data_ptr() for s in segs],
                                 [int(i.shape[0]) for i in ids])
    em.step(out)
    assert em.ex[0].error_bits() & rx.ERR_UNSORTED
    em.ex[0].clear_errors()
    # a segment id outside the batch
    seg2 = w.bags[0].slice_input.copy()
    seg2[-1, 0] = B + 3
    segs = [_dev(seg2), segs[1]]
    em.inputs[0] = rx.StepInputs([i.data_ptr() for i in ids], [s.data_ptr() for s in segs],
                                 [int(i.shape[0]) for i in ids])
    em.step(out)
    assert em.ex[0].error_bits() & rx.ERR_SEGMENT
    em.ex[0].clear_errors()
    em.inputs[0] = good
    em.step(out)
    assert em.ex[0].error_bits() == 0
    em.close()


def test_wait_gives_up_after_its_limit():
    """A rank whose peer never arrives: the wait runs out after the limit (50 ms here), the
    step completes, the time-out is reported and the context stays usable."""
    rows = [100]
    B, D = 32, 64
    works = [synth.embedding_workload(3, rows, D, B, 4, 1.05, input_seed=r) for r in range(2)]
    em = Emulated(2, rows, D, B, works, [0], 0, works[0].tables)
    em.ex[0].set_timeout_ms(50)
    out = torch.zeros((B, 1, D), device="cuda")
    em.ex[0].begin(em.inputs[0])   # rank 1 never begins: its flag stays behind
    em.ex[0].pool()
    em.ex[0].finish(out.data_ptr(), D)
    with pytest.raises(Exception) as e:
        em.ex[0].error_bits()
    assert "did not arrive" in str(e.value)
    assert em.ex[0].error_bits(raise_on_timeout=False) & rx.ERR_TIMEOUT
    assert torch.isfinite(out).all()  # the context still answers
    em.close()

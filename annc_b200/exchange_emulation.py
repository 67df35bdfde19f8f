"""One-GPU emulation of the row exchange: `world` exchange objects in one process, every
"peer" buffer on the same device, each rank with its own batch of the DLRM workload (shared
popularity maps), the phases run rank by rank (begin on all, pool on all, finish on all).
Prints the per-phase kernel times of every emulated rank (CUDA events inside the library) and
what would cross NVLink.  For sizing a deployment, or for profiling the exchange's kernels,
without a multi-GPU box:

    python -m annc_b200.exchange_emulation [world=8] [hot_rows=65536] [batch=65536] [max_rows=1e7]

No NVLink is involved: the pooling kernel's time here is its gather time, the floor of what it
takes on real GPUs.  Parity of emulated ranks against the CPU oracle is the job of
tests/test_gpu_row_exchange.py.
"""
from __future__ import annotations

import sys

import numpy as np
import torch

from . import row_exchange as rx
from . import synth


def _rank_batches(model, world: int, batch: int):
    """Rank 0 takes the model's own batch; the others draw theirs from the same per-table
    popularity maps with their own seeds (what bench.py's ranks do)."""
    T = len(model.table_rows)
    emb_seed = int(np.random.default_rng(0).spawn(3)[2].integers(0, 2 ** 31))

    def bags_for(input_seed):
        ch = np.random.default_rng(emb_seed).spawn(2 * T)
        own = np.random.default_rng(input_seed).spawn(T)
        return [synth._bag_inputs(own[t], batch, 20, 1.05, table_rng=ch[2 * t + 1]) for t in range(T)]

    works = [model.emb.bags] + [bags_for(1000 + r) for r in range(1, world)]
    assert np.array_equal(works[0][0].lut, works[-1][0].lut), "ranks must share the popularity maps"
    return works


def run(world: int = 8, hot_rows: int = 65536, batch: int = 65536, max_rows: float = 1e7, dim: int = 64,
        steps: int = 4):
    model = synth.dlrm_model(seed=0, batch=batch, input_seed=1000, max_rows=max_rows)
    rows = model.table_rows
    T = len(rows)
    works = _rank_batches(model, world, batch)
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    hot = [model.emb.bags[t].popular_rows(hot_rows, rows[t]) for t in range(T)]
    hot_dev = [dev(h) if 0 < h.shape[0] < rows[t] else None for t, h in enumerate(hot)]
    print("replicated rows: %.2f GB per rank" % (sum(h.shape[0] for h in hot) * dim * 4 / 1e9), flush=True)

    keep, cfgs = [], []
    nnz_max = max(sum(b.raw_ids.shape[0] for b in w) for w in works)
    per_table = max(b.raw_ids.shape[0] for w in works for b in w)
    for r in range(world):
        tabs = []
        for t in range(T):
            shard = model.emb.tables[t][r::world]
            both = dev(np.concatenate([shard, model.emb.tables[t][hot[t]]]))
            keep.append(both)
            tabs.append(dict(shard=both.data_ptr(), local_rows=shard.shape[0], rows=rows[t],
                             hot_rows=hot_dev[t].data_ptr() if hot_dev[t] is not None else 0,
                             hot_count=int(hot[t].shape[0])))
        cfgs.append(rx.make_config(world, r, tabs, dim, batch, nnz_max, per_table))
    nbytes = rx.peer_bytes(cfgs[0][0])
    print("peer buffer: %.2f GB per rank" % (nbytes / 1e9), flush=True)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    ex = [rx.RowExchange(c, k, [b.data_ptr() for b in bufs]) for c, k in cfgs]
    inputs = []
    for w in works:
        ids = [dev(b.raw_ids) for b in w]
        segs = [dev(b.slice_input) for b in w]
        keep += ids + segs
        inputs.append(rx.StepInputs([i.data_ptr() for i in ids], [s.data_ptr() for s in segs],
                                    [int(i.shape[0]) for i in ids]))
    outs = [torch.zeros((batch, T, dim), device="cuda") for _ in range(world)]
    for e in ex:
        e.set_profiling(True)
    for _ in range(steps):
        for r in range(world):
            ex[r].begin(inputs[r])
        for r in range(world):
            ex[r].pool()
        for r in range(world):
            ex[r].finish(outs[r].data_ptr(), T * dim)
        torch.cuda.synchronize()
    for r in range(world):
        assert ex[r].error_bits() == 0, r
    # the barrier phases contain the other ranks' work in this emulation: split, pool, sum only
    ph = np.array([ex[r].phase_ms() for r in range(world)])
    print("world", world, "replicated rows per table", hot_rows, "batch", batch)
    print("split ms per rank", np.round(ph[:, 0], 3))
    print("pool  ms per rank", np.round(ph[:, 2], 3))
    print("sum   ms per rank", np.round(ph[:, 4], 3))
    recs, parts = ex[0].stats()
    print("rank 0: records per source", recs, "parts per owner", parts)
    print("remote parts per bag %.3f, over NVLink per rank and step %.1f MB"
          % (sum(parts[1:]) / (batch * T), (sum(parts[1:]) * dim * 4 + sum(recs[1:]) * 8) / 1e6))
    return ph


if __name__ == "__main__":
    a = sys.argv[1:]
    run(int(a[0]) if len(a) > 0 else 8, int(a[1]) if len(a) > 1 else 65536,
        int(a[2]) if len(a) > 2 else 65536, float(a[3]) if len(a) > 3 else 1e7)

"""World-size-2 gloo ranks on CPU: the partitioning logic of annc_b200.sharded.ShardPlan,
with the CPU oracle standing in for the kernels.  Row mode: every rank pools the lookups it
owns for the global batch, partial sums are exchanged and added in rank order, and the
result must match the unsharded oracle within the fp32 pooling tolerance.  Table mode: the
send/receive counts of the two all-to-alls must agree between ranks and the pooled vectors
must be bit-exact."""
import os
import sys

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _pool(tables, rows, ids, segs, batch, dim):
    from oracle import oracle
    out = np.zeros((batch, len(tables), dim), np.float32)
    oracle.embed_bags_tables(tables, rows, ids, segs, batch, dim, out, len(tables), 0)
    return out


def _worker(rank, world, port, q):
    import torch
    from annc_b200 import synth
    from annc_b200.sharded import ShardPlan
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, D, rows = 64, 16, [1000, 37, 5000, 3, 250]
        w = synth.embedding_workload(9, rows, D, B, 12, 1.05, threads=1, input_seed=50 + rank)
        T = len(rows)
        nnz_all = [None] * world
        dist.all_gather_object(nnz_all, [int(b.raw_ids.shape[0]) for b in w.bags])
        want = _pool(w.tables, rows, [b.raw_ids for b in w.bags], [b.slice_input for b in w.bags], B, D)

        # ---- row mode
        plan = ShardPlan("row", world, rank, rows, np.array(nnz_all))
        L = plan.gathered_len()
        ids = np.zeros(L, np.int64)
        seg = np.zeros((L, 2), np.int64)
        flat_ids = np.concatenate([b.raw_ids for b in w.bags])
        flat_seg = np.concatenate([b.slice_input for b in w.bags])
        ids[:flat_ids.shape[0]] = flat_ids
        seg[:flat_seg.shape[0]] = flat_seg
        g_ids = [torch.zeros(L, dtype=torch.int64) for _ in range(world)]
        g_seg = [torch.zeros((L, 2), dtype=torch.int64) for _ in range(world)]
        dist.all_gather(g_ids, torch.from_numpy(ids))
        dist.all_gather(g_seg, torch.from_numpy(seg))
        partial = np.zeros((world, B, T, D), np.float32)
        for s in range(world):
            lt, li, ls, lr = [], [], [], []
            for t in range(T):
                off, n = plan.gathered_offset(s, t), int(plan.nnz[s, t])
                raw = g_ids[s].numpy()[off:off + n]
                sg = g_seg[s].numpy()[off:off + n]
                bucket = raw.astype(np.uint64) % np.uint64(rows[t])
                own = (bucket % np.uint64(world)) == np.uint64(rank)
                local = (bucket[own] // np.uint64(world)).astype(np.int64)
                shard = plan.local_shard(w.tables[t])
                assert shard.shape[0] == plan.local_rows(t)
                assert local.size == 0 or local.max() < shard.shape[0]
                lt.append(shard if shard.shape[0] else np.zeros((1, D), np.float32))
                lr.append(max(shard.shape[0], 1) * 10 ** 9)  # local ids are already rows: modulus is a no-op
                li.append(local)
                ls.append(np.ascontiguousarray(sg[own]))
            partial[s] = _pool(lt, lr, li, ls, B, D)
        gathered = [torch.zeros((world, B, T, D)) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(partial))  # stands in for the all-to-all
        got = np.zeros((B, T, D), np.float32)
        for s in range(world):  # ascending rank order, like annc_sum_partials_dev
            got = got + gathered[s].numpy()[rank]
        err_row = float(np.abs(got - want).max() / np.abs(want).max())

        # ---- table mode
        tp = ShardPlan("table", world, rank, rows, np.array(nnz_all))
        counts = [None] * world
        dist.all_gather_object(counts, (tp.send_counts(), tp.recv_counts()))
        ok_counts = all(counts[s][0][rank] == tp.recv_counts()[s] for s in range(world))
        assert sorted(sum(tp.owned, [])) == list(range(T))
        all_ids = [None] * world
        dist.all_gather_object(all_ids, ([b.raw_ids for b in w.bags], [b.slice_input for b in w.bags]))
        mine = tp.owned[rank]
        exact = True
        for s in range(world):  # the owner pools source s' lookups of its tables
            pooled = _pool([w.tables[t] for t in mine], [rows[t] for t in mine],
                           [all_ids[s][0][t] for t in mine], [all_ids[s][1][t] for t in mine], B, D) \
                if mine else np.zeros((B, 0, D), np.float32)
            if s == rank and mine:
                exact = exact and np.array_equal(pooled, want[:, mine, :])
            off = sum(tp.recv_counts()[:s])
            for j, t in enumerate(mine):
                assert tp.recv_offset(s, j) == off
                off += int(tp.nnz[s, t])
        q.put((rank, err_row, ok_counts, exact))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_shard_plan_on_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err_row, ok_counts, exact in res:
        assert err_row <= 1e-5, (rank, err_row)
        assert ok_counts and exact


def test_local_rows_rule():
    from annc_b200.sharded import ShardPlan
    for rows in (1, 2, 7, 8, 9, 1000):
        for g in (1, 2, 3, 8):
            tot = 0
            for r in range(g):
                p = ShardPlan("row", g, r, [rows], np.zeros((g, 1)))
                assert p.local_rows(0) == len(range(r, rows, g))
                tot += p.local_rows(0)
            assert tot == rows


def test_tables_replicated_whole_stay_out_of_the_exchange():
    from annc_b200.sharded import whole_and_sharded_tables
    rows = [1000, 65536, 65537, 10_000_000, 5]
    assert whole_and_sharded_tables(rows, 0) == ([], [0, 1, 2, 3, 4])          # no replicated rows at all
    assert whole_and_sharded_tables(rows, 65536) == ([0, 1, 4], [2, 3])        # up to and including K rows
    assert whole_and_sharded_tables(rows, 999) == ([4], [0, 1, 2, 3])
    # nothing left to shard: every table stays in the exchange (which then replicates them all)
    assert whole_and_sharded_tables([10, 20], 100) == ([], [0, 1])
    whole, part = whole_and_sharded_tables(rows, 70000)
    assert sorted(whole + part) == list(range(len(rows))) and not set(whole) & set(part)


# ---------------------------------------------------------------- partition-at-source protocol

def _worker_partitioned(rank, world, port, q):
    """The row exchange's protocol on CPU ranks, numpy and the CPU oracle standing in for the
    kernels, gloo collectives for the peer loads and stores: split own lookups by owner into
    record lists (local row, bag), hot rows staying with the source -> every owner reads the
    lists meant for it -> pools them record by record, one part per (source, bag) that has
    records -> parts go to the sample owner -> masked sum in rank order (x 1/len for mean).
    Must match the unsharded oracle within the fp32 pooling tolerance."""
    import torch
    from annc_b200 import synth
    from annc_b200.sharded import ShardPlan, partition_lookups
    from oracle import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, D, rows = 48, 8, [1000, 37, 5000, 3]
        T = len(rows)
        w = synth.embedding_workload(21, rows, D, B, 30, 1.2, threads=1, input_seed=70 + rank)
        plan = ShardPlan("row", world, rank, rows, np.zeros((world, T)))
        hot_k = [40, 0, 200, 3]  # table 3 is replicated whole, table 1 has no hot rows
        hot_rows = [w.bags[t].popular_rows(hot_k[t], rows[t]) for t in range(T)]
        # what this rank holds of table t: its shard, then the replicated hot rows
        held = [np.concatenate([plan.local_shard(w.tables[t]), w.tables[t][hot_rows[t]]]) for t in range(T)]
        errs = []
        for combiner in (0, 1):
            want = np.zeros((B, T, D), np.float32)
            for t, bag in enumerate(w.bags):
                idx = oracle.hash_bucket(bag.raw_ids.view(np.uint64), rows[t])
                o, _ = oracle.sparse_segment_reduce(w.tables[t], idx, bag.slice_input, np.array([0, 0], np.int32),
                                                    np.array([0], np.int32), combiner)
                want[:o.shape[0], t] = o
            # 1. split at the source: mine[t][g] = (local rows, bags) for owner g
            mine = [partition_lookups(b.raw_ids, b.slice_input[:, 0], rows[t], world, source=rank,
                                      hot_rows=hot_rows[t], local_rows_of_source=plan.local_rows(t))
                    for t, b in enumerate(w.bags)]
            lens = np.stack([np.bincount(b.slice_input[:, 0], minlength=B) for b in w.bags])  # [T, B]
            # 2. owners read the lists meant for them (all_gather_object stands in for the peer loads)
            everyone = [None] * world
            dist.all_gather_object(everyone, [[mine[t][g] for t in range(T)] for g in range(world)])
            # 3. this owner pools, for every source s, the records of its list
            parts_out = np.zeros((world, B, T, D), np.float32)   # [source, ...]: goes back to s
            for s in range(world):
                for t in range(T):
                    local, seg = everyone[s][rank][t]
                    if local.size == 0:
                        continue
                    assert int(local.max()) < held[t].shape[0]
                    sl = np.stack([seg, np.zeros_like(seg)], axis=1)
                    o, _ = oracle.sparse_segment_reduce(held[t], local.astype(np.int64), sl, np.array([0, 0], np.int32),
                                                        np.array([0], np.int32), 0)
                    parts_out[s, :o.shape[0], t] = o
            # 4. parts travel to the sample owner (an all_gather stands in for the peer stores:
            #    rank g's part for source s is gathered[g][s])
            gathered = [torch.zeros((world, B, T, D)) for _ in range(world)]
            dist.all_gather(gathered, torch.from_numpy(parts_out))
            recv = [gathered[g][rank] for g in range(world)]
            # 5. masked sum in rank order; the mask comes from this rank's own split
            got = np.zeros((B, T, D), np.float32)
            for g in range(world):
                for t in range(T):
                    have = np.zeros(B, bool)
                    have[mine[t][g][1]] = True
                    got[have, t] = got[have, t] + recv[g].numpy()[have, t]
            if combiner == 1:
                inv = np.where(lens > 0, np.float32(1.0) / np.maximum(lens, 1).astype(np.float32), np.float32(1.0))
                got = got * inv.T[:, :, None].astype(np.float32)
            errs.append(float(np.abs(got - want).max() / np.abs(want).max()))
            # nothing of a whole-replicated table crosses ranks
            assert all(mine[3][g][0].size == 0 for g in range(world) if g != rank)
        q.put((rank, errs))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_row_protocol_on_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + world
    procs = [ctx.Process(target=_worker_partitioned, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in res:
        assert max(errs) <= 1e-5, (rank, errs)

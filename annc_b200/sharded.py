"""Multi-GPU embedding step of the DLRM-style pipeline: one process per GPU.

Partitionings of the tables; the MLPs always run on the rank's own batch slice (no collective
in the MLP):

  row      every table row-sharded with the reference's mod rule
           (owner = bucket % G, local row = bucket / G,
           annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:70-71), optionally
           with a small replicated set of hot rows per table.  The whole step protocol lives in
           the library (annc_row_exchange_*, mirrored by annc_b200/row_exchange.py): lookups are
           split by owner at their source, the owners read their lists through peer-mapped
           pointers, pool them and store each partial sum straight into the memory of the rank
           that owns the sample; flags in peer memory order the ranks (no NCCL call on the
           data path); the owner adds the parts in rank order.
  row_nccl the baseline the fused step is measured against: raw ids and bag offsets are
           all-gathered, every rank pools the lookups it owns, and the partial sums go through
           an NCCL all-to-all.
  table    whole tables per rank (contiguous blocks); the owners fetch the ids and bag offsets
           of their tables through peer-mapped pointers and the bag kernel stores finished
           pooled vectors into the sample owner's memory (TableShardedBags); no add.
  table_nccl  the same partitioning with NCCL: ids travel to the owners by all-to-all,
           finished pooled vectors come back by all-to-all.
  replica  every rank holds every table; no exchange (scaling ceiling when tables fit).

ShardPlan is pure numpy so that the partitioning logic is testable on CPU ranks.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np


class ShardPlan:
    """Sizes and offsets of the exchange.  nnz[s][t] = lookups of rank s in table t."""

    def __init__(self, mode: str, world: int, rank: int, table_rows: List[int], nnz: np.ndarray):
        assert mode in ("row", "row_nccl", "table", "table_nccl", "replica")
        self.mode, self.world, self.rank = mode, world, rank
        self.table_rows = list(table_rows)
        self.T = len(table_rows)
        self.nnz = np.asarray(nnz, np.int64).reshape(world, self.T)
        # table mode: contiguous blocks of tables per owner
        blocks = np.array_split(np.arange(self.T), world)
        self.owned = [list(map(int, b)) for b in blocks]
        self.owner_of = np.zeros(self.T, np.int64)
        for p, b in enumerate(self.owned):
            self.owner_of[b] = p

    # ---- row mode
    def local_rows(self, t: int) -> int:
        """Rows of table t stored on this rank: r with r % world == rank."""
        rows, g, r = self.table_rows[t], self.world, self.rank
        return (rows - r + g - 1) // g if rows > r else 0

    def local_shard(self, table: np.ndarray) -> np.ndarray:
        return np.ascontiguousarray(table[self.rank::self.world])

    def gathered_len(self) -> int:
        """Per-rank length of the padded id buffer that is all-gathered."""
        return int(self.nnz.sum(axis=1).max())

    def gathered_offset(self, s: int, t: int) -> int:
        """Offset of rank s' lookups of table t inside its (table-ordered) flat buffer."""
        return int(self.nnz[s, :t].sum())

    # ---- table mode
    def send_counts(self) -> List[int]:
        """Lookups this rank sends to each owner (its buffer is table-ordered, and tables
        are owned in contiguous blocks, so each destination's part is contiguous)."""
        return [int(self.nnz[self.rank, self.owned[p]].sum()) for p in range(self.world)]

    def recv_counts(self) -> List[int]:
        """Lookups this rank receives from each source for the tables it owns."""
        return [int(self.nnz[s, self.owned[self.rank]].sum()) for s in range(self.world)]

    def recv_offset(self, s: int, j: int) -> int:
        """Offset, inside the receive buffer, of source s' lookups of my j-th owned table."""
        rc = self.recv_counts()
        mine = self.owned[self.rank]
        return int(sum(rc[:s]) + self.nnz[s, mine[:j]].sum())


def whole_and_sharded_tables(table_rows, hot_rows: int):
    """Tables of a row-sharded model that are replicated whole (no more rows than the replicated
    set of `hot_rows` rows per table: they stay out of the exchange) and the tables that are
    sharded.  When nothing would be left to shard, every table stays in the exchange."""
    whole = [t for t, r in enumerate(table_rows) if 0 < int(r) <= int(hot_rows)]
    part = [t for t in range(len(table_rows)) if t not in whole]
    if not part:
        return [], list(range(len(table_rows)))
    return whole, part


def partition_lookups(raw_ids, seg_ids, table_rows: int, shards: int, source: int = 0, hot_rows=None,
                      local_rows_of_source: int = 0):
    """Host statement of the split the row exchange makes for one table of one source rank
    (the GPU tests compare the library with it; the gloo CPU test runs the protocol on it):
    bucket = uint64(id) % table_rows; a bucket in `hot_rows` (ascending) stays with the source
    at local row local_rows_of_source + (index in hot_rows); otherwise owner = bucket % shards
    and local row = bucket // shards.  Returns per owner the records (local row, segment id)
    in lookup order."""
    bucket = (np.asarray(raw_ids).view(np.uint64) % np.uint64(table_rows)).astype(np.int64)
    owner, local = bucket % shards, bucket // shards
    if hot_rows is not None and len(hot_rows):
        hot_rows = np.asarray(hot_rows, np.int64)
        idx = np.searchsorted(hot_rows, bucket)
        idx_c = np.minimum(idx, len(hot_rows) - 1)
        is_hot = hot_rows[idx_c] == bucket
        owner = np.where(is_hot, source, owner)
        local = np.where(is_hot, local_rows_of_source + idx_c, local)
    seg = np.asarray(seg_ids, np.int64)
    return [(local[owner == g].astype(np.int32), seg[owner == g]) for g in range(shards)]


class RowShardedBags:
    """Embedding bags over row-sharded tables, one process per GPU of one node: the torch side
    of annc_row_exchange_* (peer buffers allocated and exchanged here, every step phase in the
    library).  prefetch(i) splits input set i by owner and publishes the lists; run(i, out)
    pools the lists meant for this rank, storing the partial sums into the owners' memory, and
    adds the parts of this rank's batch into `out` (f32, or bf16 with out_bf16) as
    [batch, tables, dim] rows of `out_stride` elements.

    local_tables[t]: f32[local_rows[t] + h, dim], the shard's rows followed by the h replicated
    hot rows; hot: optional per-table (h, hot_rows i64[h] tensor or None for "all rows");
    None = no hot rows."""

    def __init__(self, world: int, rank: int, device, local_tables, local_rows, table_rows, batch: int,
                 dim: int, nnz_all, id_sets, combiner: int = 0, id_kind: int = 2, hot=None,
                 out_slots=None, bags_per_sample: Optional[int] = None):
        """out_slots: table t of the exchange is written to slot out_slots[t] of the output rows
        (the caller pools other tables into the remaining slots itself); bags_per_sample: the
        number of tables of the whole model, for the per-bag figures of exchange_stats()."""
        import torch
        import torch.distributed as dist

        from . import device as dev
        from . import row_exchange as rx
        self.rx, self.dist, self.torch = rx, dist, torch
        self.world, self.rank = world, rank
        T = len(local_tables)
        self.T, self.B, self.D = T, batch, dim
        nnz_all = np.asarray(nnz_all, np.int64).reshape(world, T)
        tabs = []
        self.hot_bytes = 0
        for t in range(T):
            h_count, h_rows = (hot[t] if hot is not None and hot[t] is not None else (0, None))
            self.hot_bytes += h_count * dim * 4
            assert int(local_tables[t].shape[0]) >= int(local_rows[t]) + h_count
            tabs.append(dict(shard=local_tables[t].data_ptr() if int(local_rows[t]) + h_count > 0 else 0,
                             local_rows=int(local_rows[t]), rows=int(table_rows[t]),
                             hot_rows=h_rows.data_ptr() if (h_count and h_rows is not None) else 0,
                             hot_count=h_count))
        self._keep = (list(local_tables), hot)
        cfg, keep = rx.make_config(world, rank, tabs, dim, batch,
                                   max(1, int(nnz_all.sum(axis=1).max())), max(1, int(nnz_all.max())),
                                   combiner=combiner, id_kind=id_kind)
        self.peer = dev.PeerBuffers(rx.peer_bytes(cfg), world, rank)
        self.ex = rx.RowExchange(cfg, keep, self.peer.ptrs)
        if out_slots is not None:
            self.ex.set_output_slots(out_slots)
        self.bags_per_sample = int(bags_per_sample) if bags_per_sample else T
        if world > 1:
            dist.barrier()  # every rank's flags are cleared before anybody's first step
        self.inputs = [rx.StepInputs([x.data_ptr() for x in st["ids"]], [x.data_ptr() for x in st["segs"]],
                                     [int(x.shape[0]) for x in st["ids"]]) for st in id_sets]
        self.ncols = int(id_sets[0]["segs"][0].shape[1])
        self.launches_per_step = 12 + (1 if combiner == 1 else 0)
        self.exchange_bytes = 0  # measured: see exchange_stats()
        self._begun_set = None   # input set whose lists are published for the next run()
        self._ahead_set = None   # input set published one step further ahead

    def prefetch(self, set_index: int) -> None:
        """Splits and publishes input set `set_index` for the next run() unless that has been
        done ahead of time."""
        if self._begun_set is None:
            self.ex.begin(self.inputs[set_index], self.ncols, 0)
            self._begun_set = set_index

    def prefetch_next(self, set_index: int) -> None:
        """One step of lookahead: splits and publishes the input set of the step AFTER the one
        whose run() comes next (whose prefetch has been issued), typically from a second stream,
        so that the split of step i + 1 runs under the pooling of step i."""
        assert self._begun_set is not None and self._ahead_set is None
        self.ex.begin(self.inputs[set_index], self.ncols, 0)
        self._ahead_set = set_index

    def run(self, set_index: int, out_ptr: int, out_stride: int, out_bf16: bool = False) -> None:
        if self._begun_set is not None and self._begun_set != set_index:
            # a step was published for another input set: it has to be completed (the peers
            # have seen it); its result is overwritten below
            self.ex.pool()
            self.ex.finish(out_ptr, out_stride, out_bf16)
            self._begun_set, self._ahead_set = self._ahead_set, None
            return self.run(set_index, out_ptr, out_stride, out_bf16)
        self.prefetch(set_index)
        self.ex.pool()
        self.ex.finish(out_ptr, out_stride, out_bf16)
        self._begun_set, self._ahead_set = self._ahead_set, None

    def run_pool(self, set_index: int) -> None:
        """First half of run(): pooling + exchange of input set `set_index` on the current stream."""
        if self._begun_set is not None and self._begun_set != set_index:
            raise ValueError("a step of another input set is published: complete it with run() first")
        self.prefetch(set_index)
        self.ex.pool()

    def run_finish(self, out_ptr: int, out_stride: int, out_bf16: bool = False) -> None:
        """Second half of run(): second barrier + sum of the parts, on the current stream (which
        may be another stream than run_pool's, ordered after it by the caller)."""
        self.ex.finish(out_ptr, out_stride, out_bf16)
        self._begun_set, self._ahead_set = self._ahead_set, None

    def exchange_stats(self) -> dict:
        """Last step: records pooled per source, parts received per owner, and the bytes that
        crossed NVLink into and out of this rank (records read from peers, parts stored)."""
        recs, parts = self.ex.stats()
        remote_recs = sum(r for q, r in enumerate(recs) if q != self.rank)
        remote_parts = sum(p for q, p in enumerate(parts) if q != self.rank)
        self.exchange_bytes = remote_recs * 8 + remote_parts * self.D * 4
        return dict(records_per_source=recs, parts_per_owner=parts, remote_records=remote_recs,
                    remote_parts_received=remote_parts,
                    remote_parts_per_bag=remote_parts / (self.B * self.bags_per_sample),
                    nvlink_bytes=self.exchange_bytes, hot_bytes=self.hot_bytes)

    def error_bits(self) -> int:
        return self.ex.error_bits()

    def close(self) -> None:
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()  # nobody still reads or writes a peer's buffer
        self.ex.destroy()
        self.peer.close()


class TableShardedBags:
    """Embedding bags over table-wise sharded tables (contiguous blocks of whole tables per
    rank), one process per GPU of one node, with the exchange fused into the bag kernel's
    stores: each owner fetches the raw ids and bag offsets of its tables from every source
    (device-to-device copies through peer-mapped pointers, sizes known on the host), pools
    whole bags — so sums keep the reference's order and are bit-exact — and stores every
    finished pooled vector straight into the source rank's [batch, tables, dim] buffer.
    Nothing is added afterwards and no all-to-all runs; 1/G of the bytes of row sharding
    cross NVLink.  Two one-element all-reduces order the steps.

    local_tables: the tables this rank owns (plan.owned[rank]), full size.  run() leaves this
    rank's pooled vectors, fp32, in `self.out` ([batch, tables, dim], inside the peer buffer)."""

    def __init__(self, world: int, rank: int, device, plan: ShardPlan, local_tables, batch: int, dim: int,
                 id_sets, combiner: int = 0, id_kind: int = 2):
        import torch
        import torch.distributed as dist

        from . import device as dev
        self.dist, self.dev, self.torch = dist, dev, torch
        self.world, self.rank, self.plan = world, rank, plan
        T, B, D = plan.T, batch, dim
        self.T, self.B, self.D = T, B, D
        nnz = plan.nnz                      # [world, T]
        mine = plan.owned[rank]
        self.sets = [dict(prepass=dev.BagPrepass(st["segs"], B), ids_all=st["ids_all"]) for st in id_sets]
        wsb = self.sets[0]["prepass"].ws_bytes
        up256 = lambda n: (n + 255) // 256 * 256
        Lmax = int(nnz.sum(axis=1).max())
        out_bytes = B * T * D * 4
        off_ids = 2 * out_bytes                 # two output buffers, then this rank's ids, then its offsets
        off_off = off_ids + up256(max(1, Lmax) * 8)
        self.peer = dev.PeerBuffers(off_off + up256(wsb), world, rank)
        self.out_bytes, self._off_ids, self._off_off = out_bytes, off_ids, off_off
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.my_nnz_total = int(nnz[rank].sum())
        # what this rank fetches: for every source s, the ids and offsets of the owned tables
        To = len(mine)
        counts = [int(nnz[s, mine].sum()) for s in range(world)]
        self.ids_in = torch.zeros(max(1, sum(counts)), dtype=torch.int64, device=device)
        self.off_in = torch.zeros(max(1, world * To * (B + 1)), dtype=torch.int32, device=device)
        self.copies = []
        pos = 0
        for s in range(world):
            if To == 0:
                break
            first = mine[0]
            src_ids = self.peer.ptrs[s] + off_ids + int(nnz[s, :first].sum()) * 8
            self.copies.append((self.ids_in.data_ptr() + pos * 8, src_ids, counts[s] * 8))
            src_off = self.peer.ptrs[s] + off_off + 512 + first * (B + 1) * 4
            self.copies.append((self.off_in.data_ptr() + s * To * (B + 1) * 4, src_off, To * (B + 1) * 4))
            pos += counts[s]
        self.launches = []
        for buf in range(2):
            entries = []
            pos = 0
            for s in range(world):
                for j, t in enumerate(mine):
                    entries.append((local_tables[j].data_ptr(), plan.table_rows[t], plan.table_rows[t],
                                    self.ids_in.data_ptr() + pos * 8, None, int(nnz[s, t]),
                                    self.peer.ptrs[s] + buf * out_bytes + t * D * 4,
                                    self.off_in.data_ptr() + ((s * To + j) * (B + 1)) * 4))
                    pos += int(nnz[s, t])
            self.launches.append(dev.BagLaunch(entries, D, B, 2, T * D, device, id_kind=id_kind,
                                               combiner=combiner) if entries else None)
        self.step = 0
        self.out_ptr = self.peer.local
        self.launches_per_step = 3 * ((world * max(To, 1) + 119) // 120) + 2 * world + 4
        self.exchange_bytes = (sum(counts) - counts[rank]) * 8 + (world - 1) * To * B * D * 4
        self._work = None

    def prefetch(self, set_index: int) -> None:
        st = self.sets[set_index]
        # this rank's ids and bag offsets into the part of its buffer the owners read
        self.dev.peer_copy(self.peer.local + self._off_ids, st["ids_all"].data_ptr(), self.my_nnz_total * 8)
        ws = self.peer.local + self._off_off
        st["prepass"].run_ptr(ws)
        self._work = self.dist.all_reduce(self.flag, async_op=True)

    def run(self, set_index: int) -> int:
        """Returns the device address of this step's fp32 [batch, tables, dim] pooled vectors."""
        if self._work is None:
            self.prefetch(set_index)
        self._work.wait()
        self._work = None
        buf = self.step % 2
        self.step += 1
        for dst, src, nbytes in self.copies:
            self.dev.peer_copy(dst, src, nbytes)
        if self.launches[buf] is not None:
            self.launches[buf].run()     # pooled vectors land in their sources' memory
        self.dist.all_reduce(self.flag)  # every owner's bag kernel has finished
        return self.peer.local + buf * self.out_bytes

    def error_bits(self) -> int:
        bits = 0
        for l in self.launches:
            if l is not None:
                bits |= l.error_bits()
        return bits

    def close(self) -> None:
        self.peer.close()


class ShardedDlrmPipeline:
    """Built lazily to keep torch out of ShardPlan's import path."""

    def __new__(cls, *args, **kwargs):
        return _make_pipeline(*args, **kwargs)


def _make_pipeline(model, device, mode: str, math=None, keep_host_inputs: bool = False, hot_rows: int = 0):
    import torch
    import torch.distributed as dist

    from . import device as dev
    from ._lib import MATH_AUTO, lib
    from .dlrm import DlrmPipeline

    world, rank = dist.get_world_size(), dist.get_rank()

    class _Pipe(DlrmPipeline):
        def _setup_embedding(self, m) -> None:
            emb = m.emb
            T, B, D = self.T, self.batch, self.dim
            nnz_all = [None] * world
            dist.all_gather_object(nnz_all, [int(x) for x in self.nnz])
            self.shard = plan = ShardPlan(mode, world, rank, [t.shape[0] for t in emb.tables],
                                          np.array(nnz_all))
            f32 = dict(dtype=torch.float32, device=self.device)
            i64 = dict(dtype=torch.int64, device=self.device)
            if mode == "replica":
                DlrmPipeline._setup_embedding(self, m)
                self.exchange_bytes = 0
                return
            if mode == "row":
                self._setup_row_partitioned(m, plan)
                return
            if mode == "row_nccl":
                # Only the raw ids (8 bytes per lookup) and the bag offsets of each rank's
                # batch travel: every rank runs the prepass on its own index matrices and
                # the offsets (4 bytes per bag) are gathered with the ids.
                self.tables = [self._up(plan.local_shard(t)) for t in emb.tables]
                L = plan.gathered_len()
                self.ids_pad = torch.zeros(L, **i64)
                self.ids_g = torch.zeros((world, L), **i64)
                for st in self.sets:
                    st["prepass"] = dev.BagPrepass(st["segs"], B)
                wsb = self.sets[0]["prepass"].ws_bytes
                self.off_ws = torch.zeros(wsb, dtype=torch.uint8, device=self.device)
                self.off_g = torch.zeros((world, wsb), dtype=torch.uint8, device=self.device)
                part_bytes = B * T * D * 4
                self.partial = torch.empty((world, B, T, D), **f32)
                self.recv = torch.empty((world, B, T, D), **f32)
                entries = []
                for s in range(world):
                    for t in range(T):
                        off = plan.gathered_offset(s, t)
                        entries.append((self.tables[t].data_ptr(), plan.local_rows(t),
                                        plan.table_rows[t],
                                        self.ids_g.data_ptr() + (s * L + off) * 8, None,
                                        int(plan.nnz[s, t]), self.partial.data_ptr() + s * part_bytes + t * D * 4,
                                        self.off_g.data_ptr() + s * wsb + 512 + t * (B + 1) * 4))
                self.launch = dev.BagLaunch(entries, D, B, 2, T * D, self.device,
                                            shard_count=world, shard_rank=rank)
                self.embed_launches = 2 * ((len(entries) + 119) // 120) + 2
                self.exchange_bytes = (world - 1) * (B * T * D * 4 + L * 8 + wsb)
                self._works = None
                return
            if mode == "table":
                mine = plan.owned[rank]
                self.tables = [self._up(emb.tables[t]) for t in mine]
                self.tbags = TableShardedBags(
                    world, rank, self.device, plan, self.tables, B, D,
                    [dict(ids_all=st["ids_all"], segs=st["segs"]) for st in self.sets], combiner=0)
                self.peer = self.tbags.peer
                self.embed_launches = self.tbags.launches_per_step + 1
                self.exchange_bytes = self.tbags.exchange_bytes
                return
            # table_nccl mode
            mine = plan.owned[rank]
            self.tables = [self._up(emb.tables[t]) for t in mine]
            sc, rc = plan.send_counts(), plan.recv_counts()
            self.sc, self.rc = sc, rc
            self.ids_r = torch.zeros(max(1, sum(rc)), **i64)
            To = len(mine)
            # bag offsets travel instead of the index matrices: 4 bytes per bag, not 16 per lookup
            for st in self.sets:
                st["prepass"] = dev.BagPrepass(st["segs"], B)
            wsb = self.sets[0]["prepass"].ws_bytes
            self.off_ws = torch.zeros(wsb, dtype=torch.uint8, device=self.device)
            self.off_send = self.off_ws[512:512 + T * (B + 1) * 4].view(torch.int32)
            self.off_sc = [len(plan.owned[p]) * (B + 1) for p in range(world)]
            self.off_r = torch.zeros(max(1, world * To * (B + 1)), dtype=torch.int32, device=self.device)
            self.pooled = torch.empty((world, B, max(To, 1), D), **f32)
            counts_back = [len(plan.owned[p]) * B * D for p in range(world)]
            self.back = torch.empty(sum(counts_back), **f32)
            self.back_counts = counts_back
            entries = []
            for s in range(world):
                for j, t in enumerate(mine):
                    off = plan.recv_offset(s, j)
                    entries.append((self.tables[j].data_ptr(), plan.table_rows[t], plan.table_rows[t],
                                    self.ids_r.data_ptr() + off * 8, None, int(plan.nnz[s, t]),
                                    self.pooled.data_ptr() + ((s * B) * To + j) * D * 4,
                                    self.off_r.data_ptr() + ((s * To + j) * (B + 1)) * 4))
            self.launch = dev.BagLaunch(entries, D, B, 2, max(To, 1) * D, self.device) if entries else None
            self.embed_launches = 3 * ((len(entries) + 119) // 120) + world
            self.exchange_bytes = (sum(sc) - sc[rank]) * 8 + (T - To) * (B + 1) * 4 + (T - To) * B * D * 4

        def _setup_row_partitioned(self, m, plan) -> None:
            emb = m.emb
            # Per table: this rank's shard, then the replicated hot set behind it: the rows of
            # the table's most popular ids (its own popularity map, identical on every rank).
            # A table with no more rows than the replicated set is replicated whole: it stays
            # out of the exchange altogether (no split, no parts, no sum) and is pooled by the
            # one-GPU kernel straight into its slots of z.  The exchange takes the other tables.
            whole, part = whole_and_sharded_tables([t.shape[0] for t in emb.tables], hot_rows)
            self.whole_tables, self.part_tables = whole, part
            self.tables, hot = [], []
            for t in part:
                tab, bag = emb.tables[t], emb.bags[t]
                rows_t = tab.shape[0]
                hr = bag.popular_rows(hot_rows, rows_t) if hot_rows > 0 else np.zeros(0, np.int64)
                self.tables.append(self._up(np.concatenate([plan.local_shard(tab), tab[hr]])))
                hot.append((int(hr.shape[0]), self._up(hr) if 0 < hr.shape[0] < rows_t else None))
            self.rowbags = RowShardedBags(
                world, rank, self.device, self.tables, [plan.local_rows(t) for t in part],
                [plan.table_rows[t] for t in part], self.batch, self.dim, plan.nnz[:, part],
                [dict(ids=[st["ids"][t] for t in part], segs=[st["segs"][t] for t in part])
                 for st in self.sets], combiner=0, hot=hot,
                out_slots=part if whole else None, bags_per_sample=self.T)
            self.whole_bytes = 0
            self.whole_on_side = 0
            if whole:
                self.tables_whole = [self._up(emb.tables[t]) for t in whole]
                self.whole_bytes = int(sum(x.numel() * 4 for x in self.tables_whole))
                for st in self.sets:
                    st["whole_plans"] = [dev.BagPlan(self.tables_whole, [st["ids"][t] for t in whole],
                                                     [st["segs"][t] for t in whole], b["z"], 1, self.batch,
                                                     id_kind=2, col=0, combiner=0, out_slots=whole)
                                         for b in self._bufs]
            self.peer = self.rowbags.peer
            self.embed_launches = self.rowbags.launches_per_step + (3 if whole else 0)
            self.exchange_bytes = 0
            self.split_finish = True  # forward_pipelined may run the sum of the parts on the dense stream

        def embed(self) -> None:
            plan = self.shard
            T, B, D, F = self.T, self.batch, self.dim, self.F
            if mode == "replica":
                return DlrmPipeline.embed(self)
            if mode == "row":
                self._pool_whole_tables()
                self.rowbags.run(self.cur, self.z.data_ptr() + D * 4, F * D)
                return
            if mode == "row_nccl":
                if self._works is None:
                    self.embed_prefetch()
                for w in self._works:
                    w.wait()
                self._works = None
                self.launch.run()
                dist.all_to_all_single(self.recv, self.partial)
                dev.sum_partials(self.recv, world, B * T * D, B, T * D, T * D,
                                 self.z.data_ptr() + D * 4, F * D)
                return
            if mode == "table":
                pooled = self.tbags.run(self.cur)  # fp32 [B, T, D] written by the owners
                dev.copy_rows(self.z.data_ptr() + D * 4, F * D, pooled, T * D, T * D, B)
                return
            # table_nccl mode: ids to the owners, pooled vectors back
            To = len(plan.owned[rank])
            self.sets[self.cur]["prepass"].run(self.off_ws)
            dist.all_to_all_single(self.ids_r[:sum(self.rc)], self.ids_all, self.rc, self.sc)
            dist.all_to_all_single(self.off_r[:world * To * (B + 1)], self.off_send,
                                   [To * (B + 1)] * world, self.off_sc)
            if self.launch is not None:
                self.launch.run()
            send = self.pooled.view(-1)[:world * B * To * D]
            dist.all_to_all_single(self.back, send, self.back_counts, [B * To * D] * world)
            off = 0
            for p in range(world):
                tp = len(plan.owned[p])
                if tp:
                    first = plan.owned[p][0]
                    dev.copy_rows(self.z.data_ptr() + (1 + first) * D * 4, F * D,
                                  self.back.data_ptr() + off * 4, tp * D, tp * D, B)
                off += self.back_counts[p]

        def _pool_whole_tables(self) -> None:
            """The tables replicated whole, by the one-GPU kernel, before the exchange's pooling
            (it runs while the peers' lists are still on their way)."""
            plans = self.sets[self.cur].get("whole_plans")
            if plans:
                plans[self._buf].run()

        def embed_pool(self) -> None:
            if mode == "row":
                if not self.whole_on_side:
                    self._pool_whole_tables()
                self.rowbags.run_pool(self.cur)
            else:
                self.embed()

        def embed_side(self) -> None:
            """With whole_on_side = k > 0: the tables replicated whole are pooled on the side
            stream with k blocks per SM, beside the exchange's pooling kernel on the main stream
            (which is bound by its NVLink stores from four GPUs on and should be given k blocks
            per SM fewer: RowExchange.set_pool_ctas_per_sm(-k))."""
            if mode == "row" and self.whole_on_side:
                lib.annc_embed_bag_set_stream_ctas_per_sm(int(self.whole_on_side))
                try:
                    self._pool_whole_tables()
                finally:
                    lib.annc_embed_bag_set_stream_ctas_per_sm(0)

        def embed_finish(self) -> None:
            if mode == "row":
                self.rowbags.run_finish(self.z.data_ptr() + self.dim * 4, self.F * self.dim)

        def embed_prefetch(self) -> None:
            """Starts the exchange (row: split + publish; table: ids into peer-visible memory;
            row_nccl: the gathers of ids and bag offsets); the bottom MLP runs beside it."""
            if mode == "row":
                self.rowbags.prefetch(self.cur)
                return
            if mode == "table":
                self.tbags.prefetch(self.cur)
                return
            if mode != "row_nccl":
                return
            n = self.nnz_total
            self.ids_pad[:n].copy_(self.ids_all)
            self.sets[self.cur]["prepass"].run(self.off_ws)
            self._works = [dist.all_gather_into_tensor(self.ids_g, self.ids_pad, async_op=True),
                           dist.all_gather_into_tensor(self.off_g, self.off_ws, async_op=True)]

        def embed_prefetch_next(self) -> None:
            """Lookahead for back-to-back steps on the same input set (row mode): the split of
            the next step, issued on the stream the bottom MLP runs on."""
            if mode == "row":
                self.rowbags.prefetch_next(self.cur)

        def embed_error_bits(self) -> int:
            if mode == "replica":
                return DlrmPipeline.embed_error_bits(self)
            if mode == "row":
                bits = self.rowbags.error_bits()
                for st in self.sets:
                    for p in st.get("whole_plans", []):
                        bits |= p.error_bits()
                return bits
            if mode == "table":
                return self.tbags.error_bits()
            return self.launch.error_bits() if self.launch is not None else 0

        def close_exchange(self) -> None:
            """Releases the peer mappings (collective: every rank calls it)."""
            torch.cuda.synchronize()
            if mode == "row":
                self.rowbags.close()
            elif mode == "table":
                self.tbags.close()

    return _Pipe(model, device, math=MATH_AUTO if math is None else math,
                 keep_host_inputs=keep_host_inputs)

"""Large row-sharded recsys step (one process per GPU): `tables` hashed embedding tables,
row-sharded with the mod rule over the ranks, mean pooling, concat -> MLP in BF16 with bias +
ReLU epilogues and a final sigmoid.  The tables are filled on the device, shard by shard, from
a counter-based hash (annc_synth_fill_rows_dev), so no host copy of the 655 GB exists; the CPU
oracle regenerates the rows it needs (synth.hashed_table_rows).

Step (row mode): the library's row exchange (lookups split by owner at their source, owners pool
their lists and store partial sums into the sample owner's memory, masked rank-order sum * 1/len
written as bf16 straight into the MLP input) -> tcgen05 BF16 GEMMs (bf16 activations between
layers) -> fp32 last layer.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import device as dev
from ._lib import (ACT_RELU, ACT_SIGMOID, IO_A_BF16, IO_B_BF16, IO_C_BF16, MATH_BF16, MATH_FP32, check,
                   lib)
from .sharded import RowShardedBags, ShardPlan, TableShardedBags
from .synth import RecsysModel


class RecsysPipeline:
    def __init__(self, model: RecsysModel, device: torch.device, keep_host_inputs: bool = False,
                 shard: str = "row", hot_rows: int = 0):
        """shard: "row" (mod rule, partial sums stored into the sample owner's memory) or "table"
        (whole tables per rank, finished pooled vectors stored into the sample owner's memory).
        hot_rows > 0 (row mode): the rows of each table's `hot_rows` most popular ids are
        replicated on every rank (generated from the same hash) and pooled where the sample is."""
        assert shard in ("row", "table")
        world, rank = dist.get_world_size(), dist.get_rank()
        self.world, self.rank, self.device, self.shard = world, rank, device, shard
        self.model = model
        T, R, D, B = model.tables, model.rows, model.dim, model.batch
        self.T, self.D, self.batch = T, D, B
        s = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        if shard == "row":
            self.local_rows = len(range(rank, R, world))
            # Replicated hot rows (generated from the same hash) sit behind each shard's rows.
            hot_lists = [model.bags[t].popular_rows(hot_rows, R) if hot_rows > 0 else np.zeros(0, np.int64)
                         for t in range(T)]
            hmax = max(int(h.shape[0]) for h in hot_lists)
            # one allocation for all local shards: [T, local_rows + hot rows, D]
            self.table_mem = torch.empty((T, max(self.local_rows + hmax, 1), D), dtype=torch.float32, device=device)
            self._hot = []
            for t in range(T):
                check(lib.annc_synth_fill_rows_dev(C.c_void_p(self.table_mem[t].data_ptr()),
                                                   C.c_int64(self.local_rows), C.c_int64(D),
                                                   C.c_uint64(model.seed), C.c_int64(t), C.c_int64(rank),
                                                   C.c_int64(world), s))
                h = int(hot_lists[t].shape[0])
                hr = up(hot_lists[t]) if h else None
                if h:
                    check(lib.annc_synth_fill_row_list_dev(
                        C.c_void_p(self.table_mem[t][self.local_rows:].data_ptr()), C.c_void_p(hr.data_ptr()),
                        C.c_int64(h), C.c_int64(D), C.c_uint64(model.seed), C.c_int64(t), s))
                self._hot.append((h, hr if 0 < h < R else None))
        else:
            self.owned = [int(t) for t in np.array_split(np.arange(T), world)[rank]]
            self.local_rows = R
            self.table_mem = torch.empty((max(len(self.owned), 1), R, D), dtype=torch.float32, device=device)
            for j, t in enumerate(self.owned):
                check(lib.annc_synth_fill_rows_dev(C.c_void_p(self.table_mem[j].data_ptr()), C.c_int64(R),
                                                   C.c_int64(D), C.c_uint64(model.seed), C.c_int64(t),
                                                   C.c_int64(0), C.c_int64(1), s))
        nnz = [int(b.raw_ids.shape[0]) for b in model.bags]
        self.nnz, self.nnz_total = nnz, int(sum(nnz))
        ids_host = np.concatenate([b.raw_ids for b in model.bags])
        seg_host = np.concatenate([b.slice_input for b in model.bags])
        offs = np.concatenate([[0], np.cumsum(nnz)])
        self.sets = []
        for _ in range(2 if keep_host_inputs else 1):
            st = {"ids_all": up(ids_host), "seg_all": up(seg_host)}
            st["ids"] = [st["ids_all"][offs[t]:offs[t + 1]] for t in range(T)]
            st["segs"] = [st["seg_all"][offs[t]:offs[t + 1]] for t in range(T)]
            self.sets.append(st)
        if keep_host_inputs:
            self.h_ids = torch.from_numpy(ids_host).pin_memory()
            self.h_seg = torch.from_numpy(seg_host).pin_memory()
            self.h_out = torch.empty((B, 1), dtype=torch.float32).pin_memory()
            self.copy_stream = torch.cuda.Stream(device=device)
            self.ready = [torch.cuda.Event() for _ in self.sets]
            self.done = [torch.cuda.Event() for _ in self.sets]
            self._prefetched = [False, False]
        self._step = 0
        nnz_all = [None] * world
        dist.all_gather_object(nnz_all, nnz)
        if shard == "row":
            hot = self._hot
            self.bags = RowShardedBags(world, rank, device, [self.table_mem[t] for t in range(T)],
                                       [self.local_rows] * T, [R] * T, B, D, np.array(nnz_all),
                                       [dict(ids=st["ids"], segs=st["segs"]) for st in self.sets], combiner=1,
                                       hot=hot)
        else:
            plan = ShardPlan("table", world, rank, [R] * T, np.array(nnz_all))
            assert plan.owned[rank] == self.owned
            self.bags = TableShardedBags(world, rank, device, plan,
                                         [self.table_mem[j] for j in range(len(self.owned))], B, D,
                                         [dict(ids_all=st["ids_all"], segs=st["segs"]) for st in self.sets],
                                         combiner=1)
        # MLP: bf16 weights [N,K] converted once; the last layer (n = 1) stays fp32
        self.layers = []
        for i, (w, b) in enumerate(model.mlp):
            wd = up(w)
            last = i == len(model.mlp) - 1
            self.layers.append((wd if last else dev.bf16_weight(wd), up(b), w.shape[0], w.shape[1]))
        self.x0 = torch.empty((B, T * D), dtype=torch.bfloat16, device=device)
        self.acts = []
        for i, (_, _, k, n) in enumerate(self.layers):
            last2 = i >= len(self.layers) - 2  # the input of the fp32 last layer, and its output, are fp32
            self.acts.append(torch.empty((B, n), dtype=torch.float32 if last2 else torch.bfloat16, device=device))
        self.out = self.acts[-1]
        self.kernel_names = []
        self.launches_per_step = self.bags.launches_per_step + len(self.layers)

    def forward(self, set_index: int = 0) -> torch.Tensor:
        B = self.batch
        self.bags.prefetch(set_index)
        if self.shard == "row":
            self.bags.run(set_index, self.x0.data_ptr(), self.T * self.D, out_bf16=True)
        else:  # the owners have stored finished fp32 means; one pass makes the MLP's bf16 input
            pooled = self.bags.run(set_index)
            dev.cast_bf16_ptr(pooled, self.x0.data_ptr(), B * self.T * self.D)
        x = self.x0
        names = []
        n_layers = len(self.layers)
        for i, (w, b, k, n) in enumerate(self.layers):
            y = self.acts[i]
            if i == n_layers - 1:
                names.append(dev.gemm(x, w, y, m=B, n=n, k=k, bias=b, activation=ACT_SIGMOID, math=MATH_FP32))
            else:
                flags = IO_A_BF16 | IO_B_BF16 | (IO_C_BF16 if y.dtype == torch.bfloat16 else 0)
                names.append(dev.gemm(x, w, y, m=B, n=n, k=k, trans_b=True, bias=b, activation=ACT_RELU,
                                      math=MATH_BF16, io_flags=flags))
            x = y
        self.kernel_names = names
        return self.out

    def _issue_copy(self, i: int) -> None:
        st = self.sets[i]
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.done[i])
            st["ids_all"].copy_(self.h_ids, non_blocking=True)
            st["seg_all"].copy_(self.h_seg, non_blocking=True)
            self.ready[i].record(self.copy_stream)
        self._prefetched[i] = True

    def forward_e2e(self) -> torch.Tensor:
        """Host ids and index matrices in, host predictions out; the next step's copies are
        issued first on a second stream and overlap this step's kernels."""
        cur = self._step % 2
        if not self._prefetched[cur]:
            self._issue_copy(cur)
        self._issue_copy(1 - cur)
        torch.cuda.current_stream().wait_event(self.ready[cur])
        out = self.forward(cur)
        self.h_out.copy_(out, non_blocking=True)
        self.done[cur].record()
        self._prefetched[cur] = False
        self._step += 1
        return self.h_out

    @property
    def h2d_bytes(self) -> int:
        return self.sets[0]["ids_all"].numel() * 8 + self.sets[0]["seg_all"].numel() * 8

    @property
    def d2h_bytes(self) -> int:
        return self.out.numel() * 4

    def algorithmic_embed_bytes(self) -> int:
        """Row read + raw id + segment id per lookup, one pooled row per bag (this rank's batch)."""
        return self.nnz_total * (4 * self.D + 16) + self.T * self.batch * 4 * self.D

    def embed_error_bits(self) -> int:
        return self.bags.error_bits()

    def close(self) -> None:
        torch.cuda.synchronize()
        self.bags.close()

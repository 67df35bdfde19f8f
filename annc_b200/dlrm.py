"""DLRM-style inference step assembled from the library's operator entry points,
the way an ANNC-rewritten graph would call them:

  bottom MLP   3 x matmul + bias + ReLU            (annc_gemm_run, bias-row epilogue)
  embeddings   hash-bucket + gather + segment sum  (annc_embed_bags_dev, all tables, one launch)
  interaction  batch_matmul Z Z^T, lower triangle  (annc_dot_interaction_dev)
  top MLP      2 x matmul + bias + ReLU, 1 x matmul + bias + sigmoid

torch holds the device buffers and the stream; all kernels are from libannc_b200.so.
Buffers are allocated once in __init__, a step allocates nothing.

forward() runs one step and leaves its result ordered on the current stream.
forward_pipelined() is the throughput form for back-to-back batches: the embedding part of a
step (gather-latency bound, tensor cores idle) runs on the current stream while the dense part
of the previous step (interaction + top MLP, tensor-core work) runs on a second stream; two
sets of intermediate buffers alternate.  Where the embedding part has a separate closing pass
(row-sharded tables: second barrier + sum of the parts), forward_pipelined(split=True) moves
that pass to the dense stream as well, so the current stream carries nothing but the pooling
kernels, back to back (they are bound by their NVLink stores on four and more GPUs).  Results
are the same; sync_pipeline() orders the current stream after the last step.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np
import torch

from . import device as dev
from ._lib import ACT_RELU, ACT_SIGMOID, MATH_AUTO, lib
from .synth import DlrmModel


class DlrmPipeline:
    def __init__(self, model: DlrmModel, device: torch.device, math: int = MATH_AUTO,
                 keep_host_inputs: bool = False):
        self.device = device
        self.math = math
        emb = model.emb
        self.batch = B = emb.batch
        self.dim = D = emb.dim
        self.T = T = len(emb.tables)
        self.F = F = T + 1
        tri = F * (F - 1) // 2
        self.inter = D + tri
        self.inter_pad = (self.inter + 3) // 4 * 4  # 16-byte rows for the tensor-core loader

        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(device)
        self._up = up
        self.bottom = [(up(w), up(b)) for w, b in model.bottom]
        top = []
        for i, (w, b) in enumerate(model.top):
            if i == 0 and w.shape[0] != self.inter_pad:
                w = np.concatenate([w, np.zeros((self.inter_pad - w.shape[0], w.shape[1]), np.float32)])
            top.append((up(w), up(b)))
        self.top = top

        # step inputs: one flat buffer per kind so that an end-to-end step is three copies.
        # With host inputs kept there are two device input sets, so the copies of the next
        # step overlap the kernels of the current one.
        nnz = [b.raw_ids.shape[0] for b in emb.bags]
        self.nnz = nnz
        self.nnz_total = int(sum(nnz))
        ids_host = np.concatenate([b.raw_ids for b in emb.bags])
        seg_host = np.concatenate([b.slice_input for b in emb.bags])
        offs = np.concatenate([[0], np.cumsum(nnz)])
        self.sets = []
        for _ in range(2 if keep_host_inputs else 1):
            st = {"ids_all": up(ids_host), "seg_all": up(seg_host), "dense": up(model.dense)}
            st["ids"] = [st["ids_all"][offs[t]:offs[t + 1]] for t in range(T)]
            st["segs"] = [st["seg_all"][offs[t]:offs[t + 1]] for t in range(T)]
            self.sets.append(st)
        self._use(0)
        self._step = 0
        if keep_host_inputs:
            self.h_ids = torch.from_numpy(ids_host).pin_memory()
            self.h_seg = torch.from_numpy(seg_host).pin_memory()
            self.h_dense = torch.from_numpy(np.ascontiguousarray(model.dense)).pin_memory()
            self.h_out = torch.empty((B, 1), dtype=torch.float32).pin_memory()
            self.copy_stream = torch.cuda.Stream(device=device)
            self.ready = [torch.cuda.Event() for _ in self.sets]
            self.done = [torch.cuda.Event() for _ in self.sets]
            self._prefetched = [False, False]

        f32 = dict(dtype=torch.float32, device=device)
        self.acts_b = [torch.empty((B, w.shape[1]), **f32) for w, _ in self.bottom[:-1]]
        # two sets of step buffers: forward() uses set 0, forward_pipelined() alternates
        self._bufs = [dict(z=torch.empty((B, F, D), **f32),
                           inter=torch.empty((B, self.inter_pad), **f32),
                           acts_t=[torch.empty((B, w.shape[1]), **f32) for w, _ in self.top])
                      for _ in range(2)]
        self._buf = 0
        self._select(0)
        self.dense_stream = torch.cuda.Stream(device=device)
        self._dense_done = [torch.cuda.Event() for _ in range(2)]
        self._sum_done = [torch.cuda.Event() for _ in range(2)]
        self._bottom_done = [torch.cuda.Event() for _ in range(2)]
        self._begin_done = torch.cuda.Event()
        self._pooled = torch.cuda.Event()
        self.split_finish = False  # embed() = embed_pool() + embed_finish(), the latter movable
        self._pstep = 0
        self.kernel_names: List[str] = []
        self.launches_per_step = 0
        # The bottom MLP does not depend on the embeddings: it runs on a second stream beside the
        # prepass and the bag kernel (which is bound by gather latency, not by bandwidth) and
        # joins before the interaction.
        self.side_stream = torch.cuda.Stream(device=device)
        self.embed_launches = 3  # prepass + bag + atomic route
        self._setup_embedding(model)

    def _select(self, buf: int) -> None:
        """Makes buffer set `buf` the one the next step writes (z, interaction, top activations)."""
        b = self._bufs[buf]
        self._buf = buf
        self.z, self.inter_buf, self.acts_t = b["z"], b["inter"], b["acts_t"]
        self.out = self.acts_t[-1]
        if getattr(self, "cur", None) is not None and "plans" in self.sets[self.cur]:
            self.plan = self.sets[self.cur]["plans"][buf]

    def _use(self, i: int) -> None:
        """Makes input set i the one the next forward() reads."""
        st = self.sets[i]
        self.cur = i
        self.ids_all, self.seg_all, self.dense = st["ids_all"], st["seg_all"], st["dense"]
        self.ids, self.segs = st["ids"], st["segs"]
        if "plans" in st:
            self.plan = st["plans"][self._buf]

    def _setup_embedding(self, model: DlrmModel) -> None:
        """Single GPU: every table resident, one grouped bag launch writes slots 1.. of z."""
        self.tables = [self._up(t) for t in model.emb.tables]
        for st in self.sets:
            st["plans"] = [dev.BagPlan(self.tables, st["ids"], st["segs"], b["z"], 1, self.batch,
                                       id_kind=2, col=0, combiner=0) for b in self._bufs]
        self._use(self.cur)

    def embed_prefetch(self) -> None:
        """Hook called before the bottom MLP (multi-GPU variants start their exchange here)."""

    def embed_prefetch_next(self) -> None:
        """Hook of the pipelined form, called on the second stream after the bottom MLP: work of
        the NEXT step that may run under this step's pooling (row sharding: its split)."""

    def embed(self) -> None:
        self.plan.run()

    def embed_pool(self) -> None:
        """embed() without its closing pass (pipelines with split_finish)."""
        self.embed()

    def embed_side(self) -> None:
        """Part of the embedding work that forward_pipelined(split=True) may run on the side
        stream, beside embed_pool() on the current stream (nothing by default)."""

    def embed_finish(self) -> None:
        """The closing pass of embed(): completes z.  May run on another stream than embed_pool."""

    def embed_error_bits(self) -> int:
        bits = 0
        for st in self.sets:
            for p in st.get("plans", []):
                bits |= p.error_bits()
        return bits

    # ------------------------------------------------------------------ one step
    def _sparse_part(self, names, lookahead: bool = False) -> None:
        """Bottom MLP (second stream) beside the embedding pooling; z is complete afterwards."""
        B, F, D = self.batch, self.F, self.dim
        x = self.dense
        nb = len(self.bottom)
        main = torch.cuda.current_stream()
        self.embed_prefetch()
        self.side_stream.wait_stream(main)  # this step's inputs, and the previous readers of z
        with torch.cuda.stream(self.side_stream):
            for i, (w, b) in enumerate(self.bottom):
                last = i == nb - 1
                y = self.z if last else self.acts_b[i]
                names.append(dev.gemm(x, w, y, m=B, n=w.shape[1], k=w.shape[0], bias=b,
                                      activation=ACT_RELU, ldc=(F * D if last else None),
                                      math=self.math))
                x = y
            if lookahead:
                # after a step issued with split=True the previous sum ran on the dense stream
                self.side_stream.wait_event(self._sum_done[1 - self._buf])
                self.embed_prefetch_next()
        self.embed()
        main.wait_stream(self.side_stream)

    def _dense_part(self, names) -> None:
        """Interaction + top MLP on the current stream."""
        B = self.batch
        dev.dot_interaction(self.z, self.inter_buf, self.math)
        x = self.inter_buf
        nt = len(self.top)
        for i, (w, b) in enumerate(self.top):
            y = self.acts_t[i]
            act = ACT_SIGMOID if i == nt - 1 else ACT_RELU
            names.append(dev.gemm(x, w, y, m=B, n=w.shape[1], k=w.shape[0], bias=b, activation=act,
                                  math=self.math))
            x = y
        self.kernel_names = names
        # embedding launches + interaction + one kernel per MLP layer
        self.launches_per_step = self.embed_launches + 1 + len(names)

    def forward(self) -> torch.Tensor:
        self.sync_pipeline()
        self._select(0)
        names = []
        self._sparse_part(names)
        self._dense_part(names)
        return self.out

    def _forward_split(self) -> torch.Tensor:
        """forward_pipelined with the closing pass of the embedding part on the dense stream.
        Stream plan of step i (buffers i % 2):
          current  pooling(i)                                   [needs split(i), issued in step i-1]
          side     bottom MLP(i), then split(i+1)               [split(i+1) after sum(i-1): same buffers]
          dense    sum(i), interaction(i), top MLP(i)           [after pooling(i) and bottom MLP(i)]"""
        buf = self._pstep % 2
        self._pstep += 1
        self._select(buf)
        main = torch.cuda.current_stream()
        main.wait_event(self._dense_done[buf])  # the step before last has finished with this set
        names = []
        B, F, D = self.batch, self.F, self.dim
        self.embed_prefetch()                   # first step only: nothing has been split ahead
        self.side_stream.wait_stream(main)
        with torch.cuda.stream(self.side_stream):
            x = self.dense
            nb = len(self.bottom)
            for i, (w, b) in enumerate(self.bottom):
                last = i == nb - 1
                y = self.z if last else self.acts_b[i]
                names.append(dev.gemm(x, w, y, m=B, n=w.shape[1], k=w.shape[0], bias=b,
                                      activation=ACT_RELU, ldc=(F * D if last else None),
                                      math=self.math))
                x = y
            self.embed_side()                   # embedding work that needs no peer (writes z too)
            self._bottom_done[buf].record(self.side_stream)
            # the next step's split reuses the masks and lists of the step before this one
            self.side_stream.wait_event(self._sum_done[1 - buf])
            self.embed_prefetch_next()
            self._begin_done.record(self.side_stream)
        self.embed_pool()
        self._pooled.record(main)
        main.wait_event(self._begin_done)       # the next pooling starts after its split
        self.dense_stream.wait_event(self._pooled)
        self.dense_stream.wait_event(self._bottom_done[buf])
        with torch.cuda.stream(self.dense_stream):
            self.embed_finish()
            self._sum_done[buf].record(self.dense_stream)
            self._dense_part(names)
            self._dense_done[buf].record(self.dense_stream)
        return self.out

    def forward_pipelined(self, split: bool = False) -> torch.Tensor:
        """One step of a back-to-back sequence: its dense part is queued on `dense_stream` and
        overlaps the next step's embedding part.  The returned tensor is valid after
        sync_pipeline() (or a device synchronize).  split=True (pipelines with split_finish):
        the closing pass of the embedding part runs on the dense stream too."""
        if split and self.split_finish:
            return self._forward_split()
        buf = self._pstep % 2
        self._pstep += 1
        self._select(buf)
        main = torch.cuda.current_stream()
        main.wait_event(self._dense_done[buf])  # the step before last has finished with this set
        names = []
        self._sparse_part(names, lookahead=True)
        self.dense_stream.wait_stream(main)
        with torch.cuda.stream(self.dense_stream):
            self._dense_part(names)
            self._dense_done[buf].record(self.dense_stream)
        return self.out

    def sync_pipeline(self) -> None:
        """Orders the current stream after every queued dense part."""
        main = torch.cuda.current_stream()
        main.wait_stream(self.dense_stream)
        main.wait_stream(self.side_stream)

    def _issue_copy(self, i: int) -> None:
        st = self.sets[i]
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(self.done[i])  # the step that last read set i is over
            st["ids_all"].copy_(self.h_ids, non_blocking=True)
            st["seg_all"].copy_(self.h_seg, non_blocking=True)
            st["dense"].copy_(self.h_dense, non_blocking=True)
            self.ready[i].record(self.copy_stream)
        self._prefetched[i] = True

    def forward_e2e(self) -> torch.Tensor:
        """Host buffers in, host result out.  Every step copies its three input buffers from
        pinned host memory and its predictions back; the copy of the following step's
        inputs is issued on a second stream first, so it overlaps this step's kernels."""
        cur = self._step % 2
        if not self._prefetched[cur]:
            self._issue_copy(cur)
        self._issue_copy(1 - cur)
        torch.cuda.current_stream().wait_event(self.ready[cur])
        self._use(cur)
        out = self.forward()
        self.h_out.copy_(out, non_blocking=True)
        self.done[cur].record()
        self._prefetched[cur] = False
        self._step += 1
        return self.h_out

    @property
    def h2d_bytes(self) -> int:
        return self.ids_all.numel() * 8 + self.seg_all.numel() * 8 + self.dense.numel() * 4

    @property
    def d2h_bytes(self) -> int:
        return self.out.numel() * 4

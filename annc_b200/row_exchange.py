"""ctypes mirror of the row-sharded embedding exchange (annc_row_exchange_* in
libannc_b200.so).  All protocol logic lives in the library; this module only marshals the
table descriptions, the per-step input descriptors and the peer-buffer pointers.

Partitioning: owner = row % world, local row = row // world
(annc/tensorflow/kernels/embedding_fused_sparse_dynamic_stitch.cc:70-71), plus an optional
replicated set of hot rows per table."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

from ._lib import BagTable, check, lib

ERR_ROW, ERR_SEGMENT, ERR_UNSORTED, ERR_TIMEOUT, ERR_BOUNDS = 1, 2, 4, 8, 16
PHASES = ("split", "barrier1", "pool_exchange", "barrier2", "sum")


class ShardTable(C.Structure):
    _fields_ = [("shard", C.c_void_p), ("local_rows", C.c_int64), ("rows", C.c_int64),
                ("hot_rows", C.c_void_p), ("hot_count", C.c_int64)]


class Config(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("num_tables", C.c_int32),
                ("id_kind", C.c_int32), ("combiner", C.c_int32), ("reserved", C.c_int32),
                ("dim", C.c_int64), ("batch", C.c_int64), ("max_lookups", C.c_int64),
                ("max_lookups_per_table", C.c_int64), ("tables", C.POINTER(ShardTable))]


lib.annc_row_exchange_peer_bytes.restype = C.c_size_t
lib.annc_row_exchange_peer_bytes.argtypes = [C.POINTER(Config)]
lib.annc_row_exchange_create.argtypes = [C.POINTER(Config), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
lib.annc_row_exchange_destroy.argtypes = [C.c_void_p]
lib.annc_row_exchange_begin.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p]
lib.annc_row_exchange_pool.argtypes = [C.c_void_p, C.c_void_p]
lib.annc_row_exchange_finish.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_void_p]
lib.annc_row_exchange_step.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_void_p,
                                       C.c_int64, C.c_int, C.c_void_p]
lib.annc_row_exchange_check.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int)]
lib.annc_row_exchange_clear_errors.argtypes = [C.c_void_p, C.c_void_p]
lib.annc_row_exchange_set_timeout_ms.argtypes = [C.c_void_p, C.c_int64]
lib.annc_row_exchange_set_profiling.argtypes = [C.c_void_p, C.c_int]
lib.annc_row_exchange_set_pool_ctas_per_sm.argtypes = [C.c_void_p, C.c_int]
lib.annc_row_exchange_set_output_slots.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
lib.annc_row_exchange_phase_ms.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
lib.annc_row_exchange_stats.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]


def _stream() -> C.c_void_p:
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def make_config(world: int, rank: int, tables: Sequence[dict], dim: int, batch: int,
                max_lookups: int, max_lookups_per_table: int, combiner: int = 0,
                id_kind: int = 2):
    """tables: per table a dict(shard=ptr of f32[local_rows + hot_count, D], local_rows=, rows=,
    hot_rows=ptr|0, hot_count=).  Returns (Config, keep-alive array)."""
    arr = (ShardTable * len(tables))()
    for i, t in enumerate(tables):
        arr[i].shard = t["shard"] or None
        arr[i].local_rows = int(t["local_rows"])
        arr[i].rows = int(t["rows"])
        arr[i].hot_rows = t.get("hot_rows") or None
        arr[i].hot_count = int(t.get("hot_count", 0))
    cfg = Config(world, rank, len(tables), id_kind, combiner, 0, dim, batch, int(max_lookups),
                 int(max_lookups_per_table), arr)
    return cfg, arr


def peer_bytes(cfg: Config) -> int:
    return int(lib.annc_row_exchange_peer_bytes(C.byref(cfg)))


class StepInputs:
    """Host descriptor array of one batch: per table the ids and the index matrix."""

    def __init__(self, ids_ptrs: Sequence[int], seg_ptrs: Sequence[int], nnz: Sequence[int]):
        self.n = len(nnz)
        self.desc = (BagTable * self.n)()
        for t in range(self.n):
            self.desc[t].ids = ids_ptrs[t] or None
            self.desc[t].slice_input = seg_ptrs[t] or None
            self.desc[t].nnz = int(nnz[t])


class RowExchange:
    def __init__(self, cfg: Config, keep, peer_ptrs: Sequence[int]):
        self.cfg, self._keep = cfg, keep
        self.world = cfg.world
        ptrs = (C.c_void_p * cfg.world)(*[C.c_void_p(int(p)) for p in peer_ptrs])
        h = C.c_void_p()
        check(lib.annc_row_exchange_create(C.byref(cfg), ptrs, C.byref(h)))
        self.h = h

    def begin(self, inputs: StepInputs, ncols: int = 2, col: int = 0) -> None:
        check(lib.annc_row_exchange_begin(self.h, inputs.desc, C.c_int64(ncols), C.c_int32(col), _stream()))

    def pool(self) -> None:
        check(lib.annc_row_exchange_pool(self.h, _stream()))

    def finish(self, out_ptr: int, out_stride: int, out_bf16: bool = False) -> None:
        check(lib.annc_row_exchange_finish(self.h, C.c_void_p(out_ptr), C.c_int64(out_stride),
                                           C.c_int(int(out_bf16)), _stream()))

    def step(self, inputs: StepInputs, out_ptr: int, out_stride: int, out_bf16: bool = False,
             ncols: int = 2, col: int = 0) -> None:
        check(lib.annc_row_exchange_step(self.h, inputs.desc, C.c_int64(ncols), C.c_int32(col),
                                         C.c_void_p(out_ptr), C.c_int64(out_stride),
                                         C.c_int(int(out_bf16)), _stream()))

    def error_bits(self, raise_on_timeout: bool = True) -> int:
        bits = C.c_int(0)
        rc = lib.annc_row_exchange_check(self.h, _stream(), C.byref(bits))
        if rc != 0 and raise_on_timeout:
            check(rc)
        return bits.value

    def clear_errors(self) -> None:
        check(lib.annc_row_exchange_clear_errors(self.h, _stream()))

    def set_timeout_ms(self, ms: int) -> None:
        check(lib.annc_row_exchange_set_timeout_ms(self.h, C.c_int64(ms)))

    def set_output_slots(self, slots) -> None:
        """Table t of the exchange goes to slot slots[t] of the output rows (None: identity)."""
        if slots is None:
            check(lib.annc_row_exchange_set_output_slots(self.h, None, _stream()))
            return
        arr = (C.c_int32 * len(slots))(*[int(v) for v in slots])
        check(lib.annc_row_exchange_set_output_slots(self.h, arr, _stream()))

    def set_pool_ctas_per_sm(self, n: int) -> None:
        check(lib.annc_row_exchange_set_pool_ctas_per_sm(self.h, C.c_int(int(n))))

    def set_profiling(self, on: bool) -> None:
        check(lib.annc_row_exchange_set_profiling(self.h, C.c_int(int(on))))

    def phase_ms(self) -> List[float]:
        ms = (C.c_float * 5)()
        check(lib.annc_row_exchange_phase_ms(self.h, ms))
        return [float(v) for v in ms]

    def stats(self):
        a = (C.c_int64 * self.world)()
        b = (C.c_int64 * self.world)()
        check(lib.annc_row_exchange_stats(self.h, _stream(), a, b))
        return list(a), list(b)

    def destroy(self) -> None:
        if self.h:
            check(lib.annc_row_exchange_destroy(self.h))
            self.h = None

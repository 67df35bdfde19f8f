"""Device-pointer entry points (`*_dev`, annc_gemm_run) on torch CUDA tensors.

torch supplies device memory and the stream; every kernel that runs is from
libannc_b200.so.  Nothing here allocates inside a call: outputs and workspaces are
passed in, so the calls can sit in a timed loop or under stream capture."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from ._lib import (ACT_NONE, B_PLAIN, MATH_AUTO, BagTable, GemmDesc, check, lib)


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class BagPlan:
    """Holds the host descriptor array and the device workspace of one grouped
    embedding-bag call (tables, id buffers, segment matrices and outputs fixed)."""

    def __init__(self, tables: Sequence[torch.Tensor], ids: Sequence[torch.Tensor],
                 slice_inputs: Sequence[torch.Tensor], out: torch.Tensor, out_slot0: int,
                 batch: int, id_kind: int = 2, col: int = 0, combiner: int = 0,
                 num_buckets: Optional[Sequence[int]] = None,
                 out_slots: Optional[Sequence[int]] = None):
        self.n = len(tables)
        self.dim = int(tables[0].shape[1])
        self.batch = int(batch)
        self.id_kind, self.col, self.combiner = id_kind, col, combiner
        self.ncols = int(slice_inputs[0].shape[1])
        self.out = out
        # out is [batch, slots, dim]; table t writes slot out_slot0 + t (or out_slot0 + out_slots[t])
        slots = int(out.shape[1]) if out.dim() == 3 else 1
        self.out_stride = slots * self.dim
        self.keep = (list(tables), list(ids), list(slice_inputs))
        self.desc = (BagTable * self.n)()
        esz = out.element_size()
        for t in range(self.n):
            d = self.desc[t]
            d.table = tables[t].data_ptr()
            d.rows = int(tables[t].shape[0])
            d.num_buckets = int(num_buckets[t]) if num_buckets is not None else int(tables[t].shape[0])
            d.ids = ids[t].data_ptr()
            d.slice_input = slice_inputs[t].data_ptr()
            d.nnz = int(ids[t].shape[0])
            d.out = out.data_ptr() + (out_slot0 + (out_slots[t] if out_slots is not None else t)) * self.dim * esz
        self.ws_bytes = int(lib.annc_embed_bag_workspace_bytes(self.n, self.batch))
        self.ws = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=out.device)

    def run(self) -> None:
        check(lib.annc_embed_bags_dev(self.desc, C.c_int(self.n), C.c_int64(self.dim),
                                      C.c_int(self.id_kind), C.c_int64(self.ncols),
                                      C.c_int32(self.col), C.c_int(self.combiner),
                                      C.c_int64(self.batch), C.c_int64(self.out_stride),
                                      C.c_void_p(self.ws.data_ptr()), C.c_size_t(self.ws_bytes),
                                      _stream()))

    def error_bits(self) -> int:
        bits = C.c_int(0)
        check(lib.annc_embed_bag_check(C.c_void_p(self.ws.data_ptr()), _stream(), C.byref(bits)))
        return bits.value


def gemm(a: torch.Tensor, b: torch.Tensor, c: torch.Tensor, *, m: int, n: int, k: int,
         trans_a: bool = False, trans_b: bool = False, batch: int = 1,
         lda: Optional[int] = None, ldb: Optional[int] = None, ldc: Optional[int] = None,
         stride_a: int = 0, stride_b: int = 0, stride_c: int = 0,
         alpha: float = 1.0, beta: float = 0.0, addend: Optional[torch.Tensor] = None,
         ld_addend: Optional[int] = None, stride_addend: int = 0,
         bias: Optional[torch.Tensor] = None, activation: int = ACT_NONE,
         b_format: int = B_PLAIN, math: int = MATH_AUTO,
         workspace: Optional[torch.Tensor] = None, io_flags: int = 0) -> str:
    """annc_gemm_run; returns the name of the kernel family that ran."""
    d = GemmDesc()
    d.trans_a, d.trans_b = int(trans_a), int(trans_b)
    d.m, d.n, d.k, d.batch = m, n, k, batch
    d.lda = lda if lda is not None else (m if trans_a else k)
    d.ldb = ldb if ldb is not None else (k if trans_b else n)
    d.ldc = ldc if ldc is not None else n
    d.ld_addend = ld_addend if ld_addend is not None else n
    d.stride_a, d.stride_b, d.stride_c, d.stride_addend = stride_a, stride_b, stride_c, stride_addend
    d.alpha, d.beta = alpha, beta
    d.a, d.b, d.c = a.data_ptr(), b.data_ptr(), c.data_ptr()
    d.addend = addend.data_ptr() if addend is not None else None
    d.bias = bias.data_ptr() if bias is not None else None
    d.activation, d.b_format, d.math = activation, b_format, math
    d.io_flags = io_flags
    if workspace is not None:
        d.workspace, d.workspace_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    name = lib.annc_gemm_kernel_name(C.byref(d)).decode()
    check(lib.annc_gemm_run(C.byref(d), _stream()))
    return name


def softmax(x: torch.Tensor, out: torch.Tensor) -> None:
    ch = x.shape[-1]
    check(lib.annc_softmax_dev(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()),
                               C.c_int64(x.numel() // ch), C.c_int64(ch), _stream()))


def gemv(a: torch.Tensor, x: torch.Tensor, y: torch.Tensor, m: int, n: int, trans_a=False,
         alpha=1.0, beta=0.0) -> None:
    check(lib.annc_gemv_dev(C.c_int(int(trans_a)), C.c_int64(m), C.c_int64(n), C.c_float(alpha),
                            C.c_void_p(a.data_ptr()), C.c_void_p(x.data_ptr()), C.c_float(beta),
                            C.c_void_p(y.data_ptr()), _stream()))


def dot_interaction(z: torch.Tensor, out: torch.Tensor, math: int = MATH_AUTO) -> None:
    """z f32[batch, F, D] -> out f32[batch, out_stride] = [z[:,0,:] | tril(z z^T, -1) | 0 pad]."""
    batch, F, D = z.shape
    check(lib.annc_dot_interaction_dev(C.c_void_p(z.data_ptr()), C.c_int64(batch), C.c_int(F),
                                       C.c_int(D), C.c_int64(F * D), C.c_void_p(out.data_ptr()),
                                       C.c_int64(out.shape[1]), C.c_int(math), _stream()))


def bf16_weight(b_kn: torch.Tensor) -> torch.Tensor:
    """fp32 [K,N] -> bf16 [N,K] for the BF16 route (annc_bf16_weight_dev)."""
    k, n = b_kn.shape
    out = torch.empty((n, k), dtype=torch.bfloat16, device=b_kn.device)
    check(lib.annc_bf16_weight_dev(C.c_void_p(b_kn.data_ptr()), C.c_int64(b_kn.stride(0)),
                                   C.c_void_p(out.data_ptr()), C.c_int64(k), C.c_int64(n), _stream()))
    return out


def cast_bf16(x: torch.Tensor) -> torch.Tensor:
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    check(lib.annc_cast_bf16_dev(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()),
                                 C.c_int64(x.numel()), _stream()))
    return out


def kn4_pack(b_kn: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(b_kn)
    check(lib.annc_kn4_pack_dev(C.c_void_p(b_kn.data_ptr()), C.c_void_p(out.data_ptr()),
                                C.c_int64(b_kn.shape[0]), C.c_int64(b_kn.shape[1]), _stream()))
    return out


def kn4_unpack(b_packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(b_packed)
    check(lib.annc_kn4_unpack_dev(C.c_void_p(b_packed.data_ptr()), C.c_void_p(out.data_ptr()),
                                  C.c_int64(b_packed.shape[0]), C.c_int64(b_packed.shape[1]),
                                  _stream()))
    return out


def gemm_timed_out() -> bool:
    """True when a tensor-core GEMM CTA gave up on a bounded wait since the library was
    loaded (annc_gemm_check; synchronises the current stream)."""
    flag = C.c_int(0)
    check(lib.annc_gemm_check(_stream(), C.byref(flag)))
    return flag.value != 0


class BagLaunch:
    """Grouped embedding-bag launch over explicit (table, ids, segments, output) entries,
    optionally row-sharded (annc_embed_bags_sharded_dev).  Each entry is a tuple
    (table_ptr, local_rows, num_buckets, ids_ptr, seg_ptr, nnz, out_ptr[, offsets_ptr]); with
    offsets_ptr (i32[batch + 1] bag offsets) the segment matrix is not read."""

    def __init__(self, entries, dim: int, batch: int, ncols: int, out_stride: int,
                 device: torch.device, id_kind: int = 2, col: int = 0, combiner: int = 0,
                 shard_count: int = 1, shard_rank: int = 0, exchange: bool = False):
        self.exchange = exchange  # annc_embed_bags_exchange_dev: bags without an owned lookup are not written
        self.n = len(entries)
        self.dim, self.batch, self.ncols, self.out_stride = dim, batch, ncols, out_stride
        self.id_kind, self.col, self.combiner = id_kind, col, combiner
        self.shard_count, self.shard_rank = shard_count, shard_rank
        self.desc = (BagTable * self.n)()
        for i, e in enumerate(entries):
            tp, rows, nb, ip, sp, nnz, op = e[:7]
            d = self.desc[i]
            d.table, d.rows, d.num_buckets, d.ids, d.slice_input, d.nnz, d.out = \
                tp, int(rows), int(nb), ip, sp, int(nnz), op
            d.offsets = e[7] if len(e) > 7 else None
        self.ws_bytes = int(lib.annc_embed_bag_workspace_bytes(self.n, self.batch))
        self.ws = torch.zeros(self.ws_bytes, dtype=torch.uint8, device=device)

    def run(self) -> None:
        if self.exchange:
            check(lib.annc_embed_bags_exchange_dev(
                self.desc, C.c_int(self.n), C.c_int64(self.dim), C.c_int(self.id_kind),
                C.c_int(self.combiner), C.c_int64(self.batch), C.c_int64(self.out_stride),
                C.c_int(self.shard_count), C.c_int(self.shard_rank),
                C.c_void_p(self.ws.data_ptr()), C.c_size_t(self.ws_bytes), _stream()))
            return
        check(lib.annc_embed_bags_sharded_dev(
            self.desc, C.c_int(self.n), C.c_int64(self.dim), C.c_int(self.id_kind),
            C.c_int64(self.ncols), C.c_int32(self.col), C.c_int(self.combiner),
            C.c_int64(self.batch), C.c_int64(self.out_stride), C.c_int(self.shard_count),
            C.c_int(self.shard_rank), C.c_void_p(self.ws.data_ptr()), C.c_size_t(self.ws_bytes),
            _stream()))

    def error_bits(self) -> int:
        bits = C.c_int(0)
        check(lib.annc_embed_bag_check(C.c_void_p(self.ws.data_ptr()), _stream(), C.byref(bits)))
        return bits.value


def sum_partials(src: torch.Tensor, parts: int, part_stride: int, rows: int, width: int,
                 src_stride: int, out_ptr: int, out_stride: int) -> None:
    check(lib.annc_sum_partials_dev(C.c_void_p(src.data_ptr()), C.c_int(parts), C.c_int64(part_stride),
                                    C.c_int64(rows), C.c_int64(width), C.c_int64(src_stride),
                                    C.c_void_p(out_ptr), C.c_int64(out_stride), _stream()))


def sum_partials_ptr(src_ptr: int, parts: int, part_stride: int, rows: int, width: int,
                     src_stride: int, out_ptr: int, out_stride: int) -> None:
    check(lib.annc_sum_partials_dev(C.c_void_p(src_ptr), C.c_int(parts), C.c_int64(part_stride),
                                    C.c_int64(rows), C.c_int64(width), C.c_int64(src_stride),
                                    C.c_void_p(out_ptr), C.c_int64(out_stride), _stream()))


def peer_copy(dst_ptr: int, src_ptr: int, nbytes: int) -> None:
    """annc_peer_copy_dev on the current stream (raw pointers: either may be a peer mapping)."""
    check(lib.annc_peer_copy_dev(C.c_void_p(dst_ptr), C.c_void_p(src_ptr), C.c_size_t(nbytes), _stream()))


def cast_bf16_ptr(src_ptr: int, dst_ptr: int, n: int) -> None:
    check(lib.annc_cast_bf16_dev(C.c_void_p(src_ptr), C.c_void_p(dst_ptr), C.c_int64(n), _stream()))


class OwnerMask:
    """annc_embed_bag_owner_mask_dev over fixed id / offset buffers: which ranks hold a part
    of each bag of this rank's batch.  entries: (ids_ptr, nnz, num_buckets, offsets_ptr)."""

    def __init__(self, entries, batch: int, shard_count: int, device: torch.device, id_kind: int = 2):
        self.n, self.batch, self.shard_count, self.id_kind = len(entries), batch, shard_count, id_kind
        self.desc = (BagTable * self.n)()
        for i, (ip, nnz, nb, op) in enumerate(entries):
            d = self.desc[i]
            d.ids, d.nnz, d.num_buckets, d.offsets = ip, int(nnz), int(nb), op
        self.mask = torch.zeros(self.n * batch, dtype=torch.int32, device=device)

    def run(self) -> None:
        check(lib.annc_embed_bag_owner_mask_dev(self.desc, C.c_int(self.n), C.c_int(self.id_kind),
                                                C.c_int64(self.batch), C.c_int(self.shard_count),
                                                C.c_void_p(self.mask.data_ptr()), _stream()))


def sum_partials_masked(src_ptr: int, mask: torch.Tensor, parts: int, part_stride: int, rows: int,
                        slots: int, slot_width: int, out_ptr: int, out_stride: int,
                        mean_offsets_ptr: Optional[int] = None, out_bf16: bool = False) -> None:
    check(lib.annc_sum_partials_masked_dev(C.c_void_p(src_ptr), C.c_void_p(mask.data_ptr()),
                                           C.c_int(parts), C.c_int64(part_stride), C.c_int64(rows),
                                           C.c_int(slots), C.c_int64(slot_width),
                                           C.c_void_p(mean_offsets_ptr), C.c_void_p(out_ptr),
                                           C.c_int64(out_stride), C.c_int(int(out_bf16)), _stream()))


class PeerBuffers:
    """One receive buffer per rank, mapped into every rank (annc_peer_buffer_*).  `local` is
    this rank's buffer, `ptrs[p]` the address under which rank p's buffer is seen here.
    Handles travel through torch.distributed (host side); the data path is plain stores."""

    def __init__(self, nbytes: int, world: int, rank: int):
        import torch.distributed as dist
        ptr = C.c_void_p()
        handle = (C.c_ubyte * 64)()
        check(lib.annc_peer_buffer_create(C.c_size_t(nbytes), C.byref(ptr), handle))
        self.local = int(ptr.value)
        self.nbytes, self.rank = nbytes, rank
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle))
        self.ptrs = []
        for p in range(world):
            if p == rank:
                self.ptrs.append(self.local)
                continue
            q = C.c_void_p()
            buf = (C.c_ubyte * 64).from_buffer_copy(handles[p])
            check(lib.annc_peer_buffer_open(buf, C.byref(q)))
            self.ptrs.append(int(q.value))

    def close(self) -> None:
        """Unmaps the peers' buffers, waits for every rank to have done so, frees this one."""
        import torch.distributed as dist
        for p, q in enumerate(self.ptrs):
            if p != self.rank and q:
                check(lib.annc_peer_buffer_close(C.c_void_p(q)))
        self.ptrs = []
        if dist.is_initialized():
            dist.barrier()
        if self.local:
            check(lib.annc_peer_buffer_destroy(C.c_void_p(self.local)))
            self.local = 0


def copy_rows(dst_ptr: int, dst_stride: int, src_ptr: int, src_stride: int, width: int,
              rows: int) -> None:
    """2-D device copy of `rows` rows of `width` floats between pitched buffers."""
    check(lib.annc_copy_rows_dev(C.c_void_p(dst_ptr), C.c_int64(dst_stride), C.c_void_p(src_ptr),
                                 C.c_int64(src_stride), C.c_int64(width), C.c_int64(rows), _stream()))


class BagPrepass:
    """Segment prepass alone (annc_embed_bag_prepass_dev): bag offsets of every table's
    lookups into `ws` (512-byte header, then i32 offsets[tables][batch + 1])."""

    def __init__(self, slice_inputs: Sequence[torch.Tensor], batch: int, col: int = 0):
        self.n = len(slice_inputs)
        self.batch, self.col = int(batch), col
        self.ncols = int(slice_inputs[0].shape[1])
        self.desc = (BagTable * self.n)()
        for t, s in enumerate(slice_inputs):
            self.desc[t].slice_input = s.data_ptr()
            self.desc[t].nnz = int(s.shape[0])
        self.ws_bytes = int(lib.annc_embed_bag_workspace_bytes(self.n, self.batch))

    def run(self, ws: torch.Tensor) -> None:
        self.run_ptr(ws.data_ptr())

    def run_ptr(self, ws_ptr: int) -> None:
        check(lib.annc_embed_bag_prepass_dev(self.desc, C.c_int(self.n), C.c_int64(self.ncols),
                                             C.c_int32(self.col), C.c_int64(self.batch),
                                             C.c_void_p(ws_ptr), C.c_size_t(self.ws_bytes),
                                             _stream()))

#!/usr/bin/env python
"""DLRM-style inference benchmark of annc_b200 (one process per GPU).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --steps K --warmup W    # CPU reference arm
    ... --workload recsys                                    # the large row-sharded configuration

The default workload is the DLRM-style model below.  `--workload recsys` is the 64-table,
dim-128, mean-pooled, BF16-MLP configuration whose 655 GB of tables need 8 GPUs: tables are
hashed on the device and row-sharded, each GPU holds 2.5 M rows of every table at every N
(20 M rows per table at N = 8) and a batch of 16384 samples.

A step is one inference pass over one synthetic batch of the DLRM-style config
(13 dense, bottom MLP 13-512-256-64, 26 tables with log-uniform rows 1e3..1e7,
dim 64, Zipf 1.05 ids, bags 1..20, dot interaction, top MLP 415-512-256-1,
batch 65536 per GPU, fp32 weights / TF32 tensor-core math).  Prints one JSON line.

Timing: W >= 3 warm-up steps, then K steps bracketed by a barrier and a device
synchronize, CUDA events on the launching stream, max over ranks.  Every step's
inputs (6.6 GB of tables, 0.43 GB of ids) are far larger than the 126 MB L2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "dlrm_inference_samples_per_s"
UNIT = "samples/s"

# DRAM bytes (read + write) of one bag-kernel launch: a constant, not measured by this run.  It is
# the dram__bytes_read.sum + dram__bytes_write.sum of a profiler capture of the small case
# (batch 16384, rows <= 1e6: 0.5465 GB for 4,472,660 lookups) scaled to this workload by the lookups
# per launch; traffic grows in proportion (the same scaling of the previous kernel's small-case
# figure matched a full-size capture within 2 %).  Keyed by (batch, max_rows, seed); any other
# workload reports null.
NCU_BAG_TRAFFIC_BYTES = {(65536, 1e7, 0): 0.5465e9 * 17883957 / 4472660}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="annc_b200", choices=["annc_b200", "reference"])
    ap.add_argument("--workload", default="dlrm", choices=["dlrm", "recsys"])
    ap.add_argument("--batch", type=int, default=None,
                    help="samples per GPU per step (default 65536 for dlrm, 16384 for recsys)")
    ap.add_argument("--rows-per-gpu", type=float, default=2.5e6,
                    help="recsys: rows of every table held by one GPU (table rows = this x GPUs)")
    ap.add_argument("--tables", type=int, default=64, help="recsys: number of tables")
    ap.add_argument("--max-rows", type=float, default=1e7)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--shard", default="row", choices=["row", "row_nccl", "table", "table_nccl", "replica"],
                    help="table partitioning timed as the line's `value` for --gpus > 1: row = mod "
                         "row-sharding (the library's row exchange: lookups split by owner at their "
                         "source, partial sums stored into the sample owner's memory, optional "
                         "replicated hot rows); row_nccl = all-gathered ids and an NCCL all-to-all; "
                         "table = whole tables per rank; replica = no exchange")
    ap.add_argument("--hot-rows", type=int, default=65536,
                    help="row sharding: rows of each table's this many most popular ids are replicated "
                         "on every rank and pooled where the sample is (0 = pure row sharding)")
    ap.add_argument("--extras", default="row_k0,row_k262144,table,replica",
                    help="--gpus > 1: other partitionings timed after the headline and reported as "
                         "labelled sub-records (comma list of row_k0, row_k<K> = row sharding with K "
                         "replicated rows per table, row_nccl, table, table_nccl, replica; empty = none)")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-operator record at N=1")
    ap.add_argument("--no-abi", action="store_true", help="skip the host-buffer ABI leg at N=1")
    args = ap.parse_args()
    if args.batch is None:
        args.batch = 65536 if args.workload == "dlrm" else 16384
    return args


def parallelism_label(args, world, mode=None):
    mode = mode or args.shard
    if world == 1 and args.workload == "dlrm":
        return "single"
    hot = (" + rows of each table's %d most popular ids replicated (a table with no more rows than that is "
           "replicated whole and pooled outside the exchange)" % args.hot_rows) if args.hot_rows > 0 else ""
    return {
        "row": "dp%d MLP + row-sharded tables (owner = row %% %d)%s; lookups split by owner at their source, "
               "partial sums stored into the sample owner's memory by the pooling kernel, flag barriers"
               % (world, world, hot),
        "row_k0": "dp%d MLP + row-sharded tables (owner = row %% %d), no replicated rows" % (world, world),
        "row_kK": "dp%d MLP + row-sharded tables (owner = row %% %d) + rows of each table's %s most popular "
                  "ids replicated" % (world, world, (mode or "")[5:]),
        "row_nccl": "dp%d MLP + row-sharded tables, all-gathered ids + NCCL all-to-all of partial sums" % world,
        "table": "dp%d MLP + whole tables per rank, pooled vectors stored into the sample owner's memory" % world,
        "table_nccl": "dp%d MLP + whole tables per rank, NCCL all-to-all of ids and pooled vectors" % world,
        "replica": "dp%d MLP + every table on every rank (no exchange)" % world,
    }["row_kK" if mode.startswith("row_k") and mode != "row_k0" else mode]


def workload_config(args, world):
    if args.workload == "recsys":
        rows = int(args.rows_per_gpu) * world
        return {"workload": "recsys_%dtables_x_%drows_dim128_mean_pool_bf16_mlp_8192-1024-512-1_batch%d"
                            % (args.tables, rows, args.batch * world),
                "global_batch": args.batch * world, "per_gpu_batch": args.batch, "tables": args.tables,
                "dim": 128, "rows": rows, "bag": "U{1..50}, Zipf 1.2, mean",
                "table_bytes_total": args.tables * rows * 512,
                "parallelism": parallelism_label(args, world),
                "l2": "inputs larger than L2 (table shard %.1f GB per GPU)" % (args.tables * int(args.rows_per_gpu) * 512 / 1e9)}
    return {"workload": "dlrm_style_fp32w_tf32math_batch%d_26tables_dim64_zipf1.05" % args.batch,
            "global_batch": args.batch * world, "per_gpu_batch": args.batch,
            "tables": 26, "dim": 64, "rows": "log-uniform 1e3..%g" % args.max_rows,
            "parallelism": parallelism_label(args, world),
            "l2": "inputs larger than L2 (tables 6.6 GB, ids 0.43 GB per step)"}


# ---------------------------------------------------------------- clocks

class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""

    def __init__(self, index: int, period: float = 0.05):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._halt.set()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


def bind_to_gpu_numa_node(gpu_index: int):
    """Restricts this process to the CPU cores NVML names as local to its GPU (intersected with
    the cores it may use), before any pinned host buffer is allocated: with one process per GPU
    the pinned step inputs then sit on the GPU's own NUMA node and the host-to-device copies of
    eight ranks do not all cross one socket.  Returns the number of cores kept, or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        local = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        keep = local & os.sched_getaffinity(0)
        if keep and keep != os.sched_getaffinity(0):
            os.sched_setaffinity(0, keep)
        return len(keep) if keep else None
    except Exception:
        return None


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ---------------------------------------------------------------- CPU arm

def cpu_forward_timed(model, threads, reps, sample=None):
    from oracle import oracle
    oracle.dlrm_forward(model, sample=min(2048, model.emb.batch), threads=threads)  # page-in
    t = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.dlrm_forward(model, sample=sample, threads=threads)
        t.append(time.perf_counter() - t0)
    return t


def recsys_cpu_timed(args, threads, reps):
    """CPU arm of the recsys workload on a bounded sample: ONE of the tables with its rows
    reduced to 1e6 (regenerated from the hash), this batch's bags mean-pooled by the C port,
    the time scaled by the number of tables, plus the fp32 MLP (OpenBLAS sgemm) on the full
    [batch, tables*128] input."""
    import numpy as np
    from annc_b200 import synth
    from oracle import oracle
    rows = 1_000_000
    model = synth.recsys_model(seed=args.seed, tables=1, rows=rows, batch=args.batch, input_seed=1000)
    table = synth.hashed_table_rows(args.seed, 0, np.arange(rows), 128)
    bag = model.bags[0]
    idx = oracle.hash_bucket(bag.raw_ids.view(np.uint64), rows)
    full = synth.recsys_model(seed=args.seed, tables=args.tables, rows=rows, batch=8, input_seed=1000)
    x = np.random.default_rng(0).standard_normal((args.batch, args.tables * 128), dtype=np.float32)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.sparse_segment_reduce(table, idx, bag.slice_input, np.array([0, 0], np.int32),
                                     np.array([0], np.int32), 1)
        t_pool = (time.perf_counter() - t0) * args.tables / max(1, min(threads, args.tables))
        t0 = time.perf_counter()
        h = x
        for i, (w, b) in enumerate(full.mlp):
            h = oracle.matmul(h, w) + b
            h = np.maximum(h, 0) if i < len(full.mlp) - 1 else 1 / (1 + np.exp(-h))
        ts.append(t_pool + time.perf_counter() - t0)
    return ts


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from annc_b200 import synth
    from oracle import oracle
    if args.workload == "recsys":
        threads = oracle.host_threads()
        times = recsys_cpu_timed(args, threads, args.warmup + args.steps)[args.warmup:]
        ms = 1e3 * sum(times) / len(times)
        value = args.batch / (ms / 1e3)
        sample = ("1 of %d tables pooled (rows reduced to 1e6), time x %d / min(threads, tables); "
                  "fp32 MLP on the full batch of %d" % (args.tables, args.tables, args.batch))
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
                "config": workload_config(args, 1),
                "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
                "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return
    model = synth.dlrm_model(seed=args.seed, batch=args.batch, max_rows=args.max_rows)
    threads = oracle.host_threads()
    n = model.emb.batch
    times = cpu_forward_timed(model, threads, args.warmup + args.steps)[args.warmup:]
    ms = 1e3 * sum(times) / len(times)
    value = n / (ms / 1e3)
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
            "config": workload_config(args, 1),
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                             "sample": "one full batch of %d samples per step; C restatement of the "
                                       "reference kernels + OpenBLAS sgemm" % n},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- GPU arm

def cpu_baselines(args, model, pipe_out):
    """CPU legs at N=1 (DLRM): the C port of the reference kernels + OpenBLAS on all host cores
    over full batches, the same on one thread (the reference's deployment setting,
    OMP_NUM_THREADS=1) over a bounded sample, and the parity of the GPU predictions of the very
    batch that was timed against the all-core leg's output."""
    import numpy as np
    from oracle import oracle
    threads = oracle.host_threads()
    oracle.set_blas_threads(threads)
    oracle.dlrm_forward(model, sample=min(2048, model.emb.batch), threads=threads)  # page-in
    t, ref = [], None
    for _ in range(3):
        t0 = time.perf_counter()
        ref = oracle.dlrm_forward(model, threads=threads)
        t.append(time.perf_counter() - t0)
    cpu_ms = 1e3 * sum(t) / len(t)
    base = {"value": args.batch / (cpu_ms / 1e3), "unit": UNIT, "cores": threads, "kind": "port",
            "ms_per_step": cpu_ms,
            "sample": "3 full batches of %d samples (C restatement of the reference kernels, one table "
                      "per thread, + OpenBLAS sgemm)" % args.batch}
    parity = float(np.abs(pipe_out - ref).max())
    n1 = min(8192, model.emb.batch)
    oracle.set_blas_threads(1)
    t1 = []
    for _ in range(2):
        t0 = time.perf_counter()
        oracle.dlrm_forward(model, sample=n1, threads=1)
        t1.append(time.perf_counter() - t0)
    oracle.set_blas_threads(threads)
    ms1 = 1e3 * sum(t1) / len(t1)
    one = {"value": n1 / (ms1 / 1e3), "unit": UNIT, "cores": 1, "kind": "port", "ms_per_sample_batch": ms1,
           "sample": "2 passes over the first %d samples of the batch, one thread (OMP_NUM_THREADS=1 is the "
                     "reference's deployment setting)" % n1}
    return base, one, parity


def abi_leg(args, model, pipe_out):
    """The same step through the reference-named entry points with HOST buffers (the drop-in
    path itself): Σ of the time inside the library's calls per step.  Every step gets a new
    batch in the same input buffers; weights, tables and broadcast biases upload once, and an
    operand the host did not touch since the library wrote it is not uploaded again."""
    import numpy as np
    from annc_b200._lib import lib
    from annc_b200.abi_step import AbiDlrmStep
    import ctypes as C
    step = AbiDlrmStep(model)
    step.load_batch(1)
    step.forward()
    step.load_batch(0)
    got = step.forward()
    err = float(np.abs(got - pipe_out).max()) if pipe_out is not None else None
    cnt = [C.c_uint64(0) for _ in range(3)]
    lib.annc_staging_counters(*[C.byref(c) for c in cnt])
    h0, d0 = cnt[0].value, cnt[1].value
    step.call_seconds, step.calls = 0.0, 0
    n = 3
    for i in range(n):
        step.load_batch(2 + i)
        step.forward()
    lib.annc_staging_counters(*[C.byref(c) for c in cnt])
    ms = 1e3 * step.call_seconds / n
    h2d, d2h = (cnt[0].value - h0) // n, (cnt[1].value - d0) // n
    lib.annc_release_device_memory()
    return {"value": args.batch / (ms / 1e3), "unit": UNIT, "ms_per_step": ms, "calls_per_step": step.calls // n,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
            "pcie_floor_ms_at_55GBs": (h2d + d2h) / 55e9 * 1e3,
            "max_abs_diff_vs_device_pipeline": err,
            "what": "sum of the time inside the %d reference-named calls of one step "
                    "(__matmul_add_relu / __matmul_add per MLP layer, KPFusedSparseSegmentReduce per "
                    "table, __batch_matmul for the interaction) with pageable host buffers in and out; "
                    "every intermediate returns to the host as the reference's ABI requires; the "
                    "graph's own glue between calls is not timed" % (step.calls // n)}


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import numpy as np

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (annc_b200 has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    devi = torch.device("cuda", local_rank)
    numa_cores = bind_to_gpu_numa_node(physical_gpu_index(local_rank)) if world > 1 else None
    if world > 1:
        dist.init_process_group("nccl", device_id=devi)

    from annc_b200 import synth
    from annc_b200._lib import lib
    from annc_b200.dlrm import DlrmPipeline
    import ctypes as C

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, sync=None):
        """Device time of `steps` calls, max over ranks.  `sync` orders the timing stream after
        work the calls queued on other streams, so that all of it lies inside the timed region."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        if sync is not None:
            sync()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=devi)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def close(pipe):
        torch.cuda.synchronize()
        if args.workload == "recsys":
            pipe.close()
        elif hasattr(pipe, "close_exchange"):
            pipe.close_exchange()

    recsys = args.workload == "recsys"
    if recsys:
        from annc_b200.recsys import RecsysPipeline
        if world == 1:  # the peer buffers are exchanged over torch.distributed at every N
            dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % (29000 + os.getpid() % 2000),
                                    rank=0, world_size=1, device_id=devi)
        args.shard = "table" if args.shard == "table" else "row"
        model = synth.recsys_model(seed=args.seed, tables=args.tables, rows=int(args.rows_per_gpu) * world,
                                   batch=args.batch, input_seed=1000 + rank)
        nnz = model.nnz
        emb_bytes = nnz * (4 * 128 + 8 + 8) + args.tables * args.batch * 4 * 128
        bag_kernel = "pool_kernel<32,1> (row exchange: gather + segment mean + peer stores, %d tables)" % args.tables
        if args.shard == "table":
            bag_kernel = "bag_reduce_kernel<32,1> (hash-bucket + gather + segment mean, %d tables)" % args.tables

        def build(mode):
            return RecsysPipeline(model, devi, keep_host_inputs=True, shard="table" if mode == "table" else "row",
                                  hot_rows=args.hot_rows if mode == "row" else 0)
    else:
        model = synth.dlrm_model(seed=args.seed, batch=args.batch, max_rows=args.max_rows,
                                 input_seed=(1000 + rank) if world > 1 else None)
        emb_bytes = model.emb.algorithmic_bytes()
        nnz = model.emb.nnz
        bag_kernel = "bag_stream_kernel<8,4,2,16,2,5> (hash-bucket + gather + segment sum, 26 tables in one launch)"

        def build(mode):
            if world == 1:
                return DlrmPipeline(model, devi, keep_host_inputs=True)
            from annc_b200.sharded import ShardedDlrmPipeline
            if mode.startswith("row_k"):
                return ShardedDlrmPipeline(model, devi, "row", keep_host_inputs=True, hot_rows=int(mode[5:]))
            return ShardedDlrmPipeline(model, devi, mode, keep_host_inputs=True,
                                       hot_rows=args.hot_rows if mode == "row" else 0)

    pipe = build(args.shard)
    for _ in range(max(3, args.warmup)):
        pipe.forward()
    torch.cuda.synchronize()
    assert pipe.embed_error_bits() == 0, "embedding kernels flagged an index error"

    # device-resident pass: the whole step, and (N=1) the bag kernel alone through event hooks
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    pairs = [(C.c_void_p(lib.annc_timer_create()), C.c_void_p(lib.annc_timer_create()))
             for _ in range(args.steps)]
    it = iter(pairs)

    # Back-to-back batches may be issued in two orders: one step after the other (forward), or
    # with the dense part of a step (interaction + top MLP) on a second stream under the next
    # step's embedding part and, under row sharding, the split of the next step under this
    # step's pooling (DlrmPipeline.forward_pipelined).  Which one is faster depends on how much
    # of the GPU the embedding part leaves free; five steps of each decide, the same on all ranks.
    # Under row sharding there is a third order (forward_pipelined(split=True)): the sum of the
    # parts moves to the dense stream as well, so the pooling kernels, bound by their NVLink
    # stores, follow one another on the main stream; optionally with one block per SM fewer
    # in the pooling grid, which leaves room for the kernels of the other streams.
    step_fn, issue_order, order_ms = pipe.forward, "none", {}
    if hasattr(pipe, "forward_pipelined"):
        rowex = getattr(getattr(pipe, "rowbags", None), "ex", None)
        cands = [("none", pipe.forward, 0), ("dense_part_under_next_embedding", pipe.forward_pipelined, 0)]
        if getattr(pipe, "split_finish", False) and rowex is not None:
            fs = lambda: pipe.forward_pipelined(split=True)
            cands += [("sum_and_dense_part_under_next_pooling", fs, 0),
                      ("sum_and_dense_part_under_next_pooling_grid_minus_1", fs, -1),
                      ("sum_and_dense_part_under_next_pooling_grid_minus_2", fs, -2)]
        if getattr(pipe, "whole_tables", None) and rowex is not None:
            # the tables replicated whole pooled on the side stream with k blocks per SM, the
            # exchange's pooling kernel with k fewer
            cands += [("sum_and_dense_part_under_next_pooling_whole_tables_beside_it_%d_blocks" % k, fs, -k)
                      for k in (2, 3)]
            # the same with one block slot per SM left free for the split and the sum
            cands += [("sum_and_dense_part_under_next_pooling_whole_tables_beside_it_2_blocks_pooling_2", fs, 2)]
        best, order_ms = None, {}
        for name, fn, ctas in cands:
            if rowex is not None:
                rowex.set_pool_ctas_per_sm(ctas)
            if hasattr(pipe, "whole_on_side"):
                pipe.whole_on_side = (-ctas if ctas < 0 else 2) if "whole_tables_beside" in name else 0
            for _ in range(3):
                fn()
            t = timed(fn, 5, pipe.sync_pipeline)
            order_ms[name] = round(t / 5, 4)
            if best is None or t < best[0]:
                best = (t, name, fn, ctas)
        _, issue_order, step_fn, ctas = best
        if rowex is not None:
            rowex.set_pool_ctas_per_sm(ctas)
        if hasattr(pipe, "whole_on_side"):
            pipe.whole_on_side = (-ctas if ctas < 0 else 2) if "whole_tables_beside" in issue_order else 0

    def step_with_hooks():
        a, b = next(it)
        lib.annc_embed_bag_set_timing_events(a, b)
        step_fn()

    hooks = world == 1 and not recsys
    for _ in range(3):
        step_fn()
    torch.cuda.synchronize()
    ms_total = timed(step_with_hooks if hooks else step_fn, args.steps, getattr(pipe, "sync_pipeline", None))
    lib.annc_embed_bag_set_timing_events(None, None)
    bag_ms = []
    for a, b in pairs:
        if hooks:
            v = C.c_float(0)
            lib.annc_timer_elapsed_ms(a, b, C.byref(v))
            bag_ms.append(v.value)
        lib.annc_timer_destroy(a)
        lib.annc_timer_destroy(b)
    ms_step = ms_total / args.steps
    if getattr(getattr(pipe, "rowbags", None), "ex", None) is not None:
        pipe.rowbags.ex.set_pool_ctas_per_sm(0)  # the single steps below use the whole grid
    assert pipe.embed_error_bits() == 0, "embedding kernels flagged an error in the timed steps"
    # one step alone, nothing of a neighbouring step under it (latency rather than throughput)
    ms_alone = timed(pipe.forward, args.steps) / args.steps

    # end-to-end pass: host buffers in, host result out
    for _ in range(2):
        pipe.forward_e2e()
    ms_e2e = timed(pipe.forward_e2e, args.steps) / args.steps
    sampler.stop()
    sampler.join(timeout=2)

    value = args.batch * world / (ms_step / 1e3)
    e2e_value = args.batch * world / (ms_e2e / 1e3)

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_source = "measured" if "hbm_gbs" in peaks else "fallback"

    # row exchange: per-rank phase times (CUDA events inside the library, profiled steps after
    # the timed region) and what crossed NVLink
    exchange = None
    rowbags = getattr(pipe, "rowbags", None) or (getattr(pipe, "bags", None) if recsys and args.shard == "row" else None)
    if rowbags is not None and hasattr(rowbags, "ex"):
        rowbags.ex.set_profiling(True)
        ph = []
        for _ in range(5):
            barrier()
            pipe.forward()
            torch.cuda.synchronize()
            ph.append(rowbags.ex.phase_ms())
        rowbags.ex.set_profiling(False)
        med = [float(np.median([p[i] for p in ph])) for i in range(5)]
        st = rowbags.exchange_stats()
        mine = torch.tensor(med + [float(st["nvlink_bytes"]), float(st["remote_parts_received"]),
                                   float(st["remote_records"])], device=devi, dtype=torch.float64)
        if world > 1:
            allr = [torch.zeros_like(mine) for _ in range(world)]
            dist.all_gather(allr, mine)
        else:
            allr = [mine]
        allr = [x.cpu().tolist() for x in allr]
        from annc_b200.row_exchange import PHASES
        pool_ms = max(x[2] for x in allr)
        nv_bytes = max(x[5] for x in allr)
        exchange = {
            "phases": list(PHASES),
            "phase_ms_per_rank": [[round(v, 4) for v in x[:5]] for x in allr],
            "phase_ms_max_over_ranks": [round(max(x[i] for x in allr), 4) for i in range(5)],
            "hot_rows_per_table": args.hot_rows,
            "tables_replicated_whole": len(getattr(pipe, "whole_tables", [])),
            "hot_bytes_per_gpu": st["hot_bytes"] + getattr(pipe, "whole_bytes", 0),
            "remote_parts_per_bag": st["remote_parts_per_bag"],
            "nvlink_bytes_per_gpu_per_step": nv_bytes,
            "nvlink_gbs_in_pool_kernel": nv_bytes / (pool_ms / 1e3) / 1e9 if pool_ms > 0 else None,
            "nvlink_peak_gbs": 900.0, "nvlink_measured_peer_copy_gbs": 770.0,
            "limiting_kernel": "pool_kernel (pooling + peer stores)" if pool_ms >= max(x[0] for x in allr)
                               else "classify + scan + scatter",
            "limiting_kernel_ms": round(max(pool_ms, max(x[0] for x in allr)), 4),
            "nvlink_frac_of_nominal_in_pool_kernel": (nv_bytes / (pool_ms / 1e3) / 1e9 / 900.0) if pool_ms > 0 else None,
            "note": "phase 'barrier1' also holds the pooling of the tables replicated whole (one-GPU kernel, no peer)",
        }

    roofline = None
    if hooks:
        bag_avg_ms = sum(bag_ms) / len(bag_ms)
        achieved = emb_bytes / (bag_avg_ms / 1e3) / 1e9
        traffic = NCU_BAG_TRAFFIC_BYTES.get((args.batch, float(args.max_rows), args.seed))
        roofline = {"bound": "hbm", "kernel": bag_kernel,
                    "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                    "peak_source": peak_source,
                    "label": "algorithmic GB/s (L2-assisted): algorithmic bytes per launch / kernel time; "
                             "Zipf-hot rows are served by L2, so DRAM moves less (dram_frac)",
                    "limited_by": "instruction issue and L2 / row-gather latency, not DRAM bandwidth",
                    "algorithmic_bytes_per_launch": emb_bytes, "lookups_per_launch": nnz,
                    "kernel_ms": bag_avg_ms, "traffic": traffic,
                    "traffic_source": "constant, not measured by this run: ncu dram__bytes_read.sum + "
                                      "dram__bytes_write.sum of the small case (batch 16384, rows <= 1e6) scaled "
                                      "by the lookups per launch" if traffic else None,
                    "dram_gbs": traffic / (bag_avg_ms / 1e3) / 1e9 if traffic else None,
                    "dram_frac": traffic / (bag_avg_ms / 1e3) / 1e9 / hbm_peak if traffic else None}
    else:
        roofline = {"bound": "hbm", "kernel": bag_kernel, "achieved": None, "peak": hbm_peak,
                    "unit": "GB/s", "frac": None, "traffic": None, "peak_source": peak_source,
                    "note": "the bag kernel is timed alone at N=1; the sharded step's pooling kernel also "
                            "stores over NVLink: its time and bytes are in `exchange`"}
        if exchange is not None:
            pool_ms = exchange["phase_ms_max_over_ranks"][2]
            roofline.update(kernel_ms=pool_ms, achieved=emb_bytes / (pool_ms / 1e3) / 1e9 if pool_ms else None,
                            frac=emb_bytes / (pool_ms / 1e3) / 1e9 / hbm_peak if pool_ms else None,
                            algorithmic_bytes_per_launch=emb_bytes,
                            label="algorithmic GB/s (L2-assisted) of the pooling + exchange kernel: one rank's "
                                  "lookups x (row + raw id + segment id) + one output row per bag")

    line = None
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None,
                "dtype": "tf32" if not recsys else "bf16", "data": "synthetic",
                "impl": "annc_b200", "config": workload_config(args, world),
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
                        # the end-to-end step is bound by the host-to-device copy of the ids and
                        # index matrices (the operands' own format): GB/s this rank's copies reach
                        "h2d_gbs": pipe.h2d_bytes / (ms_e2e / 1e3) / 1e9,
                        "host_cores_local_to_gpu": numa_cores},
                "ms_per_step_unpipelined": ms_alone,
                "pipelining": ("the timed steps are issued back to back in the order '%s' (chosen by five "
                               "calibration steps of each order): work of neighbouring steps overlaps on "
                               "second and third streams, two sets of intermediate buffers; "
                               "ms_per_step_unpipelined is one step with nothing overlapping it" % issue_order)
                              if issue_order != "none" else "none",
                "issue_orders_ms_per_step": order_ms,
                "gpu_launches": pipe.launches_per_step * args.steps,
                "gemm_kernels": sorted(set(pipe.kernel_names)),
                "roofline": roofline, "clocks": sampler.summary()}
        if exchange is not None:
            line["exchange"] = exchange

    pipe_out = pipe.out.float().cpu().numpy() if (world == 1 and not recsys) else None
    close(pipe)
    del pipe
    torch.cuda.empty_cache()

    # other partitionings, as labelled sub-records of the same line
    if world > 1 and not recsys and args.extras:
        extras = {}
        for mode in [m for m in args.extras.split(",") if m and m != args.shard]:
            if mode.startswith("row_k") and int(mode[5:]) == args.hot_rows:
                continue
            p2 = build(mode)
            for _ in range(3):
                p2.forward()
            torch.cuda.synchronize()
            assert p2.embed_error_bits() == 0
            ms2 = min(timed(p2.forward, args.steps),
                      timed(p2.forward_pipelined, args.steps, p2.sync_pipeline)) / args.steps
            if getattr(p2, "split_finish", False):
                p2.rowbags.ex.set_pool_ctas_per_sm(-1)
                split = lambda: p2.forward_pipelined(split=True)
                for _ in range(3):
                    split()
                ms2 = min(ms2, timed(split, args.steps, p2.sync_pipeline) / args.steps)
                p2.rowbags.ex.set_pool_ctas_per_sm(0)
            rec = {"value": args.batch * world / (ms2 / 1e3), "unit": UNIT, "ms_per_step": ms2,
                   "parallelism": parallelism_label(args, world, mode)}
            rb = getattr(p2, "rowbags", None)
            if rb is not None:
                st = rb.exchange_stats()
                rec["remote_parts_per_bag"] = st["remote_parts_per_bag"]
                rec["nvlink_bytes_per_gpu_per_step"] = st["nvlink_bytes"]
                rec["hot_bytes_per_gpu"] = st["hot_bytes"] + getattr(p2, "whole_bytes", 0)
            extras[mode] = rec
            close(p2)
            del p2
            torch.cuda.empty_cache()
        if rank == 0:
            line["extras"] = extras

    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and recsys:
            from oracle import oracle
            threads = oracle.host_threads()
            t = recsys_cpu_timed(args, threads, 2)
            cpu_ms = 1e3 * sum(t) / len(t)
            line["cpu_baseline"] = {"value": args.batch / (cpu_ms / 1e3), "unit": UNIT, "cores": threads,
                                    "kind": "port", "ms_per_step": cpu_ms,
                                    "sample": "1 of %d tables pooled (rows reduced to 1e6), time x %d / "
                                              "min(threads, tables); fp32 MLP on the full batch"
                                              % (args.tables, args.tables)}
        elif world == 1 and not args.no_cpu_baseline:
            base, one, parity = cpu_baselines(args, model, pipe_out)
            line["cpu_baseline"] = base
            line["cpu_baseline_1thread"] = one
            line["parity_max_abs_err"] = parity
            line["parity_note"] = ("max |p_gpu - p_cpu| over the %d predictions of the timed batch "
                                   "(TF32 tensor-core MLP against fp32 OpenBLAS; bound 2e-3)" % args.batch)
            assert parity <= 2e-3, "GPU predictions differ from the CPU reference path by %g" % parity
        if world == 1 and not recsys and not args.no_ops:
            from annc_b200 import opbench
            line["ops"] = opbench.ops_record()
        if world == 1 and not recsys and not args.no_abi:
            line["e2e_abi"] = abi_leg(args, model, pipe_out)
        print(json.dumps(line), flush=True)
    if recsys or world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()

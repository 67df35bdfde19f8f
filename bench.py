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

# DRAM bytes (read + write) of one bag-kernel launch, from a single-pass ncu capture of this
# command's default workload (profiles/bag_reduce_kernel_dlrm_batch65536_traffic_and_launch_list.md).
# Keyed by (batch, max_rows, seed); any other workload reports null.
NCU_BAG_TRAFFIC_BYTES = {(65536, 1e7, 0): 1.573e9}


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
    ap.add_argument("--shard", default="auto", choices=["auto", "row", "row_gather", "row_nccl", "table", "table_nccl", "replica"],
                    help="table partitioning for --gpus > 1: row = mod row-sharding, lookups split by "
                         "owner at their source, the bag kernel stores partial sums into the owner "
                         "rank's memory; row_gather = the same stores with all-gathered ids; row_nccl = "
                         "all-gathered ids and a separate NCCL all-to-all; table = whole tables per rank; replica = no exchange; auto = "
                         "row when the tables exceed --hbm-budget-gb per GPU, else replica")
    ap.add_argument("--hbm-budget-gb", type=float, default=100.0,
                    help="per-GPU memory the tables may take before auto switches to row sharding")
    args = ap.parse_args()
    if args.batch is None:
        args.batch = 65536 if args.workload == "dlrm" else 16384
    return args


def workload_config(args, world):
    if args.workload == "recsys":
        rows = int(args.rows_per_gpu) * world
        return {"workload": "recsys_%dtables_x_%drows_dim128_mean_pool_bf16_mlp_8192-1024-512-1_batch%d"
                            % (args.tables, rows, args.batch * world),
                "global_batch": args.batch * world, "per_gpu_batch": args.batch, "tables": args.tables,
                "dim": 128, "rows": rows, "bag": "U{1..50}, Zipf 1.2, mean",
                "table_bytes_total": args.tables * rows * 512,
                "parallelism": ("table-wise sharded tables over %d GPU(s), pooled vectors stored into the "
                                "sample owner's memory; dp MLP" % world) if args.shard == "table" else
                               ("row-sharded tables (mod rule) over %d GPU(s), lookups split at their "
                                "source, partial sums stored into the owner's memory; dp MLP" % world),
                "l2": "inputs larger than L2 (table shard %.1f GB per GPU)" % (args.tables * int(args.rows_per_gpu) * 512 / 1e9)}
    return {"workload": "dlrm_style_fp32w_tf32math_batch%d_26tables_dim64_zipf1.05" % args.batch,
            "global_batch": args.batch * world, "per_gpu_batch": args.batch,
            "tables": 26, "dim": 64, "rows": "log-uniform 1e3..%g" % args.max_rows,
            "parallelism": ("dp%d MLP + %s-sharded tables" % (world, args.shard)) if world > 1 else "single",
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

def run_gpu(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (annc_b200 has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    devi = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=devi)

    from annc_b200 import synth
    from annc_b200._lib import lib
    from annc_b200.dlrm import DlrmPipeline
    import ctypes as C

    if args.workload == "recsys":
        from annc_b200.recsys import RecsysPipeline
        if world == 1:  # the row-sharded step uses torch.distributed for its barriers at every N
            dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % (29000 + os.getpid() % 2000),
                                    rank=0, world_size=1, device_id=devi)
        args.shard = "table" if args.shard == "table" else "row"
        model = synth.recsys_model(seed=args.seed, tables=args.tables, rows=int(args.rows_per_gpu) * world,
                                   batch=args.batch, input_seed=1000 + rank)
        pipe = RecsysPipeline(model, devi, keep_host_inputs=True, shard=args.shard)
        nnz = model.nnz
        # the bag kernel of the partitioned step reads an int32 local row per lookup and two
        # int32 positions per bag, and writes one fp32 part per bag
        emb_bytes = nnz * (4 * 128 + 4) + args.tables * args.batch * (4 * 128 + 8)
        bag_kernel = "bag_reduce_kernel<32,1> (gather + segment sum of the partitioned step, %d tables)" % args.tables
        if args.shard == "table":  # whole bags: raw 8-byte ids hashed in the kernel, mean applied there
            emb_bytes = nnz * (4 * 128 + 8) + args.tables * args.batch * (4 * 128 + 8)
            bag_kernel = "bag_reduce_kernel<32,1> (hash-bucket + gather + segment mean, %d tables)" % args.tables
    else:
        model = synth.dlrm_model(seed=args.seed, batch=args.batch, max_rows=args.max_rows,
                                 input_seed=(1000 + rank) if world > 1 else None)
        if world > 1:
            from annc_b200.sharded import ShardedDlrmPipeline
            if args.shard == "auto":
                table_gb = sum(t.nbytes for t in model.emb.tables) / 1e9
                args.shard = "row" if table_gb > args.hbm_budget_gb else "replica"
            pipe = ShardedDlrmPipeline(model, devi, args.shard, keep_host_inputs=True)
        else:
            pipe = DlrmPipeline(model, devi, keep_host_inputs=True)
        emb_bytes = model.emb.algorithmic_bytes()
        nnz = model.emb.nnz
        bag_kernel = "bag_reduce_kernel<16,1> (hash-bucket + gather + segment sum, 26 tables in one launch)"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=devi)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(max(3, args.warmup)):
        pipe.forward()
    torch.cuda.synchronize()
    assert pipe.embed_error_bits() == 0, "embedding kernels flagged an index error"

    # device-resident pass: the whole step, and the bag kernel alone through event hooks
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    pairs = [(C.c_void_p(lib.annc_timer_create()), C.c_void_p(lib.annc_timer_create()))
             for _ in range(args.steps)]
    it = iter(pairs)

    def step_with_hooks():
        a, b = next(it)
        lib.annc_embed_bag_set_timing_events(a, b)
        pipe.forward()

    ms_total = timed(step_with_hooks, args.steps)
    lib.annc_embed_bag_set_timing_events(None, None)
    bag_ms = []
    for a, b in pairs:
        v = C.c_float(0)
        lib.annc_timer_elapsed_ms(a, b, C.byref(v))
        bag_ms.append(v.value)
        lib.annc_timer_destroy(a)
        lib.annc_timer_destroy(b)
    ms_step = ms_total / args.steps

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
    bag_avg_ms = sum(bag_ms) / len(bag_ms)
    achieved = emb_bytes / (bag_avg_ms / 1e3) / 1e9
    roofline = {"bound": "hbm", "kernel": bag_kernel,
                "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                "peak_source": "measured" if "hbm_gbs" in peaks else "fallback",
                "algorithmic_bytes_per_launch": emb_bytes, "lookups_per_launch": nnz,
                "kernel_ms": bag_avg_ms,
                "traffic": NCU_BAG_TRAFFIC_BYTES.get((args.batch, float(args.max_rows), args.seed))
                if args.workload == "dlrm" else None,
                "traffic_note": "dram read+write bytes per launch from ncu; below the algorithmic "
                                "bytes because Zipf-hot rows are served by L2"}

    if world > 1:
        roofline = {"bound": "hbm", "kernel": roofline["kernel"], "achieved": None, "peak": hbm_peak,
                    "unit": "GB/s", "frac": None, "traffic": None,
                    "note": "the bag kernel is timed alone at N=1; a sharded step launches it in "
                            "several groups and its bytes per launch depend on the partitioning"}
    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None,
                "dtype": "tf32" if args.workload == "dlrm" else "bf16", "data": "synthetic",
                "impl": "annc_b200", "config": workload_config(args, world),
                "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": pipe.h2d_bytes, "d2h_bytes_per_step": pipe.d2h_bytes,
                        # the end-to-end step is bound by the host-to-device copy of the ids and
                        # index matrices (the operands' own format): GB/s this rank's copies reach
                        "h2d_gbs": pipe.h2d_bytes / (ms_e2e / 1e3) / 1e9},
                "gpu_launches": pipe.launches_per_step * args.steps,
                "gemm_kernels": sorted(set(pipe.kernel_names)),
                "roofline": roofline, "clocks": sampler.summary()}
        if world == 1 and not args.no_cpu_baseline and args.workload == "recsys":
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
            from oracle import oracle
            threads = oracle.host_threads()
            t = cpu_forward_timed(model, threads, 3)
            cpu_ms = 1e3 * sum(t) / len(t)
            line["cpu_baseline"] = {"value": args.batch / (cpu_ms / 1e3), "unit": UNIT, "cores": threads,
                                    "kind": "port", "ms_per_step": cpu_ms,
                                    "sample": "3 full batches of %d samples (C restatement of the "
                                              "reference kernels, one table per thread, + OpenBLAS sgemm)"
                                              % args.batch}
        print(json.dumps(line), flush=True)
    if args.workload == "recsys":
        pipe.close()
        dist.destroy_process_group()
    elif world > 1:
        if hasattr(pipe, "peer"):
            torch.cuda.synchronize()
            pipe.peer.close()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()

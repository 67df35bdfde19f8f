"""Per-operator timing on one GPU: GEMM TFLOP/s against the tensor peak and bandwidth
kernels against the HBM peak, for the benchmark configurations and the DLRM layers.

    python -m annc_b200.opbench [--only gemm|embed|misc] [--reps 20]

CUDA events on the launching stream, 3 warm-ups, a 256 MB L2 flush between repetitions
for working sets smaller than L2.  Prints one JSON line per case."""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import device as dev
from . import synth
from ._lib import (ACT_NONE, ACT_RELU, B_KN4, B_PLAIN, IO_A_BF16, IO_B_BF16, IO_C_BF16, IO_SOFTMAX,
                   MATH_AUTO, MATH_BF16)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def peaks():
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]) / 2, "measured"
    except Exception:
        return 6650.0, 1590.0 / 2, "fallback"


_flush = None
_nvml = None


def sm_clock_mhz():
    """Current SM clock (read only), reported beside each timing: the tensor-core cases move
    with the clock the power cap allows."""
    global _nvml
    try:
        if _nvml is None:
            import pynvml
            pynvml.nvmlInit()
            _nvml = (pynvml, pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device()))
        return int(_nvml[0].nvmlDeviceGetClockInfo(_nvml[1], _nvml[0].NVML_CLOCK_SM))
    except Exception:
        return None


def time_ms(fn, reps, flush):
    global _flush
    if flush and _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush:
            _flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1))
    global LAST_CLOCK
    LAST_CLOCK = sm_clock_mhz()
    return float(np.median(ts))


LAST_CLOCK = None


def bmm_case(name, b, m, n, k, reps):
    if MATCH and MATCH not in f"{name}/kn":
        return
    hbm, tf32, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((b, m, k), device="cuda", generator=g)
    w = torch.randn((b, k, n), device="cuda", generator=g)
    c = torch.empty((b, m, n), device="cuda")
    names = []
    fn = lambda: names.append(dev.gemm(a, w, c, m=m, n=n, k=k, batch=b, stride_a=m * k,
                                       stride_b=k * n, stride_c=m * n))
    byt = 4 * b * (m * k + k * n + m * n)
    ms = time_ms(fn, reps, flush=True)
    fl = 2.0 * b * m * n * k
    print(json.dumps({"op": name, "kernel": names[-1], "b": "kn", "m": m, "n": n, "k": k, "batch": b,
                      "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                      "frac_tf32_peak": round(fl / ms / 1e9 / tf32, 3),
                      "gbs": round(byt / ms / 1e6, 1), "frac_hbm": round(byt / ms / 1e6 / hbm, 3),
                      "peak": src, "sm_mhz": LAST_CLOCK}), flush=True)


MATCH = ""


def bf16_case(name, m, n, k, reps):
    """bf16 A [M,K] x bf16 B [N,K] -> bf16 C with bias + ReLU (the large recsys MLP layers)."""
    if MATCH and MATCH not in f"{name}/bf16":
        return
    hbm, tf32, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), device="cuda", generator=g).to(torch.bfloat16)
    b = (torch.randn((n, k), device="cuda", generator=g) / k ** 0.5).to(torch.bfloat16)
    bv = torch.randn(n, device="cuda", generator=g)
    c = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    names = []
    fn = lambda: names.append(dev.gemm(a, b, c, m=m, n=n, k=k, trans_b=True, bias=bv, activation=ACT_RELU,
                                       math=MATH_BF16, io_flags=IO_A_BF16 | IO_B_BF16 | IO_C_BF16))
    byt = 2 * (m * k + k * n + m * n)
    ms = time_ms(fn, reps, flush=byt < (200 << 20))
    fl = 2.0 * m * n * k
    print(json.dumps({"op": name, "kernel": names[-1], "b": "nk bf16", "m": m, "n": n, "k": k,
                      "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                      "frac_bf16_peak": round(fl / ms / 1e9 / (2 * tf32), 3),
                      "gbs": round(byt / ms / 1e6, 1), "frac_hbm": round(byt / ms / 1e6 / hbm, 3),
                      "peak": src, "sm_mhz": LAST_CLOCK}), flush=True)


def bmm_softmax_case(name, b, m, n, k, reps):
    """batch_matmul + row softmax: two kernels (matmul, then softmax) against the fused epilogue."""
    if MATCH and MATCH not in f"{name}/kn":
        return
    hbm, _, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((b, m, k), device="cuda", generator=g) / 8
    w = torch.randn((b, k, n), device="cuda", generator=g)
    c = torch.empty((b, m, n), device="cuda")
    y = torch.empty((b, m, n), device="cuda")
    kw = dict(m=m, n=n, k=k, batch=b, stride_a=m * k, stride_b=k * n, stride_c=m * n)

    def two():
        dev.gemm(a, w, c, **kw)
        dev.softmax(c.view(-1, n), y.view(-1, n))
    ms2 = time_ms(two, reps, flush=True)
    ms1 = time_ms(lambda: dev.gemm(a, w, y, io_flags=IO_SOFTMAX, **kw), reps, flush=True)
    byt = 4 * b * (m * k + k * n + m * n)
    print(json.dumps({"op": name, "two_kernels_ms": round(ms2, 4), "fused_ms": round(ms1, 4),
                      "fused_gbs": round(byt / ms1 / 1e6, 1), "fused_frac_hbm": round(byt / ms1 / 1e6 / hbm, 3),
                      "peak": src, "sm_mhz": LAST_CLOCK}), flush=True)


def gemm_case(name, m, n, k, reps, bsrc="kn", bias=False, act=ACT_NONE, addend=False):
    if MATCH and MATCH not in f"{name}/{bsrc}":
        return
    hbm, tf32, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), device="cuda", generator=g)
    w = torch.randn((k, n), device="cuda", generator=g)
    c = torch.empty((m, n), device="cuda")
    bv = torch.randn(n, device="cuda", generator=g) if bias else None
    ad = torch.randn((m, n), device="cuda", generator=g) if addend else None
    kw = dict(m=m, n=n, k=k, bias=bv, addend=ad, activation=act, math=MATH_AUTO)
    if bsrc == "nk":
        b = w.t().contiguous()
        kw["trans_b"] = True
    elif bsrc in ("kn4", "kn4+ws"):
        b = dev.kn4_pack(w)
        kw["b_format"] = B_KN4
        if bsrc == "kn4+ws":
            kw["workspace"] = torch.empty((k, n), device="cuda")
    else:
        b = w
    names = []
    fn = lambda: names.append(dev.gemm(a, b, c, **kw))
    byt = 4 * (m * k + k * n + m * n * (2 if addend else 1))
    ms = time_ms(fn, reps, flush=byt < (200 << 20))
    fl = 2.0 * m * n * k
    print(json.dumps({"op": name, "kernel": names[-1], "b": bsrc, "m": m, "n": n, "k": k,
                      "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
                      "frac_tf32_peak": round(fl / ms / 1e9 / tf32, 3),
                      "gbs": round(byt / ms / 1e6, 1), "frac_hbm": round(byt / ms / 1e6 / hbm, 3),
                      "peak": src, "sm_mhz": LAST_CLOCK}), flush=True)


def run_gemm(reps):
    gemm_case("matmul_add_relu C1", 512, 1024, 1024, reps, addend=True, act=ACT_RELU)
    for bsrc in ("kn4", "kn4+ws", "kn", "nk"):
        gemm_case("layout_matmul C2", 8192, 4096, 2048, reps, bsrc=bsrc)
    bmm_case("batch_matmul C2", 64, 256, 256, 64, reps)
    bmm_softmax_case("batch_matmul + softmax C2", 64, 256, 256, 64, reps)
    for (m, n, k) in ((16384, 1024, 8192), (131072, 1024, 8192), (131072, 512, 1024), (8192, 8192, 8192)):
        bf16_case("recsys MLP bf16", m, n, k, reps)
    gemm_case("square tf32", 8192, 8192, 8192, reps, bsrc="nk")
    for m in (128, 256, 512):
        gemm_case("small-M sweep", m, 1024, 1024, reps)
    for (k, n) in ((512, 256), (256, 64), (416, 512), (512, 256)):
        for bsrc in ("kn", "nk"):
            gemm_case("dlrm layer", 65536, n, k, reps, bsrc=bsrc, bias=True, act=ACT_RELU)
    gemm_case("dlrm layer0 (K=13)", 65536, 512, 13, reps, bias=True, act=ACT_RELU)


def run_embed(reps):
    hbm, _, src = peaks()
    w = synth.hash_bucket_bag_case(0)
    up = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    out = torch.empty((w.batch, len(w.tables), w.dim), device="cuda")
    plan = dev.BagPlan([up(t) for t in w.tables], [up(b.raw_ids) for b in w.bags],
                       [up(b.slice_input) for b in w.bags], out, 0, w.batch)
    ms = time_ms(plan.run, reps, flush=False)
    byt = w.algorithmic_bytes()
    print(json.dumps({"op": "embed_hash_bucket + segment sum C3 (prepass + bags)", "ms": round(ms, 4),
                      "lookups": w.nnz, "gbs": round(byt / ms / 1e6, 1),
                      "frac_hbm": round(byt / ms / 1e6 / hbm, 3),
                      "samples_per_s": round(w.batch / ms * 1e3), "peak": src, "sm_mhz": LAST_CLOCK}), flush=True)


def run_misc(reps):
    hbm, _, src = peaks()
    x = torch.randn((16384, 256), device="cuda")
    y = torch.empty_like(x)
    ms = time_ms(lambda: dev.softmax(x, y), reps, flush=True)
    print(json.dumps({"op": "softmax 16384x256", "ms": round(ms, 4),
                      "gbs": round(2 * x.numel() * 4 / ms / 1e6, 1)}), flush=True)
    z = torch.randn((65536, 27, 64), device="cuda")
    o = torch.empty((65536, 416), device="cuda")
    ms = time_ms(lambda: dev.dot_interaction(z, o), reps, flush=False)
    byt = (z.numel() + o.numel()) * 4
    print(json.dumps({"op": "dot interaction 65536x27x64", "ms": round(ms, 4),
                      "gbs": round(byt / ms / 1e6, 1), "frac_hbm": round(byt / ms / 1e6 / hbm, 3)}),
          flush=True)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="all")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--match", default="", help="run only GEMM cases whose 'name/b-source' contains this")
    a = ap.parse_args()
    MATCH = a.match
    if a.only in ("all", "gemm"):
        run_gemm(a.reps)
    if a.only in ("all", "embed"):
        run_embed(a.reps)
    if a.only in ("all", "misc"):
        run_misc(a.reps)

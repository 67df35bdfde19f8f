"""Per-operator timings on one GPU for the benchmark configurations: GEMM TFLOP/s against the
tensor peak and bandwidth kernels against the HBM peak.  `ops_record()` is what `bench.py` puts
into its JSON line; `python -m annc_b200.opbench` prints the same record, one case per line.

CUDA events on the launching stream, 3 warm-ups, median of `reps`; a 256 MB buffer is written
between repetitions when the working set is smaller than L2."""
from __future__ import annotations

import json
import os

import numpy as np
import torch

from . import device as dev
from . import synth
from ._lib import ACT_NONE, ACT_RELU, B_KN4, IO_SOFTMAX, MATH_AUTO

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_flush = None


def peaks():
    """(HBM GB/s, TF32 TFLOP/s, source).  TF32 dense peak = half the measured BF16 figure."""
    try:
        p = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]) / 2, "measured"
    except Exception:
        return 6650.0, 1590.0 / 2, "fallback"


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
    return float(np.median(ts))


def _gemm_fields(ms, m, n, k, byt, batch=1):
    hbm, tf32, src = peaks()
    fl = 2.0 * batch * m * n * k
    return {"m": m, "n": n, "k": k, "ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1),
            "frac_tf32_peak": round(fl / ms / 1e9 / tf32, 3), "gbs": round(byt / ms / 1e6, 1),
            "frac_hbm": round(byt / ms / 1e6 / hbm, 3), "peak": src}


def gemm_case(m, n, k, reps, bsrc="kn", bias=False, act=ACT_NONE, addend=False, b_cached=None):
    """bsrc: "kn" (B as [K,N]), "nk" (B as [N,K]), "kn4" (the prepacked layout, consumed
    directly), "kn4+ws" (prepacked, re-laid into a caller workspace on every call)."""
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), device="cuda", generator=g)
    w = torch.randn((k, n), device="cuda", generator=g) if b_cached is None else None
    c = torch.empty((m, n), device="cuda")
    bv = torch.randn(n, device="cuda", generator=g) if bias else None
    ad = torch.randn((m, n), device="cuda", generator=g) if addend else None
    kw = dict(m=m, n=n, k=k, bias=bv, addend=ad, activation=act, math=MATH_AUTO)
    if b_cached is not None:
        b = b_cached
        kw["b_format"] = B_KN4
    elif bsrc == "nk":
        b = w.t().contiguous()
        kw["trans_b"] = True
    elif bsrc in ("kn4", "kn4+ws"):
        b = dev.kn4_pack(w)
        kw["b_format"] = B_KN4
    else:
        b = w
    if bsrc == "kn4+ws":
        kw["workspace"] = torch.empty((k, n), device="cuda")
    names = []
    fn = lambda: names.append(dev.gemm(a, b, c, **kw))
    byt = 4 * (m * k + k * n + m * n * (2 if addend else 1))
    ms = time_ms(fn, reps, flush=byt < (200 << 20))
    r = _gemm_fields(ms, m, n, k, byt)
    r.update(kernel=names[-1], b=bsrc)
    return r


def layout_matmul_call_case(m, packed_host, k, n, reps):
    """__layout_matmul through the custom-call entry point with the packed weight in HOST memory
    (as XLA holds a constant) and device activations: the library mirrors the weight on first
    sight and keeps its re-laid form with the mirror, so a timed call uploads and re-lays
    nothing."""
    from . import ops
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), device="cuda", generator=g)
    c = torch.empty((m, n), device="cuda")
    operands = [a, packed_host, ops.shape_info(a), ops.shape_info(packed_host)]
    fn = lambda: ops._call_custom("__layout_matmul", c, operands)
    byt = 4 * (m * k + k * n + m * n)
    ms = time_ms(fn, reps, flush=byt < (200 << 20))
    r = _gemm_fields(ms, m, n, k, byt)
    r.update(b="kn4 host constant, re-laid once and kept with its mirror", entry="__layout_matmul")
    return r


def bmm_softmax_case(b, m, n, k, reps):
    """batch_matmul + row softmax: two kernels (matmul, then softmax) and the fused epilogue."""
    hbm, _, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((b, m, k), device="cuda", generator=g) / 8
    w = torch.randn((b, k, n), device="cuda", generator=g) / 8
    c = torch.empty((b, m, n), device="cuda")
    y = torch.empty((b, m, n), device="cuda")
    kw = dict(m=m, n=n, k=k, batch=b, stride_a=m * k, stride_b=k * n, stride_c=m * n)
    names = []
    ms_mm = time_ms(lambda: names.append(dev.gemm(a, w, c, **kw)), reps, flush=True)
    ms_sm = time_ms(lambda: dev.softmax(c.view(-1, n), y.view(-1, n)), reps, flush=True)
    ms_f = time_ms(lambda: dev.gemm(a, w, y, io_flags=IO_SOFTMAX, **kw), reps, flush=True)
    byt_mm = 4 * b * (m * k + k * n + m * n)
    byt_sm = 2 * 4 * b * m * n
    return {"batch_matmul": dict(_gemm_fields(ms_mm, m, n, k, byt_mm, batch=b), kernel=names[-1], batch=b),
            "softmax": {"rows": b * m, "channels": n, "ms": round(ms_sm, 4),
                        "gbs": round(byt_sm / ms_sm / 1e6, 1), "frac_hbm": round(byt_sm / ms_sm / 1e6 / hbm, 3)},
            "fused_bmm_softmax": {"ms": round(ms_f, 4), "gbs": round(byt_mm / ms_f / 1e6, 1),
                                  "frac_hbm": round(byt_mm / ms_f / 1e6 / hbm, 3),
                                  "note": "one kernel; not routed to by default while two kernels are faster"},
            "peak": src}


def embed_case(reps, tables=26, rows=1_000_000, dim=64, batch=16384):
    """26 tables x 1 M rows x dim 64, batch 16384, bags U{1..20}, Zipf 1.05 ids, sum pooling:
    prepass + grouped bag kernel.  Tables are drawn on the device (U(-0.05, 0.05)); the ids come
    from the host generator."""
    hbm, _, src = peaks()
    g = torch.Generator(device="cuda").manual_seed(0)
    tabs = [torch.rand((rows, dim), device="cuda", generator=g) * 0.1 - 0.05 for _ in range(tables)]
    rngs = np.random.default_rng(0).spawn(tables)
    bags = [synth._bag_inputs(r, batch, 20, 1.05) for r in rngs]
    up = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    out = torch.empty((batch, tables, dim), device="cuda")
    plan = dev.BagPlan(tabs, [up(b.raw_ids) for b in bags], [up(b.slice_input) for b in bags], out, 0, batch)
    ms = time_ms(plan.run, reps, flush=False)
    assert plan.error_bits() == 0
    nnz = int(sum(b.raw_ids.shape[0] for b in bags))
    byt = nnz * (4 * dim + 16) + tables * batch * 4 * dim
    return {"tables": tables, "rows": rows, "dim": dim, "batch": batch, "lookups": nnz, "ms": round(ms, 4),
            "algorithmic_gbs": round(byt / ms / 1e6, 1), "frac_hbm_algorithmic": round(byt / ms / 1e6 / hbm, 3),
            "label": "algorithmic GB/s of prepass + bag kernel (L2-assisted: Zipf-hot rows are served by "
                     "L2, DRAM traffic is lower)", "samples_per_s": round(batch / ms * 1e3), "peak": src,
            "l2": "6.6 GB of tables, larger than L2; no flush"}


def ops_record(reps: int = 10) -> dict:
    """The operator figures of the benchmark configurations (one GPU, device-resident operands)."""
    rec = {"method": "CUDA events, median of %d, 3 warm-ups; L2 flushed between repetitions when the "
                     "working set is below 200 MB" % reps}
    rec["c1_matmul_add_relu_512x1024x1024"] = gemm_case(512, 1024, 1024, reps, addend=True, act=ACT_RELU)
    g = torch.Generator(device="cuda").manual_seed(1)
    w = torch.randn((2048, 4096), device="cuda", generator=g) / 64
    packed = dev.kn4_pack(w)
    del w
    rec["c2_layout_matmul_8192x4096x2048_from_kn4_direct"] = gemm_case(8192, 4096, 2048, reps, bsrc="kn4", b_cached=packed)
    rec["c2_layout_matmul_8192x4096x2048_from_kn4_relaid_each_call"] = gemm_case(8192, 4096, 2048, reps, bsrc="kn4+ws", b_cached=packed)
    rec["c2_layout_matmul_8192x4096x2048_b_as_nk"] = gemm_case(8192, 4096, 2048, reps, bsrc="nk")
    packed_host = packed.cpu().numpy()
    rec["c2_layout_matmul_8192x4096x2048_custom_call_cached_weight"] = layout_matmul_call_case(
        8192, packed_host, 2048, 4096, reps)
    rec["small_m_sweep_layout_matmul_custom_call_cached_weight"] = {
        "M=%d" % m: layout_matmul_call_case(m, packed_host, 2048, 4096, reps) for m in (128, 256, 512)}
    rec["small_m_sweep_layout_matmul_kn4_n4096_k2048"] = {
        "M=%d" % m: gemm_case(m, 4096, 2048, reps, bsrc="kn4", b_cached=packed) for m in (128, 256, 512)}
    rec["c2_batch_matmul_softmax_64x256x64x256"] = bmm_softmax_case(64, 256, 256, 64, reps)
    torch.cuda.empty_cache()
    rec["c3_embed_hash_bucket_segment_sum"] = embed_case(reps)
    torch.cuda.empty_cache()
    return rec


if __name__ == "__main__":
    for name, val in ops_record().items():
        print(json.dumps({name: val}), flush=True)

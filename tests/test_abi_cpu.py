"""CPU-only checks of the drop-in boundary: the shared library loads, exports every
symbol the header declares (and the C++-mangled aliases), the ANNC_FLAGS parser
agrees with the reference's own parser, and host-side validation reproduces the
reference's messages without touching a GPU."""
import ctypes as C
import os
import re
import subprocess

import numpy as np
import pytest

from oracle import oracle
from tests import test_oracle_golden as tog

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "annc_b200.h")


@pytest.fixture(scope="module")
def annc():
    import annc_b200
    return annc_b200


def declared_symbols():
    src = open(HEADER).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = set(re.findall(r"\b(annc_[A-Za-z0-9_]+)\s*\(", src))
    names -= {"annc_alloc_fn"}
    names |= {"__matmul", "__layout_matmul", "__batch_matmul", "__matmul_add", "__matmul_add_relu",
              "__reduce_mean", "__pooling", "__xla_cpu_runtime_XnnPackSoftMaxND"}
    for v in ("Sequential", "Parallel", "MLIR", "Empty"):
        names |= {f"__xla_cpu_runtime_KernelSelectorGEMM{v}", f"__xla_cpu_runtime_KernelSelectorBatch3D{v}",
                  f"__xla_cpu_runtime_KernelSelectorBatch4D{v}"}
    names |= {"__xla_cpu_runtime_KernelSelectorGEMV", "__xla_cpu_runtime_KernelSelectorGEMVMLIR",
              "__xla_cpu_runtime_KernelSelectorGEMVEmpty", "__xla_cpu_runtime_ArgMax3DParallel",
              "__xla_cpu_runtime_ArgMax3DSequential", "__xla_cpu_runtime_ArgMax3DEmpty"}
    return names


def test_library_exports_every_declared_symbol(annc):
    names = declared_symbols()
    assert len(names) > 50
    for n in sorted(names):
        assert hasattr(annc.lib, n), f"missing export {n}"


def test_header_is_plain_c():
    """The boundary is a C ABI: the header must compile as C99 as well as C++ (a cgo / JNI / ctypes
    binding generator reads it as C)."""
    for cc, std, lang in (("gcc", "-std=c99", "c"), ("g++", "-std=c++17", "c++")):
        r = subprocess.run([cc, std, "-fsyntax-only", "-Wall", "-x", lang, HEADER], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr


def test_mangled_aliases_exported(annc):
    out = subprocess.run(["nm", "-D", "--defined-only", annc._lib.LIB_PATH], capture_output=True, text=True).stdout
    # names the reference's MLIR lowering calls (install/xla/matmul_lower.patch:65-68)
    assert "_ZN3xla3cpu8__matmulEPvPPKv" in out
    assert "_ZN3xla3cpu14__batch_matmulEPvPPKv" in out
    assert "_ZN3xla3cpu46__xla_cpu_runtime_KernelSelectorGEMMSequentialEPKvbbPKfS4_iiiffPf" in out


def test_flags_defaults_and_groups(annc):
    f = lambda s, n: bool(annc.lib.annc_flags_is_enabled_in(None if s is None else s.encode(), n.encode()))
    assert f(None, "annc-pass") and not f(None, "matmul")
    assert f("--gemm-opt", "matmul") and f("--gemm-opt", "layout-matmul") and f("--gemm-opt", "disable-tf-matmul-fusion")
    assert not f("--gemm-opt", "batch-matmul")
    assert f("--graph-opt", "sps-emd-2") and not f("--graph-opt", "pooling")
    assert f("--matmul=", "matmul") and f("--matmul=1", "matmul") and not f("--matmul=0", "matmul")
    assert f("--nonsense", "nonsense")  # unknown flags are reported and still stored


@pytest.mark.skipif(not oracle.flags_ref_available(), reason="reference flag parser not compiled here")
def test_flags_match_reference_parser(annc):
    for s in tog.FLAG_STRINGS:
        for n in tog.FLAG_NAMES:
            ours = bool(annc.lib.annc_flags_is_enabled_in(None if s is None else s.encode(), n.encode()))
            assert ours == oracle.flag_enabled_ref(s, n), (s, n)


def test_registry_follows_annc_pass(annc):
    # ANNC_FLAGS is unset in the test process: annc-pass defaults to on, op flags to off.
    for t in ("__matmul", "__batch_matmul", "__matmul_add", "__matmul_add_relu", "__reduce_mean",
              "__pooling", "__layout_matmul"):
        assert annc.lib.annc_lookup_custom_call(t.encode())
    assert not annc.lib.annc_lookup_custom_call(b"__nope")
    assert annc.lib.annc_select_gemm_target(2, 0) is None  # no op flag set


def test_registry_under_flags_subprocess():
    code = ("import annc_b200 as a; l=a.lib; "
            "print(l.annc_select_gemm_target(2,0), l.annc_select_gemm_target(1,0), "
            "l.annc_select_gemm_target(0,1), l.annc_select_gemm_target(0,0), l.annc_select_gemm_target(3,0))")
    env = dict(os.environ, ANNC_FLAGS="--gemm-opt --matmul-add-relu", PYTHONPATH=ROOT)
    out = subprocess.run(["python", "-c", code], capture_output=True, text=True, env=env, cwd=ROOT).stdout
    assert out.split()[-5:] == ["b'__matmul_add_relu'", "b'__matmul'", "b'__layout_matmul'", "b'__matmul'", "None"]
    env = dict(os.environ, ANNC_FLAGS="--annc-pass=0 --gemm-opt", PYTHONPATH=ROOT)
    code2 = "import annc_b200 as a; print(a.lib.annc_lookup_custom_call(b'__matmul'))"
    out = subprocess.run(["python", "-c", code2], capture_output=True, text=True, env=env, cwd=ROOT).stdout
    assert out.split()[-1] == "None"


def test_validation_messages_without_gpu(annc):
    """Shape checks run before any CUDA call, with the reference's OP_REQUIRES text."""
    from annc_b200 import AnncError, ops
    from tests.golden import reference_cases as rc
    for field, value, msg in rc.SEGMENT_REDUCE_ERRORS:
        if field in ("data", "slice_input") or "must have" in msg:
            base = dict(rc.SEGMENT_REDUCE[1])
            base[field] = value
            with pytest.raises(AnncError) as e:
                ops.kp_fused_sparse_segment_reduce(base["data"], base["indices"], base["slice_input"],
                                                   base["begin"], base["begin_1"], 0)
            assert msg in e.value.message
    for ls, rs, bs, msg in rc.BMM_ADD_SIGMOID_ERRORS:
        with pytest.raises(AnncError) as e:
            ops.kp_fused_batch_matmul_add_sigmoid(np.zeros(ls, np.float32), np.zeros(rs, np.float32),
                                                  np.zeros(bs, np.float32))
        assert msg in e.value.message


def test_kn4_offset_host_matches_oracle(annc):
    for K, N in [(12, 12), (13, 17), (353, 129), (705, 257), (400, 140), (24, 300), (1000, 1000)]:
        offs = oracle.kn4_offsets(K, N)
        rng = np.random.default_rng(K)
        for k, n in zip(rng.integers(0, K, 300), rng.integers(0, N, 300)):
            assert annc.lib.annc_kn4_offset(K, N, int(k), int(n)) == offs[k, n]
        # the map is a permutation
        assert np.array_equal(np.sort(offs.reshape(-1)), np.arange(K * N))


def test_no_gpu_means_loud_failure(annc):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from annc_b200 import AnncError, ops
    with pytest.raises(AnncError) as e:
        ops.kp_fused_sparse_dynamic_stitch(np.array([0, 1], np.int64),
                                           [np.ones((2, 2), np.float32), np.ones((2, 2), np.float32)])
    assert e.value.code == 100  # ANNC_ERR_CUDA: no fallback


# ---------------------------------------------------------------- KERNEL_MAP_FILE

KMAP_SAMPLE = "(6656,8,8) -> __xla_cpu_runtime_KernelSelectorGEMM\n"  # the reference's own gemm_map.txt line: no [kernel], rejected


def _kmap_lookup(annc, kernel, sizes):
    import ctypes as C
    annc.lib.annc_kernel_map_lookup.restype = C.c_char_p
    arr = (C.c_int * len(sizes))(*sizes)
    r = annc.lib.annc_kernel_map_lookup(kernel.encode(), arr, len(sizes))
    return r.decode() if r else None


def test_kernel_map_matches_reference_rules(annc, tmp_path):
    import ctypes as C
    text = ("[gemm](6656, 8, 8) -> __xla_cpu_runtime_KernelSelectorGEMMSequential\r\n"
            "[gemm](128:512, 1024, 416:*) -> __xla_cpu_runtime_KernelSelectorGEMMParallel\n"
            "[gemv](*) -> __xla_cpu_runtime_KernelSelectorGEMV\n"
            "[batch3d](512,26,4,4:26) -> __xla_cpu_runtime_KernelSelectorBatch3DMLIR\n"
            "[batch3d](1,2,3) -> wrong_rank\n"
            "[argmax] (1:*, *, 5) -> __xla_cpu_runtime_ArgMax3DParallel\n"
            "gemm(1,2,3) -> no_brackets\n"
            "[gemm](99999999999,1,1) -> overflow\n"
            + KMAP_SAMPLE +
            "[conv](1,2) -> unknown_kernel_stops_the_load\n"
            "[gemm](1,1,1) -> never_read\n")
    want, want_bad = oracle.kernel_map_parse(text)
    bad = C.c_int(-1)
    assert annc.lib.annc_kernel_map_load_text(text.encode(), C.byref(bad)) == 0
    assert bad.value == want_bad == 5
    assert annc.lib.annc_kernel_map_size() == len(want) == 5
    probes = [("gemm", [6656, 8, 8]), ("gemm", [128, 1024, 416]), ("gemm", [512, 1024, 9999]),
              ("gemm", [513, 1024, 416]), ("gemm", [1, 1, 1]), ("gemv", [7, 12345]), ("gemv", [7]),
              ("batch3d", [512, 26, 4, 4]), ("batch3d", [512, 26, 4, 27]), ("batch3d", [1, 2, 3]),
              ("argmax", [1, 0, 5]), ("argmax", [0, 0, 5]), ("batch4d", [1, 1, 1, 1, 1]), ("conv", [1, 2])]
    for kernel, sizes in probes:
        assert _kmap_lookup(annc, kernel, sizes) == oracle.kernel_map_lookup(want, kernel, sizes), (kernel, sizes)
    assert _kmap_lookup(annc, "gemm", [6656, 8, 8]) == "__xla_cpu_runtime_KernelSelectorGEMMSequential"
    # from a file, through the environment variable's rule, and the fallback-first order of the
    # reference's map: a `(*)` entry sorts before every specific entry and shadows it
    f = tmp_path / "map.txt"
    f.write_text("[gemm](6656,8,8) -> specific\n[gemm](*) -> fallback\n")
    assert annc.lib.annc_kernel_map_load(str(f).encode(), None) == 0
    w2, _ = oracle.kernel_map_parse(f.read_text())
    assert _kmap_lookup(annc, "gemm", [6656, 8, 8]) == oracle.kernel_map_lookup(w2, "gemm", [6656, 8, 8]) == "fallback"
    assert annc.lib.annc_kernel_map_load(b"/nonexistent/map", None) != 0
    assert annc.lib.annc_kernel_map_size() == 2  # an unreadable file leaves the table as it was
    annc.lib.annc_kernel_map_clear()


def test_kernel_map_resolves_library_symbols(annc):
    import ctypes as C
    annc.lib.annc_kernel_map_resolve.restype = C.c_void_p
    annc.lib.annc_kernel_map_load_text(b"[gemm](*) -> __xla_cpu_runtime_KernelSelectorGEMMSequential\n"
                                       b"[gemv](*) -> not_a_symbol_of_this_library\n", None)
    arr = (C.c_int * 3)(128, 256, 512)
    addr = annc.lib.annc_kernel_map_resolve(b"gemm", arr, 3)
    direct = C.cast(annc.lib.__xla_cpu_runtime_KernelSelectorGEMMSequential, C.c_void_p).value
    assert addr == direct
    arr2 = (C.c_int * 2)(1, 2)
    assert annc.lib.annc_kernel_map_resolve(b"gemv", arr2, 2) is None
    annc.lib.annc_kernel_map_clear()

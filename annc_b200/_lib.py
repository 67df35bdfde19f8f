"""ctypes binding of libannc_b200.so.  There is no fallback: if the library has not
been built the import of the package fails, and every compute call fails with
ANNC_ERR_CUDA on a machine without a CUDA device."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libannc_b200.so")

ANNC_F32, ANNC_I32, ANNC_I64, ANNC_BOOL, ANNC_U64 = 1, 3, 9, 10, 23
ACT_NONE, ACT_RELU, ACT_SIGMOID = 0, 1, 2
B_PLAIN, B_KN4 = 0, 1
MATH_AUTO, MATH_FP32, MATH_TF32, MATH_BF16 = 0, 1, 2, 3
IO_A_BF16, IO_B_BF16, IO_C_BF16, IO_SOFTMAX, IO_PAIR = 1, 2, 4, 8, 16


class AnncError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[annc {code}] {message}")
        self.code = code
        self.message = message


class Tensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int32), ("rank", C.c_int32),
                ("dims", C.c_int64 * 4)]


class BagTable(C.Structure):
    _fields_ = [("table", C.c_void_p), ("rows", C.c_int64), ("num_buckets", C.c_int64),
                ("ids", C.c_void_p), ("slice_input", C.c_void_p), ("nnz", C.c_int64),
                ("out", C.c_void_p), ("offsets", C.c_void_p)]


class GemmDesc(C.Structure):
    _fields_ = [("trans_a", C.c_int32), ("trans_b", C.c_int32),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64), ("batch", C.c_int64),
                ("lda", C.c_int64), ("ldb", C.c_int64), ("ldc", C.c_int64), ("ld_addend", C.c_int64),
                ("stride_a", C.c_int64), ("stride_b", C.c_int64), ("stride_c", C.c_int64),
                ("stride_addend", C.c_int64),
                ("alpha", C.c_float), ("beta", C.c_float),
                ("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p),
                ("addend", C.c_void_p), ("bias", C.c_void_p),
                ("activation", C.c_int32), ("b_format", C.c_int32), ("math", C.c_int32),
                ("io_flags", C.c_int32), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


ALLOC_FN = C.CFUNCTYPE(C.c_void_p, C.c_void_p, C.c_int, C.c_int32, C.c_int32, C.POINTER(C.c_int64))


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python annc_b200/build.py` "
            "(nvcc, sm_100a). annc_b200 has no CPU fallback.")
    lib = C.CDLL(LIB_PATH)
    lib.annc_last_error.restype = C.c_char_p
    lib.annc_version.restype = C.c_char_p
    lib.annc_get_stream.restype = C.c_void_p
    lib.annc_set_stream.argtypes = [C.c_void_p]
    lib.annc_lookup_custom_call.restype = C.c_void_p
    lib.annc_lookup_custom_call.argtypes = [C.c_char_p]
    lib.annc_select_gemm_target.restype = C.c_char_p
    lib.annc_gemm_kernel_name.restype = C.c_char_p
    lib.annc_embed_bag_workspace_bytes.restype = C.c_size_t
    lib.annc_embed_bag_workspace_bytes.argtypes = [C.c_int, C.c_int64]
    lib.annc_kn4_offset.restype = C.c_int64
    lib.annc_kn4_offset.argtypes = [C.c_int64] * 4
    lib.annc_timer_create.restype = C.c_void_p
    lib.annc_timer_destroy.argtypes = [C.c_void_p]
    lib.annc_timer_elapsed_ms.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]
    lib.annc_embed_bag_set_timing_events.argtypes = [C.c_void_p, C.c_void_p]
    lib.annc_embed_bag_set_stream_ctas_per_sm.argtypes = [C.c_int]
    lib.annc_embed_bag_set_stream_ctas_per_sm.restype = None
    lib.annc_peer_buffer_create.argtypes = [C.c_size_t, C.POINTER(C.c_void_p), C.c_void_p]
    lib.annc_peer_buffer_open.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    lib.annc_peer_buffer_close.argtypes = [C.c_void_p]
    lib.annc_peer_copy_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]
    lib.annc_peer_buffer_destroy.argtypes = [C.c_void_p]
    lib.annc_embed_bag_owner_mask_dev.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int64, C.c_int,
                                                  C.c_void_p, C.c_void_p]
    lib.annc_sum_partials_masked_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int64, C.c_int64,
                                                 C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_int64,
                                                 C.c_int, C.c_void_p]
    lib.annc_synth_fill_rows_dev.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_uint64, C.c_int64,
                                             C.c_int64, C.c_int64, C.c_void_p]
    lib.annc_synth_fill_row_list_dev.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_uint64,
                                                 C.c_int64, C.c_void_p]
    lib.annc_set_operand_cache.argtypes = [C.c_int, C.c_size_t]
    lib.annc_staging_counters.argtypes = [C.POINTER(C.c_uint64)] * 3
    lib.annc_register_constant.argtypes = [C.c_void_p, C.c_size_t]
    lib.annc_unregister_constant.argtypes = [C.c_void_p]
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != 0:
        raise AnncError(rc, lib.annc_last_error().decode(errors="replace"))

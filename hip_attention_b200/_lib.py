"""ctypes binding of libhipattn_sm100.so (declarations: include/hipattn.h)."""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libhipattn_sm100.so")

F32, F16, BF16 = 0, 1, 2
STATUS_PAGE_RANGE, STATUS_TOKEN_RANGE, STATUS_TIMEOUT, STATUS_CHUNK_SIZE = 1, 2, 4, 8
MAX_CHUNKS = 16384
NOALLOC_SCRATCH_BYTES = 16 * 1024 * 1024
ABI_VERSION = 9
SCAN_AUTO, SCAN_STRICT, SCAN_CHECK = 0, 1, 2
ROPE_NONE, ROPE_RELATIVE, ROPE_STREAMING = 0, 1, 2

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class Tokens(C.Structure):
    _fields_ = [("dense", vp), ("stride_b", i64), ("stride_t", i64), ("stride_h", i64),
                ("cache", vp), ("stride_page", i64), ("stride_off", i64), ("stride_ch", i64),
                ("block_table", vp), ("table_stride_b", i64), ("cache_seq_lens", vp), ("n_pages", i64),
                ("table_width", i32), ("table_is_i64", i32), ("seq_lens_is_i64", i32), ("page_size", i32),
                ("fp8_e5m2", i32), ("reserved_", i32)]


class ScanParams(C.Structure):
    _fields_ = [("q", vp), ("q_stride_b", i64), ("q_stride_t", i64), ("q_stride_h", i64),
                ("pos", vp), ("pos_stride_b", i64), ("pos_stride_t", i64),
                ("k", Tokens),
                ("left", vp), ("right", vp), ("score_max", vp),
                ("left_out", vp), ("right_out", vp), ("score_out", vp), ("status", vp), ("key_abs", vp), ("k_scaled", vp), ("stats", vp),
                ("dtype", i32), ("D", i32), ("B", i32), ("TQ", i32), ("H", i32), ("HKV", i32), ("T", i32),
                ("block_size_q", i32), ("stride_q", i32), ("n_chunks", i32), ("block_chunk", i32),
                ("scan_window", i32), ("q_scale", f32), ("k_scale", f32), ("mode", i32), ("chunk_size", i32),
                ("rope_cos", vp), ("rope_sin", vp), ("rope_stride", i64), ("rope_rows", i32), ("rope_mode", i32),
                ("access_counter", vp), ("access_stride_b", i64), ("access_stride_h", i64), ("access_n", i32), ("k_scaled_sides", i32)]


class BsaParams(C.Structure):
    _fields_ = [("q", vp), ("q_stride_b", i64), ("q_stride_t", i64), ("q_stride_h", i64),
                ("out", vp), ("o_stride_b", i64), ("o_stride_t", i64), ("o_stride_h", i64),
                ("pos", vp), ("pos_stride_b", i64), ("pos_stride_t", i64),
                ("k", Tokens), ("v", Tokens),
                ("indices", vp), ("idx_stride_n", i64), ("idx_stride_d", i64),
                ("ks", vp), ("ks_stride_n", i64), ("ks_stride_d", i64),
                ("part_o", vp), ("part_lse", vp), ("lse_out", vp), ("status", vp),
                ("dtype", i32), ("D", i32), ("B", i32), ("TQ", i32), ("H", i32), ("HKV", i32), ("T", i32),
                ("block_size_q", i32), ("index_block_q", i32), ("block_size_k", i32), ("K", i32),
                ("sink", i32), ("window", i32), ("n_splits", i32), ("heads_share_mask", i32),
                ("logit_softcap", f32), ("rope_rows", i32), ("rope_cos", vp), ("rope_sin", vp), ("rope_stride", i64)]


# name -> (restype, argtypes); every symbol include/hipattn.h declares
SYMBOLS = {
    "hipattn_scan_stage": (i32, [C.POINTER(ScanParams), vp]),
    "hipattn_key_abs_sum": (i32, [C.POINTER(Tokens), i32, i32, i32, i32, i32, f32, vp, vp, vp]),
    "hipattn_scan_prepare_keys": (i32, [C.POINTER(Tokens), i32, i32, i32, i32, i32, f32, vp, vp, vp, vp]),
    "hipattn_scan_prepare_keys_rope": (i32, [C.POINTER(Tokens), i32, i32, i32, i32, i32, f32, vp, vp, i64, i32, i32, vp, vp, vp, vp]),
    "hipattn_init_chunks": (i32, [vp, vp, vp, i64, i32, i32, i32, i32, i32, vp]),
    "hipattn_select_stage": (i32, [vp, vp, i64, i32, i32, i32, i32, i32, vp, vp, vp, vp]),
    "hipattn_finalize_indices": (i32, [vp, vp, i64, i64, vp, i64, i64, i32, i32, i32, i32, i32, i32, i32, vp, vp, vp, vp]),
    "hipattn_bsa_attention": (i32, [C.POINTER(BsaParams), vp]),
    "hipattn_merge_partials": (i32, [vp, vp, i64, i32, i32, i32, vp, i64, vp, vp]),
    "hipattn_mark_attention_access": (i32, [C.POINTER(BsaParams), vp, i64, i64, i32, i32, vp]),
    "hipattn_bsa_decode_noalloc": (i32, [C.POINTER(BsaParams), vp]),
    "hipattn_encode_score": (i32, [f32]),
    "hipattn_decode_score": (f32, [i32]),
    "hipattn_decode_scores": (i32, [vp, vp, i64, vp]),
    "hipattn_widen_i32": (i32, [vp, vp, i64, vp]),
    "hipattn_debug_bounded_wait": (i32, [vp, vp]),
    "hipattn_launch_count": (C.c_uint64, []),
    "hipattn_error_string": (C.c_char_p, []),
    "hipattn_abi_version": (i32, []),
}

_lock = threading.Lock()
_lib = None


class HipAttnError(RuntimeError):
    pass


def load():
    """Load the shared library once.  There is no fallback: a missing or stale build is an error."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise HipAttnError(
                    f"{LIB_PATH} is missing: build it with `python -m hip_attention_b200.build` "
                    "(needs nvcc; the library targets sm_100a only and there is no CPU or PyTorch fallback)")
            lib = C.CDLL(LIB_PATH)
            for name, (res, argt) in SYMBOLS.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, argt
            if lib.hipattn_abi_version() != ABI_VERSION:
                raise HipAttnError(f"{LIB_PATH} has ABI {lib.hipattn_abi_version()}, expected {ABI_VERSION}: rebuild it")
            _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc == 0:
        return
    msg = load().hipattn_error_string().decode("utf-8", "replace")
    if rc in (1, 2):
        exc = ValueError if rc == 1 else NotImplementedError
        raise exc(f"{what}: {msg}")
    raise HipAttnError(f"{what}: {msg} (code {rc})")

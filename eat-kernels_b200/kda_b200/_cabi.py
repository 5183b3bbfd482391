"""ctypes binding of include/kda_b200.h.  The library is the only compute path: a missing or unloadable
libkda_b200.so raises, there is no fallback."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libkda_b200.so"

FRONTEND_RAW, FRONTEND_PLAIN = 0, 1
STATE_VALUE_FIRST, STATE_KEY_FIRST = 0, 1
NOALLOC_MAX_SEQS, NOALLOC_MAX_HEADS = 64, 16
KERNEL_TCGEN05, KERNEL_MMA_SYNC, KERNEL_TCGEN05_TWO_TASK = 0, 1, 2
MAX_CUT_PIECES = 128
EXPORTS = ["kda_prefill_workspace_bytes", "kda_prefill_workspace_bytes_cuts", "kda_prefill_launch", "kda_prefill_plan_counts", "kda_prefill_launch_noalloc", "kda_segment_launch", "kda_scan_launch", "kda_scan_strided_launch",
           "kda_fixup_launch", "kda_fixup_tiles_launch", "kda_segment_tiles", "kda_state_rows_copy", "kda_error_string", "kda_abi_struct_bytes", "kda_version",
           "kda_debug_configure"]


class KdaPrefillArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
        ("out", C.c_void_p),
        ("ldq", C.c_int64), ("ldk", C.c_int64), ("ldv", C.c_int64), ("ldg", C.c_int64), ("ldbeta", C.c_int64),
        ("ldo", C.c_int64),
        ("A_log", C.c_void_p), ("dt_bias", C.c_void_p),
        ("scale", C.c_float), ("lower_bound", C.c_float),
        ("frontend", C.c_int32), ("state_layout", C.c_int32), ("H", C.c_int32), ("N", C.c_int32),
        ("T", C.c_int64),
        ("cu_seqlens", C.c_void_p), ("cu_is64", C.c_int32),
        ("src_base", C.c_void_p), ("src_slot_stride", C.c_int64), ("src_idx", C.c_void_p), ("src_idx_is64", C.c_int32),
        ("src_slots", C.c_int64),
        ("dst_base", C.c_void_p), ("dst_slot_stride", C.c_int64), ("dst_idx", C.c_void_p), ("dst_idx_is64", C.c_int32),
        ("dst_slots", C.c_int64),
        ("ck_base", C.c_void_p), ("ck_is_bf16", C.c_int32), ("ck_every", C.c_int32), ("ck_rows", C.c_int64),
        ("ck_starts", C.c_void_p), ("ck_starts_is64", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("kernel", C.c_int32),
        ("max_cut_pieces", C.c_int32),
    ]


class KdaSegmentArgs(C.Structure):
    _fields_ = [
        ("base", KdaPrefillArgs),
        ("n_seg", C.c_int32),
        ("seg_t0", C.c_void_p), ("seg_t1", C.c_void_p), ("seg_need_map", C.c_void_p),
        ("qt", C.c_void_p), ("P", C.c_void_p), ("S_loc", C.c_void_p),
        ("tiles", C.c_void_p), ("n_tiles", C.c_int64),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                "(nvcc, sm_100a). kda_b200 has no other compute path.")
        L = C.CDLL(str(LIB_PATH))
        L.kda_prefill_workspace_bytes.argtypes = [C.c_int32, C.c_int32]
        L.kda_prefill_workspace_bytes.restype = C.c_size_t
        L.kda_prefill_workspace_bytes_cuts.argtypes = [C.c_int32, C.c_int32, C.c_int32]
        L.kda_prefill_workspace_bytes_cuts.restype = C.c_size_t
        L.kda_prefill_launch.argtypes = [C.POINTER(KdaPrefillArgs), C.c_void_p]
        L.kda_prefill_launch.restype = C.c_int
        L.kda_prefill_plan_counts.argtypes = [C.POINTER(KdaPrefillArgs), C.POINTER(C.c_int32), C.c_void_p]
        L.kda_prefill_plan_counts.restype = C.c_int
        L.kda_prefill_launch_noalloc.argtypes = [C.POINTER(KdaPrefillArgs), C.c_void_p]
        L.kda_prefill_launch_noalloc.restype = C.c_int
        L.kda_segment_launch.argtypes = [C.POINTER(KdaSegmentArgs), C.c_void_p]
        L.kda_segment_launch.restype = C.c_int
        L.kda_scan_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                      C.c_void_p]
        L.kda_scan_launch.restype = C.c_int
        L.kda_scan_strided_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32,
                                              C.c_int64, C.c_void_p]
        L.kda_scan_strided_launch.restype = C.c_int
        L.kda_fixup_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_int32, C.c_int32, C.c_void_p]
        L.kda_fixup_launch.restype = C.c_int
        L.kda_fixup_tiles_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_void_p]
        L.kda_fixup_tiles_launch.restype = C.c_int
        L.kda_segment_tiles.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int64]
        L.kda_segment_tiles.restype = C.c_int64
        L.kda_state_rows_copy.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32,
                                          C.c_int32, C.c_void_p]
        L.kda_state_rows_copy.restype = C.c_int
        L.kda_error_string.argtypes = [C.c_int]
        L.kda_error_string.restype = C.c_char_p
        L.kda_version.restype = C.c_char_p
        L.kda_debug_configure.argtypes = [C.c_int64, C.c_int32, C.c_void_p]
        L.kda_debug_configure.restype = C.c_int
        L.kda_abi_struct_bytes.argtypes = [C.c_int]
        L.kda_abi_struct_bytes.restype = C.c_size_t
        if (L.kda_abi_struct_bytes(0) != C.sizeof(KdaPrefillArgs) or L.kda_abi_struct_bytes(1) != C.sizeof(KdaSegmentArgs)):
            raise RuntimeError("libkda_b200.so and the Python binding disagree on the argument struct layout: rebuild")
        _lib = L
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        raise RuntimeError(f"{what} failed: {lib().kda_error_string(rc).decode()} (code {rc})")

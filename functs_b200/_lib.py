"""ctypes binding of libfuncts_b200.so (the C ABI declared in include/functs_b200.h).

There is no fallback: if the library is missing or a symbol cannot be resolved, importing
this module raises.  Nothing here computes on the CPU.
"""
import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_float, c_int32, c_int64, c_uint64, c_void_p

_PKG = os.path.dirname(os.path.abspath(__file__))
# FUNCTS_B200_LIBRARY names another build of the same library (for example one compiled with profiling marks).
LIB_PATH = os.environ.get("FUNCTS_B200_LIBRARY") or os.path.join(_PKG, "libfuncts_b200.so")

FB_OK = 0
FB_STATUS_CAND_OVERFLOW = 1
FB_STATUS_WAIT_TIMEOUT = 2
FB_STATUS_INDEX_RANGE = 4


class FunctsB200Error(RuntimeError):
    """A C-ABI call returned a negative status (the message is functs_b200_last_error())."""


class AccessDesc(ctypes.Structure):
    _fields_ = [
        ("rank", c_int32),
        ("out_shape", c_int64 * 8),
        ("src_stride", c_int64 * 8),
        ("src_mod", c_int64 * 8),
        ("src_offset", c_int64),
    ]


P = c_void_p  # device pointers travel as integers

# name -> (restype, argtypes); this table mirrors include/functs_b200.h one to one
SIGNATURES = {
    "functs_b200_abi_version": (c_int32, []),
    "functs_b200_last_error": (c_char_p, []),
    "functs_b200_launch_count": (c_uint64, []),
    "functs_b200_set_stage_events": (None, [POINTER(c_void_p), c_int32]),
    "functs_b200_rows_select_add_select_rev": (c_int32, [P, P, c_int64, c_int64, c_int64, c_float, P]),
    "functs_b200_hist_bins": (c_int32, []),
    "functs_b200_threshold_compact": (c_int32, [P, c_int32, c_int64, c_float, P, P, c_int64, c_int32, P, P, P]),
    "functs_b200_select_binned_scratch_bytes": (c_int64, [c_int32]),
    "functs_b200_select_topk_binned": (c_int32, [P, P, c_int64, P, c_float, c_int32, c_int32, P, P, P, P]),
    "functs_b200_select_topk": (c_int32, [P, P, c_int64, c_int32, c_int32, P, P, P]),
    "functs_b200_nms_scratch_bytes": (c_int64, [c_int32, c_int32]),
    "functs_b200_batched_nms": (c_int32, [P, c_int64, c_int32, P, P, c_int32, c_int32, c_float, c_int32, P, P, P, P, P, P, P, P]),
    "functs_b200_pack_detections": (c_int32, [P, P, P, P, c_int32, c_int32, P, P]),
    "functs_b200_push_records": (c_int32, [P, P, c_int64, P]),
    "functs_b200_batched_nms_static_max_groups": (c_int32, []),
    "functs_b200_batched_nms_static": (c_int32, [P, c_int64, c_int32, P, P, c_int32, c_int32, c_float, c_int32, P, P, P, P, P, P, P]),
    "functs_b200_yolo_decode": (c_int32, [P, P, P, c_int32, c_int32, c_int32, c_int32, c_float, P, P, P, P, P, c_int64, P, P, P]),
    "functs_b200_yolo_scratch_bytes": (c_int64, [c_int32, c_int32, c_int32, c_int32, c_int64, c_int32]),
    "functs_b200_yolo_postprocess": (c_int32, [P, P, P, c_int32, c_int32, c_int32, c_int32, c_float, c_int32, c_float,
                                               c_int64, P, P, P, P, P, P, P, P]),
    "functs_b200_yolo_postprocess_dense": (c_int32, [P, P, P, c_int32, c_int32, c_int32, c_int32, c_float, c_int32, c_float,
                                                     c_int64, P, P, P, P, P, P, P, P, P, P, P]),
    "functs_b200_ssd_softmax_decode": (c_int32, [P, P, P, c_int32, c_int32, c_int32, c_float, P, P, P]),
    "functs_b200_ssd_class_nms": (c_int32, [P, P, c_int32, c_int32, c_int32, c_float, c_int32, c_float, P, P, P, P]),
    "functs_b200_lstm_scratch_bytes": (c_int64, [c_int32, c_int32, c_int32, c_int32]),
    "functs_b200_lstm_forward": (c_int32, [P, P, P, P, P, c_int32, c_int32, c_int32, c_int32, P, P, P, P, P]),
    "functs_b200_lstm_forward_mode": (c_int32, [P, P, P, P, P, c_int32, c_int32, c_int32, c_int32, P, P, P, P, P, c_int32]),
    "functs_b200_debug_set": (c_int32, [c_char_p, c_int32]),
    "functs_b200_yolact_masks": (c_int32, [P, P, P, c_int32, c_int32, c_int32, c_int32, c_float, P, P, P]),
    "functs_b200_access": (c_int32, [P, P, POINTER(AccessDesc), c_int32, P]),
    "functs_b200_select_rev": (c_int32, [P, P, P, POINTER(c_int64), c_int32, c_int32, c_int64, c_int32, P]),
    "functs_b200_slice_rev": (c_int32, [P, P, P, POINTER(c_int64), c_int32, c_int32, c_int64, c_int64, c_int64, c_int32, P]),
    "functs_b200_index_rows": (c_int32, [P, P, P, c_int64, c_int64, c_int64, c_int32, P, P]),
    "functs_b200_index_rows_rev": (c_int32, [P, P, P, P, c_int64, c_int64, c_int64, c_int32, P, P]),
    "functs_b200_generic_group_launch": (c_int32, [P, c_int32, c_int32, c_int32, c_int32, P]),
    "functs_b200_group_lookup": (c_int32, [c_char_p]),
    "functs_b200_group_count": (c_int32, []),
    "functs_b200_group_signature": (c_char_p, [c_int32]),
    "functs_b200_group_launch": (c_int32, [c_int32, POINTER(c_void_p), POINTER(c_int64), POINTER(c_double),
                                           POINTER(c_void_p), P, P, P]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python functs_b200/build.py` (needs nvcc with sm_100a support); "
            "functs_b200 has no CPU or eager fallback")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the library is older than the header
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    msg = lib.functs_b200_last_error()
    return msg.decode() if msg else ""


def check(rc: int, what: str = "") -> None:
    if rc != FB_OK:
        raise FunctsB200Error(f"{what or 'functs_b200 call'} failed with status {rc}: {last_error()}")


def launch_count() -> int:
    return int(lib.functs_b200_launch_count())

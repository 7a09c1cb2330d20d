"""ctypes declarations for every entry point of include/b200_flat.h."""
from __future__ import annotations

import ctypes
import os

METRIC_INNER_PRODUCT, METRIC_L2 = 0, 1
STORAGE_F32, STORAGE_F16, STORAGE_BF16 = 0, 1, 2
PATH_AUTO, PATH_SCAN, PATH_TENSOR = 0, 1, 2
PLANES_BF16X3, PLANES_FP16X2 = 0, 1
MAX_K = 4096
FUSED_MAX_K = 32
SELECT_AUTO, SELECT_FILTER, SELECT_NO_FILTER, SELECT_MATRIX = 0, 1, 2, 3
GEMM_SHAPE_AUTO, GEMM_SHAPE_SINGLE, GEMM_SHAPE_PAIR = -1, 0, 1
ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_SCRATCH, ERR_CUDA, ERR_DEVICE_WAIT = 1, 2, 3, 4, 5
ERR_NO_DEVICE, ERR_OOM, ERR_RANGE, ERR_STATE, ERR_DEVICE_CHECK = 6, 7, 8, 9, 10

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

c_i64 = ctypes.c_int64
c_i32 = ctypes.c_int32
c_int = ctypes.c_int
c_vp = ctypes.c_void_p
c_sz = ctypes.c_size_t


class B200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__("b200f status %d: %s" % (status, message))
        self.status = status


class Caps(ctypes.Structure):
    _fields_ = [
        ("device", c_i32), ("cc_major", c_i32), ("cc_minor", c_i32), ("sm_count", c_i32),
        ("max_smem_per_block", c_i32), ("l2_bytes", c_i32), ("hbm_bytes", c_i64),
        ("sm_clock_khz", c_i32), ("mem_clock_khz", c_i32), ("supported", c_i32),
        ("name", ctypes.c_char * 128),
    ]


class SearchArgs(ctypes.Structure):
    _fields_ = [
        ("queries", c_vp), ("nq", c_i64), ("d", c_i32), ("storage", c_i32),
        ("rows", c_vp), ("row_pitch", c_i64),
        ("planes", c_vp), ("plane_pitch", c_i64), ("plane_stride", c_i64),
        ("norms", c_vp), ("nb", c_i64), ("metric", c_i32), ("k", c_i32),
        ("label_base", c_i64), ("out_dist", c_vp), ("out_labels", c_vp),
        ("scratch", c_vp), ("scratch_bytes", c_sz), ("status", c_vp), ("stream", c_vp),
        ("path", c_i32), ("norm_cols", c_i32), ("plane_format", c_i32), ("plane_scale_log2", c_i32),
    ]


# name -> (restype, argtypes); the symbol test checks this table against the header
SIGNATURES = {
    "b200f_status_string": (ctypes.c_char_p, [c_int]),
    "b200f_set_selection_mode": (c_int, [c_int]),
    "b200f_get_selection_mode": (c_int, []),
    "b200f_set_gemm_shape": (c_int, [c_int]),
    "b200f_set_rank_select": (c_int, [c_int]),
    "b200f_set_debug_canaries": (c_int, [c_int]),
    "b200f_debug_wait_expiry": (c_int, [c_vp, c_i64, c_vp]),
    "b200f_debug_canary_selftest": (c_int, [c_vp, c_sz, c_int, c_vp, c_vp]),
    "b200f_device_count": (c_int, [ctypes.POINTER(c_int)]),
    "b200f_device_caps": (c_int, [c_int, ctypes.POINTER(Caps)]),
    "b200f_row_norms": (c_int, [c_vp, c_int, c_i64, c_int, c_i64, c_vp, c_vp]),
    "b200f_store_rows": (c_int, [c_vp, c_i64, c_int, c_int, c_vp, c_i64, c_vp, c_i64, c_i64, c_vp, c_int, c_vp]),
    "b200f_store_rows_fp32": (c_int, [c_vp, c_i64, c_i64, c_int, c_vp, c_i64, c_vp, c_i64, c_i64, c_int, c_int, c_vp, c_vp,
                                      c_int, c_vp]),
    "b200f_rows_absmax": (c_int, [c_vp, c_i64, c_int, c_i64, c_vp, c_vp]),
    "b200f_load_rows": (c_int, [c_vp, c_int, c_i64, c_int, c_i64, c_vp, c_vp]),
    "b200f_search_scratch_bytes": (c_sz, [c_i64, c_i64, c_int, c_int, c_int, c_int]),
    "b200f_search": (c_int, [ctypes.POINTER(SearchArgs)]),
    "b200f_noalloc_scratch_capacity": (c_sz, []),
    "b200f_search_small_noalloc": (c_int, [ctypes.POINTER(SearchArgs)]),
    "b200f_pairwise": (c_int, [ctypes.POINTER(SearchArgs), c_vp, c_i64]),
    "b200f_select_scratch_bytes": (c_sz, [c_i64, c_int]),
    "b200f_select_rows": (c_int, [c_vp, c_i64, c_i64, c_i64, c_int, c_int, c_vp, c_vp, c_vp, c_sz, c_vp]),
    "b200f_merge_lists": (c_int, [c_vp, c_vp, c_int, c_i64, c_int, c_int, c_vp, c_vp, c_vp]),
    "b200f_merge_lists_strided": (c_int, [c_vp, c_vp, c_i64, c_i64, c_int, c_i64, c_int, c_int, c_vp, c_vp, c_vp]),
    "b200f_remap_labels_block_cyclic": (c_int, [c_vp, c_i64, c_i64, c_int, c_int, c_vp]),
    "b200f_fill_synthetic": (c_int, [c_vp, c_i64, c_int, c_i64, ctypes.c_uint64, c_int, ctypes.c_float, c_vp]),
    "b200f_profile_enable": (c_int, [c_int]),
    "b200f_profile_read": (c_int, [ctypes.POINTER(c_i64), ctypes.POINTER(c_i64), ctypes.POINTER(ctypes.c_double), c_int]),
    "b200f_last_error": (ctypes.c_char_p, []),
    "b200f_debug_raise": (c_int, [c_int]),
    "b200f_resources_create": (c_int, [c_int, ctypes.POINTER(c_vp)]),
    "b200f_resources_destroy": (None, [c_vp]),
    "b200f_resources_device": (c_int, [c_vp]),
    "b200f_resources_stream": (c_vp, [c_vp]),
    "b200f_resources_wait_stream": (c_int, [c_vp, c_vp]),
    "b200f_resources_scratch_bytes": (c_sz, [c_vp]),
    "b200f_index_create": (c_int, [c_vp, c_int, c_int, c_int, ctypes.POINTER(c_vp)]),
    "b200f_index_destroy": (None, [c_vp]),
    "b200f_index_add": (c_int, [c_vp, c_i64, c_vp]),
    "b200f_index_search": (c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp]),
    "b200f_index_search_enqueue": (c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp]),
    "b200f_index_synchronize": (c_int, [c_vp]),
    "b200f_index_search_async": (c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp, ctypes.POINTER(c_vp)]),
    "b200f_token_wait": (c_int, [c_vp]),
    "b200f_token_is_ready": (c_int, [c_vp, ctypes.POINTER(c_int)]),
    "b200f_token_destroy": (None, [c_vp]),
    "b200f_index_reset": (c_int, [c_vp]),
    "b200f_index_reconstruct": (c_int, [c_vp, c_i64, c_vp]),
    "b200f_index_reconstruct_n": (c_int, [c_vp, c_i64, c_i64, c_vp]),
    "b200f_index_ntotal": (c_i64, [c_vp]),
    "b200f_index_d": (c_int, [c_vp]),
    "b200f_index_metric": (c_int, [c_vp]),
    "b200f_index_storage": (c_int, [c_vp]),
    "b200f_index_set_path": (c_int, [c_vp, c_int]),
    "b200f_index_reserve": (c_int, [c_vp, c_i64]),
    "b200f_index_set_label_base": (c_int, [c_vp, c_i64]),
    "b200f_index_set_growth_mode": (c_int, [c_vp, c_int]),
    "b200f_index_set_use_graphs": (c_int, [c_vp, c_int]),
    "b200f_index_set_fp32_planes": (c_int, [c_vp, c_int]),
    "b200f_index_fp32_planes": (c_int, [c_vp]),
    "b200f_index_device_rows": (c_vp, [c_vp]),
    "b200f_index_last_device_status": (c_int, [c_vp]),
    "b200f_index_debug_wait_expiry": (c_int, [c_vp, c_i64]),
    "b200f_comm_id_create": (c_int, [c_vp]),
    "b200f_sharded_create": (c_int, [ctypes.POINTER(c_vp), c_int, c_int, c_int, c_int, c_i64, ctypes.POINTER(c_vp)]),
    "b200f_sharded_create_rank": (c_int, [c_vp, c_int, c_int, c_vp, ctypes.POINTER(c_vp)]),
    "b200f_sharded_destroy": (None, [c_vp]),
    "b200f_sharded_add": (c_int, [c_vp, c_i64, c_vp]),
    "b200f_sharded_search": (c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp]),
    "b200f_sharded_search_enqueue": (c_int, [c_vp, c_i64, c_vp, c_i64, c_vp, c_vp]),
    "b200f_sharded_synchronize": (c_int, [c_vp]),
    "b200f_sharded_reset": (c_int, [c_vp]),
    "b200f_sharded_reconstruct": (c_int, [c_vp, c_i64, c_vp]),
    "b200f_sharded_ntotal": (c_i64, [c_vp]),
    "b200f_sharded_num_shards": (c_int, [c_vp]),
    "b200f_sharded_set_path": (c_int, [c_vp, c_int]),
    "b200f_sharded_set_use_graphs": (c_int, [c_vp, c_int]),
    "b200f_sharded_trace": (c_int, [c_vp, c_int]),
    "b200f_sharded_trace_read": (c_i64, [c_vp, c_vp, c_vp, c_i64]),
}


def lib_path() -> str:
    return os.path.join(_HERE, "lib", "libb200flat.so")


def lib() -> ctypes.CDLL:
    """Load libb200flat.so (built in-tree by build.py).  Fails loudly when missing."""
    global _LIB
    if _LIB is None:
        path = lib_path()
        if not os.path.exists(path):
            raise ImportError(
                "libb200flat.so is not built (%s); run `python faiss-metal_b200/build.py`. "
                "There is no fallback implementation." % path)
        L = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)
            fn.restype = res
            fn.argtypes = args
        _LIB = L
    return _LIB


def status_string(status: int) -> str:
    return lib().b200f_status_string(int(status)).decode()


def check(status: int, what: str = "") -> None:
    if status != 0:
        msg = lib().b200f_last_error().decode() or status_string(status)
        raise B200Error(status, (what + ": " if what else "") + msg)


def check_op(status: int, what: str = "") -> None:
    """For op-level entry points (no per-thread message)."""
    if status != 0:
        raise B200Error(status, (what + ": " if what else "") + status_string(status))

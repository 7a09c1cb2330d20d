"""CPU checks of the drop-in boundary: the library loads, exports every symbol the
header declares, and fails loudly (no CPU fallback) when there is no GPU."""
import ctypes
import os
import re

import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(REPO, "include", "b200_flat.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b(b200f_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_header_symbols_exported(fm):
    names = declared_functions()
    assert len(names) >= 35
    L = ctypes.CDLL(fm.lib_path())
    missing = [n for n in names if not hasattr(L, n)]
    assert not missing, missing


def test_ctypes_table_matches_header(fm):
    from faiss_metal_b200 import abi  # noqa: F401
    import faiss_metal_b200
    table = set(faiss_metal_b200.abi.SIGNATURES)
    assert table == set(declared_functions())


def test_search_args_layout(fm):
    # struct layout must match the C declaration (all 8-byte fields naturally aligned)
    a = fm.abi.SearchArgs
    assert ctypes.sizeof(a) == 160
    assert a.nb.offset == 72 and a.scratch.offset == 112 and a.path.offset == 144


def test_status_strings(fm):
    for code in range(0, 11):
        s = fm.status_string(code)
        assert isinstance(s, str) and s and s != "unknown status"
    assert fm.status_string(99) == "unknown status"


def test_no_gpu_fails_loudly(fm):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(fm.B200Error) as e:
        fm.StandardB200Resources(0)
    assert e.value.status == 6  # B200F_ERR_NO_DEVICE
    assert "no CPU fallback" in str(e.value)


def test_bad_arguments_rejected_without_gpu(fm):
    L = fm.lib()
    assert L.b200f_search(None) == 1
    assert L.b200f_search_scratch_bytes(10, 100, 0, 5, 0, 0) == 0
    assert L.b200f_search_scratch_bytes(10, 100, 8, 0, 0, 0) == 0
    h = ctypes.c_void_p()
    assert L.b200f_index_create(None, 8, 1, 0, ctypes.byref(h)) == 1
    assert L.b200f_merge_lists(None, None, 0, 1, 1, 1, None, None, None) == 1
    assert L.b200f_select_rows(None, 1, 10, 5, 1, 3, None, None, None, 0, None) == 1  # ld < ncols
    assert L.b200f_index_ntotal(None) == -1


def test_every_status_code_comes_out_of_a_typed_exception(fm):
    # the host layer throws exceptions that carry their status code; the C mirror returns the
    # code without looking at the message
    L = fm.lib()
    assert L.b200f_debug_raise(0) == 0
    for code in range(1, 11):
        assert L.b200f_debug_raise(code) == code
        assert fm.status_string(code) in L.b200f_last_error().decode()
    assert L.b200f_debug_raise(-1) == fm.abi.ERR_BAD_ARG     # foreign FaissException
    assert L.b200f_debug_raise(-2) == fm.abi.ERR_CUDA        # foreign runtime_error
    assert L.b200f_debug_raise(-3) == fm.abi.ERR_OOM         # bad_alloc


def test_library_switches_without_gpu(fm):
    L = fm.lib()
    old = L.b200f_get_selection_mode()
    assert old in (0, 1, 2, 3)
    for mode in (1, 2, 3, 0):
        assert L.b200f_set_selection_mode(mode) == 0 and L.b200f_get_selection_mode() == mode
    assert L.b200f_set_selection_mode(4) == 1 and L.b200f_set_selection_mode(-1) == 1
    L.b200f_set_selection_mode(old)
    assert L.b200f_set_gemm_shape(2) == 1 and L.b200f_set_gemm_shape(-1) == 0
    # debug canaries add a guard behind every slice of the scratch region
    plain = L.b200f_search_scratch_bytes(64, 100000, 128, 10, 2, 2)
    assert L.b200f_set_debug_canaries(1) == 0
    guarded = L.b200f_search_scratch_bytes(64, 100000, 128, 10, 2, 2)
    assert L.b200f_set_debug_canaries(0) == 0
    assert guarded > plain and (guarded - plain) % 256 == 0
    assert L.b200f_search_scratch_bytes(64, 100000, 128, 10, 2, 2) == plain


def test_python_mirror_validates_arrays(fm):
    # dtype / shape errors are caught before a pointer reaches the C side
    import numpy as np
    from faiss_metal_b200 import index as I
    with pytest.raises(ValueError):
        I._check(np.zeros((3, 4), np.float64), "x", "float32", (3, 4))
    with pytest.raises(ValueError):
        I._check(np.zeros((3, 5), np.float32), "x", "float32", (3, 4))
    with pytest.raises(TypeError):
        I._check([1.0, 2.0], "x", "float32", (2,))
    I._check(np.zeros((3, 4), np.float32), "x", "float32", (3, 4))

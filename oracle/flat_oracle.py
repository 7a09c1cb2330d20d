"""CPU oracle for flat k-NN search -- TEST INFRASTRUCTURE ONLY.

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product never does.

Two independent restatements of the CPU semantics the reference is compared
with (faiss::IndexFlatL2 / IndexFlatIP, tests/test_metal_flat.mm:73-78,108-113):

* ``flat_oracle.c`` (loaded through ctypes): double-accumulated loops that
  follow the reference's inline CPU code
  (tests/test_metal_distance.mm:46-51,141-147,193-198), OpenMP over queries.
* ``numpy_search`` below: a pure numpy float64 version used to cross-check the
  C file on small cases, and ``blas_search`` (sgemm + partial select, the way
  CPU FAISS evaluates large batches) used as the timed CPU baseline.

PARITY PINNING: pinned to the reference's own CPU code -- the inline loops and seeded
generators of its unit tests, compiled out of the reference tree by ``make -C oracle ref``
(ref_loops.cpp) into tests/golden/ref_loops.npz and checked by tests/test_ref_pin.py: norms,
squared-L2 and inner-product values to 1e-5 relative, rank-1 labels exactly, on the shapes of
tests/test_metal_flat.mm:477-490; plus the reference's known-answer cases (empty index,
k > ntotal padding, reconstruct round trips).  Ranks >= 2, k > 10 and BF16 storage are not
pinned by anything the reference holds; CPU FAISS, its external comparison, is not installed.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

METRIC_INNER_PRODUCT = 0  # faiss::METRIC_INNER_PRODUCT
METRIC_IP = METRIC_INNER_PRODUCT
METRIC_L2 = 1  # faiss::METRIC_L2
STORAGE_F32, STORAGE_F16, STORAGE_BF16 = 0, 1, 2  # include/faiss-metal/MetalIndexFlat.h:39-43

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libflat_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile flat_oracle.c with the Makefile beside it (gcc, OpenMP)."""
    src = os.path.join(_HERE, "flat_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        env = dict(os.environ)
        env.pop("CC", None)
        subprocess.check_call(["make", "-C", _HERE, "-s"], env=env)
    return _LIB_PATH


def build_ref(ref_root: str | None = None) -> str | None:
    """Compile the reference's own CPU loops (``make ref``: ref_loops.cpp around lines cut out of
    the reference's test files) into _ref/ref_loops.  Returns None when the reference checkout
    is not present, which is the normal case away from the machine the fixtures are made on."""
    root = ref_root or os.environ.get("B200F_REFERENCE_ROOT", "/root/reference")
    if not os.path.isfile(os.path.join(root, "tests", "test_metal_distance.mm")):
        return None
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.check_call(["make", "-C", _HERE, "-s", "ref", "REF=" + root], env=env)
    return os.path.join(_HERE, "_ref", "ref_loops")


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        c_f = ctypes.POINTER(ctypes.c_float)
        c_d = ctypes.POINTER(ctypes.c_double)
        c_l = ctypes.POINTER(ctypes.c_int64)
        c_h = ctypes.POINTER(ctypes.c_uint16)
        i64, i32 = ctypes.c_int64, ctypes.c_int
        L.oracle_num_threads.restype = i32
        L.oracle_round_storage.argtypes = [c_f, i64, i32, c_f]
        L.oracle_to_bits16.argtypes = [c_f, i64, i32, c_h]
        L.oracle_row_norms.argtypes = [c_f, i64, i32, c_f]
        L.oracle_pairwise.argtypes = [i32, c_f, i64, c_f, i64, i32, c_d]
        L.oracle_rescore.argtypes = [i32, c_f, i64, c_f, i64, i32, i64, c_l, c_d]
        L.oracle_search.argtypes = [i32, c_f, i64, c_f, i64, i32, i64, c_f, c_l, c_d]
        L.oracle_search.restype = i32
        L.oracle_merge.argtypes = [i32, i32, i64, i64, c_f, c_l, c_l, c_f, c_l]
        L.oracle_merge.restype = i32
        _lib = L
    return _lib


def _f(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def _d(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def _l(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int64))


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def round_storage(x: np.ndarray, storage: int) -> np.ndarray:
    """fp32 -> stored precision -> fp32 (src/MetalIndexFlat.mm:224-255,508-527)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().oracle_round_storage(_f(x), x.size, int(storage), _f(out))
    return out


def to_bits16(x: np.ndarray, storage: int) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_to_bits16(_f(x), x.size, int(storage), out.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)))
    return out


def row_norms(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    n, d = x.shape
    out = np.empty(n, dtype=np.float32)
    lib().oracle_row_norms(_f(x), n, d, _f(out))
    return out


def pairwise(metric: int, xb: np.ndarray, xq: np.ndarray) -> np.ndarray:
    xb = np.ascontiguousarray(xb, dtype=np.float32)
    xq = np.ascontiguousarray(xq, dtype=np.float32)
    out = np.empty((xq.shape[0], xb.shape[0]), dtype=np.float64)
    lib().oracle_pairwise(int(metric), _f(xb), xb.shape[0], _f(xq), xq.shape[0], xb.shape[1], _d(out))
    return out


def rescore(metric: int, xb: np.ndarray, xq: np.ndarray, labels: np.ndarray) -> np.ndarray:
    """Exact (double) score of every returned (query, label) pair."""
    xb = np.ascontiguousarray(xb, dtype=np.float32)
    xq = np.ascontiguousarray(xq, dtype=np.float32)
    labels = np.ascontiguousarray(labels, dtype=np.int64)
    nq, k = labels.shape
    out = np.empty((nq, k), dtype=np.float64)
    lib().oracle_rescore(int(metric), _f(xb), xb.shape[0], _f(xq), nq, xb.shape[1], k, _l(labels), _d(out))
    return out


def search(metric: int, xb: np.ndarray, xq: np.ndarray, k: int):
    """IndexFlatL2 / IndexFlatIP search: (float32 distances, int64 labels, float64 distances)."""
    xb = np.ascontiguousarray(xb, dtype=np.float32)
    xq = np.ascontiguousarray(xq, dtype=np.float32)
    nb = xb.shape[0]
    nq = xq.shape[0]
    d = xq.shape[1] if xq.ndim == 2 else xb.shape[1]
    out_d = np.empty((nq, k), dtype=np.float32)
    out_i = np.empty((nq, k), dtype=np.int64)
    out_d64 = np.empty((nq, k), dtype=np.float64)
    if nq == 0:
        return out_d, out_i, out_d64
    rc = lib().oracle_search(int(metric), _f(xb), nb, _f(xq), nq, d, k, _f(out_d), _l(out_i), _d(out_d64))
    if rc != 0:
        raise ValueError("oracle_search: bad arguments")
    return out_d, out_i, out_d64


def merge(metric: int, dist: np.ndarray, local_ids: np.ndarray, base: np.ndarray):
    """k-way merge of per-shard sorted lists: dist/local_ids are [P, nq, k]."""
    dist = np.ascontiguousarray(dist, dtype=np.float32)
    local_ids = np.ascontiguousarray(local_ids, dtype=np.int64)
    base = np.ascontiguousarray(base, dtype=np.int64)
    P, nq, k = dist.shape
    out_d = np.empty((nq, k), dtype=np.float32)
    out_i = np.empty((nq, k), dtype=np.int64)
    rc = lib().oracle_merge(int(metric), P, nq, k, _f(dist), _l(local_ids), _l(base), _f(out_d), _l(out_i))
    if rc != 0:
        raise ValueError("oracle_merge: bad arguments")
    return out_d, out_i


# ---------------------------------------------------------------------------
# numpy restatements
# ---------------------------------------------------------------------------
def numpy_search(metric: int, xb: np.ndarray, xq: np.ndarray, k: int):
    """Pure numpy float64 restatement (small cases): same contract as search()."""
    xb64 = np.asarray(xb, dtype=np.float64)
    xq64 = np.asarray(xq, dtype=np.float64)
    nb, nq = xb64.shape[0], xq64.shape[0]
    pad = np.inf if metric == METRIC_L2 else -np.inf
    out_d = np.full((nq, k), pad, dtype=np.float64)
    out_i = np.full((nq, k), -1, dtype=np.int64)
    for i in range(nq):
        if nb == 0:
            break
        if metric == METRIC_L2:
            diff = xb64 - xq64[i]
            key = np.einsum("ij,ij->i", diff, diff)
        else:
            key = -(xb64 @ xq64[i])
        order = np.lexsort((np.arange(nb), key))[: min(k, nb)]
        out_i[i, : order.size] = order
        out_d[i, : order.size] = key[order] if metric == METRIC_L2 else -key[order]
    return out_d.astype(np.float32), out_i, out_d


def blas_search(metric: int, xb: np.ndarray, xq: np.ndarray, k: int, xb_norms=None, block: int = 65536):
    """sgemm-based search, the algorithm CPU FAISS uses for batches of queries
    (norms + Q.X^T through BLAS, then a partial select per row).  Used as the
    timed CPU baseline; fp32 arithmetic, all BLAS threads."""
    xb = np.asarray(xb, dtype=np.float32)
    xq = np.asarray(xq, dtype=np.float32)
    nb, nq = xb.shape[0], xq.shape[0]
    kk = min(k, nb)
    best_d = np.full((nq, 0), 0, dtype=np.float32)
    best_i = np.full((nq, 0), 0, dtype=np.int64)
    if metric == METRIC_L2:
        qn = np.einsum("ij,ij->i", xq, xq)
        if xb_norms is None:
            xb_norms = np.einsum("ij,ij->i", xb, xb)
    for j0 in range(0, nb, block):
        j1 = min(nb, j0 + block)
        dots = xq @ xb[j0:j1].T
        if metric == METRIC_L2:
            key = qn[:, None] + xb_norms[None, j0:j1] - 2.0 * dots
            np.maximum(key, 0, out=key)
        else:
            key = -dots
        kb = min(kk, j1 - j0)
        part = np.argpartition(key, kb - 1, axis=1)[:, :kb] if kb < key.shape[1] else np.tile(np.arange(key.shape[1]), (nq, 1))
        cand_d = np.take_along_axis(key, part, axis=1)
        best_d = np.concatenate([best_d, cand_d], axis=1)
        best_i = np.concatenate([best_i, part.astype(np.int64) + j0], axis=1)
        if best_d.shape[1] > 4 * kk:
            sel = np.argpartition(best_d, kk - 1, axis=1)[:, :kk]
            best_d = np.take_along_axis(best_d, sel, axis=1)
            best_i = np.take_along_axis(best_i, sel, axis=1)
    order = np.lexsort((best_i, best_d), axis=1)[:, :kk]
    best_d = np.take_along_axis(best_d, order, axis=1)
    best_i = np.take_along_axis(best_i, order, axis=1)
    pad = np.inf if metric == METRIC_L2 else -np.inf
    out_d = np.full((nq, k), pad, dtype=np.float32)
    out_i = np.full((nq, k), -1, dtype=np.int64)
    out_d[:, :kk] = best_d if metric == METRIC_L2 else -best_d
    out_i[:, :kk] = best_i
    return out_d, out_i


# ---------------------------------------------------------------------------
# comparator
# ---------------------------------------------------------------------------
def compare_results(metric, got_d, got_i, ref_d64, ref_i, true_d64_of_got, tol, eps=1e-6):
    """Tolerance- and tie-aware comparison of a search result with the oracle.

    got_d / got_i        result under test, [nq, k]
    ref_d64 / ref_i      oracle result (double scores), [nq, k]
    true_d64_of_got      oracle score of every label the result returned
                         (``rescore``): proves a differing label is a genuine
                         near-tie and not a wrong neighbour
    tol                  relative tolerance: 1e-4 for FP32 storage, 2e-2 for
                         FP16 / BF16 storage

    Rules: (1) reported distance within tol (relative, floor eps) of the oracle
    distance at the same rank; (2) label equal to the oracle's, or the label's
    true distance within tol of the oracle's distance at that rank (a tie
    group); (3) padding (-1 labels, +/-INF) identical; (4) no label repeated
    within a row.  Returns a dict of failure counts (all zero = pass).
    """
    got_d = np.asarray(got_d, dtype=np.float64)
    got_i = np.asarray(got_i)
    ref_d64 = np.asarray(ref_d64, dtype=np.float64)
    ref_i = np.asarray(ref_i)
    true_d = np.asarray(true_d64_of_got, dtype=np.float64)
    pad_ref = ref_i < 0
    pad_got = got_i < 0
    res = {"pad_mismatch": int(np.count_nonzero(pad_ref != pad_got))}
    if metric == METRIC_L2:
        res["pad_value"] = int(np.count_nonzero(~np.isposinf(got_d[pad_got])))
    else:
        res["pad_value"] = int(np.count_nonzero(~np.isneginf(got_d[pad_got])))
    live = ~pad_ref & ~pad_got
    scale = np.maximum(np.abs(ref_d64), eps)
    with np.errstate(invalid="ignore"):
        derr = np.abs(got_d - ref_d64) / scale
        terr = np.abs(true_d - ref_d64) / scale
    res["dist"] = int(np.count_nonzero(live & ~(derr <= tol)))
    res["max_rel_dist_err"] = float(np.nanmax(np.where(live, derr, 0.0))) if live.any() else 0.0
    label_diff = live & (got_i != ref_i)
    res["label_diff"] = int(np.count_nonzero(label_diff))
    res["label_bad"] = int(np.count_nonzero(label_diff & ~(terr <= tol)))
    dup = 0
    for r in range(got_i.shape[0]):
        row = got_i[r][got_i[r] >= 0]
        dup += row.size - np.unique(row).size
    res["duplicates"] = int(dup)
    return res


def passed(res: dict) -> bool:
    return all(res[key] == 0 for key in ("pad_mismatch", "pad_value", "dist", "label_bad", "duplicates"))

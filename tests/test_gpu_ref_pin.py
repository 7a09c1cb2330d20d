"""GPU results against what the reference's own CPU loops compute on the reference's own seeded
inputs (tests/golden/ref_loops.npz, see tests/test_ref_pin.py): the same cases as
tests/test_metal_distance.mm:17-230 and tests/test_metal_flat.mm:61-121,477-490, through the
C-ABI, at the reference's tolerances or tighter."""
import ctypes
import os

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O
from test_gpu_ops import Stored, cur_stream, vp
from test_ref_pin import FLAT_CASES, flat_inputs

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_loops.npz")


@pytest.fixture(scope="module")
def ref():
    return np.load(FIX)


@pytest.mark.parametrize("case", ["norm_small", "norm_large"])
def test_row_norms_against_reference_loop(fm, res, ref, case):
    # reference tolerances: 1e-3 absolute (100 x 128), 1e-4 relative (10 x 1536); here 1e-5 relative
    x = ref[case + "_x"]
    n, d = x.shape
    st = Stored(fm, x, 0)
    out = torch.zeros(n, dtype=torch.float32, device="cuda:0")
    fm.abi.check_op(fm.lib().b200f_row_norms(vp(st.rows), 0, n, d, st.pitch, vp(out), cur_stream()), "row_norms")
    np.testing.assert_allclose(out.cpu().numpy(), ref[case + "_out"], rtol=1e-5, atol=0)
    np.testing.assert_allclose(st.norms[:n].cpu().numpy(), ref[case + "_out"], rtol=1e-5, atol=0)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("storage", [0, 1, 2])
@pytest.mark.parametrize("name", ["l2", "ip"])
def test_pairwise_against_reference_loops(fm, res, ref, name, storage, path):
    # reference tolerance 5e-2 relative on every storage; here 1e-4 (FP32 storage) / 2e-2 (16-bit)
    metric = O.METRIC_L2 if name == "l2" else O.METRIC_INNER_PRODUCT
    xq, xb, want = ref[name + "_q"], ref[name + "_x"], ref[name + "_out"].astype(np.float64)
    nq, nb = want.shape
    st = Stored(fm, xb, storage)
    out = torch.full((nq, nb), float("nan"), dtype=torch.float32, device="cuda:0")
    a = st.args(fm, torch.from_numpy(xq).cuda(), metric, 1, path)
    fm.abi.check_op(fm.lib().b200f_pairwise(ctypes.byref(a), vp(out), nb), "pairwise")
    torch.cuda.synchronize()
    assert int(st.status[0]) == 0
    got = out.cpu().numpy().astype(np.float64)
    tol = H.TOL_NORTH_STAR[storage]
    if metric == O.METRIC_L2:
        assert (np.abs(got - want) <= tol * np.maximum(want, 1e-6)).all()
    else:
        assert np.abs(got - want).max() <= tol * np.abs(want).max()
    if name == "ip" and storage == 0:
        # top-1 of the reference's CPU side (tests/test_metal_distance.mm:206-227)
        assert np.array_equal(np.argmax(got, axis=1), ref["ip_top1"])


@pytest.mark.parametrize("storage", [0, 1])
@pytest.mark.parametrize("tag", FLAT_CASES)
def test_index_search_against_reference_loops(fm, res, ref, tag, storage):
    # The reference asserts rank-1 label equality with its CPU side and prints distance
    # differences above 1e-3 (tests/test_metal_flat.mm:16-59); FP16 storage is run on the
    # 1000 x 128 and 500 x 768 shapes (:483-484).  Here: rank 1 identical, every rank within
    # the tolerance of the storage type or a proven tie, for both storages on every shape.
    xb, xq, k = flat_inputs(ref, tag)
    metric = O.METRIC_INNER_PRODUCT if "_ip_" in tag else O.METRIC_L2
    want = ref[tag + "_out"].astype(np.float64)
    key = want if metric == O.METRIC_L2 else -want
    order = np.stack([np.lexsort((np.arange(key.shape[1]), key[i]))[:k] for i in range(key.shape[0])])
    ref_d = np.take_along_axis(want, order, axis=1)
    idx = fm.B200IndexFlat(res, xb.shape[1], metric, storage)
    idx.add(xb)
    for path in (fm.PATH_AUTO, fm.PATH_SCAN, fm.PATH_TENSOR):
        idx.set_path(path)
        D, I = idx.search(xq, k)
        true_d = np.take_along_axis(want, np.maximum(I, 0), axis=1)   # the reference's value of each returned row
        tol = H.TOL_NORTH_STAR[storage]
        r = O.compare_results(metric, D, I, ref_d, order, true_d, tol, eps=1e-3 * float(np.abs(want).max()))
        assert O.passed(r), (path, r)
        if storage == 0:
            assert np.array_equal(I[:, 0], order[:, 0]), "rank 1 differs from the reference's CPU side"
            assert r["label_diff"] == 0
        else:
            # 16-bit storage may swap rows whose reference distances lie within its rounding error
            swapped = I[:, 0] != order[:, 0]
            gap = np.abs(true_d[:, 0] - ref_d[:, 0]) / np.maximum(np.abs(ref_d[:, 0]), 1e-6)
            assert (gap[swapped] <= tol).all()
    idx.close()

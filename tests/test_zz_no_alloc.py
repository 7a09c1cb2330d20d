"""GPU test of b200f_search_small_noalloc, the entry point for callers that cannot
allocate device memory when they search (a serving loop that must stay off the allocator,
a plugin without a memory pool of its own).  It must give exactly what b200f_search gives
with caller-provided scratch, call after call, although every call reuses the same built-in
scratch array and finds the previous call's leftovers in it.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already gone through every other test."""
import ctypes

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _search(fm, st, xq, metric, k, noalloc):
    xq_dev = torch.from_numpy(xq).cuda()
    nq = xq.shape[0]
    out_d = torch.full((nq, k), float("nan"), dtype=torch.float32, device="cuda:0")
    out_l = torch.full((nq, k), -7, dtype=torch.int64, device="cuda:0")
    a = st.args(fm, xq_dev, metric, k, 1, out_d, out_l)
    if noalloc:
        a.scratch = None          # the point of the entry point: no scratch from the caller
        a.scratch_bytes = 0
        rc = fm.lib().b200f_search_small_noalloc(ctypes.byref(a))
    else:
        rc = fm.lib().b200f_search(ctypes.byref(a))
    fm.abi.check_op(rc, "search")
    torch.cuda.synchronize()
    assert int(st.status[0]) == 0
    return out_d.cpu().numpy(), out_l.cpu().numpy()


@pytest.mark.parametrize("storage,metric,nb,d", [(1, O.METRIC_L2, 60_000, 128), (2, O.METRIC_INNER_PRODUCT, 3_000, 96),
                                                  (0, O.METRIC_L2, 5_000, 40)])
def test_noalloc_matches_regular_entry_point_twice(fm, res, storage, metric, nb, d):
    from test_gpu_ops import Stored
    assert fm.lib().b200f_noalloc_scratch_capacity() == 1 << 20
    xb = H.uniform_pm1(nb, d, 5)
    st = Stored(fm, xb, storage)
    # two calls in a row with different shapes: the second one finds the first one's lists
    for call, (nq, k, seed) in enumerate([(4, 32, 11), (1, 10, 12), (3, 7, 13)]):
        xq = H.uniform_pm1(nq, d, seed)
        assert fm.lib().b200f_search_scratch_bytes(nq, nb, d, k, storage, 1) <= fm.lib().b200f_noalloc_scratch_capacity()
        want_d, want_l = _search(fm, st, xq, metric, k, noalloc=False)
        got_d, got_l = _search(fm, st, xq, metric, k, noalloc=True)
        assert np.array_equal(got_l, want_l), call
        assert np.array_equal(got_d, want_d), call   # same kernels, same order: bit-equal
        H.check_against_oracle(metric, storage, storage != 0 and nb >= 50_000, xb, xq, k, got_d, got_l)


def test_noalloc_rejects_shapes_beyond_its_scratch(fm, res):
    from test_gpu_ops import Stored
    xb = H.uniform_pm1(2000, 32, 1)
    st = Stored(fm, xb, 0)
    xq = torch.from_numpy(H.uniform_pm1(8, 32, 2)).cuda()
    out_d = torch.empty((8, 10), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((8, 10), dtype=torch.int64, device="cuda:0")
    a = st.args(fm, xq, O.METRIC_L2, 10, 1, out_d, out_l)
    assert fm.lib().b200f_search_small_noalloc(ctypes.byref(a)) == 2      # nq > 4: unsupported
    xq1 = xq[:1].contiguous()
    a = st.args(fm, xq1, O.METRIC_L2, 33, 1, out_d, out_l)
    a.k = 33
    assert fm.lib().b200f_search_small_noalloc(ctypes.byref(a)) == 2      # k > 32: unsupported
    assert fm.lib().b200f_search_small_noalloc(None) == 1
    a = st.args(fm, xq1, O.METRIC_L2, 10, 1, out_d, out_l)
    a.k = 0
    assert fm.lib().b200f_search_small_noalloc(ctypes.byref(a)) == 1      # same code as b200f_search
    a.k = 10
    a.nq = -1
    assert fm.lib().b200f_search_small_noalloc(ctypes.byref(a)) == 1


def test_noalloc_leaves_device_memory_untouched(fm, res):
    """The property in the name: over many calls the driver's count of free device memory does
    not move (cudaMemGetInfo), so nothing was allocated, from any pool."""
    from test_gpu_ops import Stored
    xb = H.uniform_pm1(40_000, 64, 3)
    st = Stored(fm, xb, 1)
    xq = torch.from_numpy(H.uniform_pm1(2, 64, 4)).cuda()
    out_d = torch.empty((2, 10), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((2, 10), dtype=torch.int64, device="cuda:0")
    a = st.args(fm, xq, O.METRIC_L2, 10, 1, out_d, out_l)
    a.scratch = None
    a.scratch_bytes = 0
    L = fm.lib()
    for _ in range(3):   # first call on the device looks the array's address up; warm everything
        fm.abi.check_op(L.b200f_search_small_noalloc(ctypes.byref(a)), "noalloc")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(100):
        fm.abi.check_op(L.b200f_search_small_noalloc(ctypes.byref(a)), "noalloc")
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert int(st.status[0]) == 0

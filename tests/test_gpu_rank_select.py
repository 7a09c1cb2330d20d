"""The register-sorting / binary-search selection kernels (select_rank.cu) against the
shared-memory sorting kernel they stand in for and against numpy: bit-equal on random input, on
ties, on lists that are not in label order among equal distances, on empty slots and on labels
beyond 2^32."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu


def vp(t):
    return ctypes.c_void_p(t.data_ptr())


def cur_stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def merge(fm, dd, ll, metric, rank_select):
    P, nq, k = dd.shape
    L = fm.lib()
    d_dev = torch.from_numpy(dd).cuda()
    l_dev = torch.from_numpy(ll).cuda()
    out_d = torch.full((nq, k), 123.0, dtype=torch.float32, device="cuda:0")
    out_l = torch.full((nq, k), -7, dtype=torch.int64, device="cuda:0")
    assert L.b200f_set_rank_select(1 if rank_select else 0) == 0
    try:
        fm.abi.check_op(L.b200f_merge_lists(vp(d_dev), vp(l_dev), P, nq, k, metric, vp(out_d), vp(out_l),
                                            cur_stream()), "merge_lists")
        torch.cuda.synchronize()
    finally:
        L.b200f_set_rank_select(1)
    return out_d.cpu().numpy(), out_l.cpu().numpy()


def numpy_merge(dd, ll, metric):
    """k best of the live entries by (key, label); key = dist (L2) or -dist (inner product)."""
    P, nq, k = dd.shape
    out_d = np.full((nq, k), np.inf if metric == O.METRIC_L2 else -np.inf, dtype=np.float32)
    out_l = np.full((nq, k), -1, dtype=np.int64)
    for q in range(nq):
        d = dd[:, q, :].reshape(-1)
        l = ll[:, q, :].reshape(-1)
        live = l >= 0
        d, l = d[live], l[live]
        key = d if metric == O.METRIC_L2 else -d
        order = np.lexsort((l, key))[:k]
        out_d[q, :len(order)] = d[order]
        out_l[q, :len(order)] = l[order]
    return out_d, out_l


def make_lists(rng, P, nq, k, metric, levels, fill, label_hi=0, in_label_order=True):
    """P lists of k entries per query, best first.  `levels` distinct distance values (few = many
    ties), a fraction `fill` of every list live; labels distinct per query."""
    dd = np.empty((P, nq, k), dtype=np.float32)
    ll = np.empty((P, nq, k), dtype=np.int64)
    values = rng.standard_normal(levels).astype(np.float32)
    for q in range(nq):
        labels = rng.permutation(P * k * 3)[:P * k].astype(np.int64) + label_hi
        for p in range(P):
            live = int(round(fill * k)) if fill < 1 else k
            if fill < 1 and rng.integers(0, 4) == 0:
                live = int(rng.integers(0, k + 1))
            d = values[rng.integers(0, levels, size=live)]
            l = labels[p * k:p * k + live]
            key = d if metric == O.METRIC_L2 else -d
            if in_label_order:
                order = np.lexsort((l, key))
            else:
                # ascending key only: equal keys keep a random label order, as final distances
                # that tie after rounding do
                order = np.argsort(key, kind="stable")
            dd[p, q, :live] = d[order]
            ll[p, q, :live] = l[order]
            dd[p, q, live:] = np.inf if metric == O.METRIC_L2 else -np.inf
            ll[p, q, live:] = -1
    return dd, ll


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("P,nq,k,levels,fill", [
    (8, 300, 100, 100000, 1.0),     # the eight-shard merge of a k = 100 search
    (8, 40, 1024, 100000, 1.0),     # 8192 entries: the largest input
    (2, 50, 33, 7, 1.0),            # nearly everything ties
    (5, 64, 129, 50, 0.6),          # empty tails, some lists empty
    (16, 30, 512, 1000, 0.9),
    (1, 20, 77, 10, 0.5),           # a single list
    (7, 10, 1170, 3, 1.0),          # P k = 8190
])
def test_merge_matches_sorting_kernel_and_numpy(fm, res, metric, P, nq, k, levels, fill):
    rng = np.random.default_rng(P * 1000 + k)
    dd, ll = make_lists(rng, P, nq, k, metric, levels, fill)
    new_d, new_l = merge(fm, dd, ll, metric, True)
    old_d, old_l = merge(fm, dd, ll, metric, False)
    want_d, want_l = numpy_merge(dd, ll, metric)
    assert np.array_equal(new_l, want_l)
    assert np.array_equal(new_d, want_d)
    assert np.array_equal(new_l, old_l) and np.array_equal(new_d, old_d)


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("P,nq,k", [(8, 60, 100), (4, 12, 1024), (3, 9, 40)])
def test_merge_of_lists_not_in_label_order(fm, res, metric, P, nq, k):
    # equal distances whose labels do not ascend inside a list: ranked by counting
    rng = np.random.default_rng(k)
    dd, ll = make_lists(rng, P, nq, k, metric, levels=5, fill=0.8, in_label_order=False)
    new_d, new_l = merge(fm, dd, ll, metric, True)
    want_d, want_l = numpy_merge(dd, ll, metric)
    assert np.array_equal(new_l, want_l)
    assert np.array_equal(new_d, want_d)
    old_d, old_l = merge(fm, dd, ll, metric, False)
    assert np.array_equal(new_l, old_l) and np.array_equal(new_d, old_d)


def test_merge_labels_beyond_32_bits(fm, res):
    # labels that differ only above bit 32 among equal distances
    rng = np.random.default_rng(5)
    P, nq, k = 4, 25, 64
    dd, ll = make_lists(rng, P, nq, k, O.METRIC_L2, levels=4, fill=1.0)
    ll = np.where(ll >= 0, (ll % 3) + (ll << 32), -1)
    for p in range(P):          # restore (distance, label) order inside every list
        for q in range(nq):
            order = np.lexsort((ll[p, q], dd[p, q]))
            dd[p, q], ll[p, q] = dd[p, q][order], ll[p, q][order]
    new_d, new_l = merge(fm, dd, ll, O.METRIC_L2, True)
    want_d, want_l = numpy_merge(dd, ll, O.METRIC_L2)
    assert np.array_equal(new_l, want_l)
    assert np.array_equal(new_d, want_d)


def test_merge_interior_empty_slot(fm, res):
    # an empty slot in front of live entries (no shard produces this; the counting path takes it)
    rng = np.random.default_rng(6)
    dd, ll = make_lists(rng, 3, 8, 50, O.METRIC_L2, levels=1000, fill=1.0)
    ll[1, :, 10] = -1
    new_d, new_l = merge(fm, dd, ll, O.METRIC_L2, True)
    want_d, want_l = numpy_merge(dd, ll, O.METRIC_L2)
    assert np.array_equal(new_l, want_l)
    assert np.array_equal(new_d, want_d)


@pytest.mark.parametrize("nb,nq,d,k,storage,metric", [
    (70_000, 200, 64, 100, 1, O.METRIC_L2),              # ~700 candidates per row: 4 warps, 8 words a lane
    (140_000, 64, 32, 1024, 0, O.METRIC_L2),             # ~3000 of 8192: 8 warps
    (263_000, 129, 24, 33, 2, O.METRIC_INNER_PRODUCT),
    (66_000, 40, 100, 500, 1, O.METRIC_INNER_PRODUCT),
    (131_072, 33, 8, 129, 0, O.METRIC_L2),
])
def test_candidate_selection_matches_sorting_kernel(fm, res, nb, nq, d, k, storage, metric):
    rng = np.random.default_rng(nb + k)
    xb = rng.standard_normal((nb, d), dtype=np.float32)
    xb[1000:1400] = xb[17]                      # ties among the k best
    xb[nb // 2::499] = xb[17]
    xq = rng.standard_normal((nq, d), dtype=np.float32)
    xq[::5] = xb[17] + 0.05
    L = fm.lib()
    idx = fm.B200IndexFlat(res, d, metric, storage)
    idx.add(xb)
    idx.set_path(2)
    old_mode = L.b200f_get_selection_mode()
    assert L.b200f_set_selection_mode(1) == 0   # threshold filter wherever a pilot sample exists
    try:
        assert L.b200f_set_rank_select(1) == 0
        D1, I1 = idx.search(xq, k)
        assert L.b200f_set_rank_select(0) == 0
        D0, I0 = idx.search(xq, k)
    finally:
        L.b200f_set_rank_select(1)
        L.b200f_set_selection_mode(old_mode)
    assert np.array_equal(I1, I0), int((I1 != I0).sum())
    assert np.array_equal(D1, D0)
    idx.close()


@pytest.mark.parametrize("k,storage", [(100, 1), (600, 0)])
def test_more_ties_than_the_selection_holds(fm, res, k, storage):
    # thousands of exact copies tie at the k-th key: more candidates at or under it than the
    # register-sorting kernel holds (2048 / 4096), so the row goes to the exact redo pass; the k
    # lowest labels of the tie win
    nb, d, nq = 70_000, 32, 40
    rng = np.random.default_rng(9)
    xb = rng.standard_normal((nb, d), dtype=np.float32)
    xb[5000:10_000] = xb[17]
    xq = rng.standard_normal((nq, d), dtype=np.float32)
    xq[3] = xb[17] + 0.001
    xq[11] = xb[17]
    L = fm.lib()
    idx = fm.B200IndexFlat(res, d, O.METRIC_L2, storage)
    idx.add(xb)
    idx.set_path(2)
    old_mode = L.b200f_get_selection_mode()
    assert L.b200f_set_selection_mode(1) == 0
    try:
        D1, I1 = idx.search(xq, k)
        assert L.b200f_set_rank_select(0) == 0
        D0, I0 = idx.search(xq, k)
    finally:
        L.b200f_set_rank_select(1)
        L.b200f_set_selection_mode(old_mode)
    assert np.array_equal(I1, I0) and np.array_equal(D1, D0)
    want = np.concatenate(([17], np.arange(5000, 5000 + k - 1)))
    assert np.array_equal(I1[3], want) and np.array_equal(I1[11], want)
    idx.close()

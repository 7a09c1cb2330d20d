"""CPU tests of the oracle itself: the C restatement against the numpy one, the
reference's known-answer cases, the committed golden vectors, rounding helpers."""
import os

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "flat_small.npz")


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nv,nq,d,k", [(1000, 10, 32, 5), (1000, 10, 128, 10), (500, 5, 768, 5),
                                       (500, 5, 1536, 5), (100, 1, 32, 1)])
def test_c_matches_numpy(oracle, metric, nv, nq, d, k):
    # shapes of the reference's own cases (tests/test_metal_flat.mm:477-490), seed 42
    xb = H.uniform_pm1(nv, d, 42)
    xq = H.uniform_pm1(nq, d, 43)
    d_c, i_c, d64 = oracle.search(metric, xb, xq, k)
    d_n, i_n, d64n = oracle.numpy_search(metric, xb, xq, k)
    assert np.array_equal(i_c, i_n)
    np.testing.assert_allclose(d64, d64n, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(d_c, d_n, rtol=1e-6)


def test_inline_loops_of_reference(oracle):
    # norm loop tests/test_metal_distance.mm:46-51, L2 :141-147, IP :193-198 in plain python
    xb = H.uniform_pm1(7, 16, 99)
    xq = H.uniform_pm1(3, 16, 77)
    norms = oracle.row_norms(xb)
    for i in range(7):
        s = 0.0
        for j in range(16):
            s += float(xb[i, j]) * float(xb[i, j])
        assert abs(norms[i] - s) < 1e-5
    l2 = oracle.pairwise(O.METRIC_L2, xb, xq)
    ip = oracle.pairwise(O.METRIC_INNER_PRODUCT, xb, xq)
    for i in range(3):
        for j in range(7):
            s = 0.0
            t = 0.0
            for c in range(16):
                df = float(xq[i, c]) - float(xb[j, c])
                s += df * df
                t += float(xq[i, c]) * float(xb[j, c])
            assert abs(l2[i, j] - s) < 1e-12
            assert abs(ip[i, j] - t) < 1e-12


def test_known_answers_empty_and_padding(oracle):
    # empty index -> INFINITY / -1 (tests/test_metal_flat.mm:449-454, src/MetalIndexFlat.mm:328-334)
    xq = H.uniform_pm1(2, 8, 1)
    d, i, _ = oracle.search(O.METRIC_L2, np.zeros((0, 8), np.float32), xq, 5)
    assert np.isposinf(d).all() and (i == -1).all()
    d, i, _ = oracle.search(O.METRIC_INNER_PRODUCT, np.zeros((0, 8), np.float32), xq, 5)
    assert np.isneginf(d).all() and (i == -1).all()
    # k > ntotal tail (src/MetalIndexFlat.mm:387-399)
    xb = H.uniform_pm1(3, 8, 2)
    d, i, _ = oracle.search(O.METRIC_L2, xb, xq, 5)
    assert (i[:, :3] >= 0).all() and (i[:, 3:] == -1).all() and np.isposinf(d[:, 3:]).all()
    # exact neighbour: a query equal to a row has distance 0 and that label first
    d, i, _ = oracle.search(O.METRIC_L2, xb, xb[1:2], 2)
    assert i[0, 0] == 1 and d[0, 0] == 0.0


def test_ties_go_to_lower_label(oracle):
    xb = np.zeros((6, 4), np.float32)
    xb[[1, 3, 4]] = 1.0  # rows 1,3,4 identical; rows 0,2,5 identical
    xq = np.ones((1, 4), np.float32)
    _, i, _ = oracle.search(O.METRIC_L2, xb, xq, 6)
    assert i[0].tolist() == [1, 3, 4, 0, 2, 5]
    _, i, _ = oracle.search(O.METRIC_INNER_PRODUCT, xb, xq, 4)
    assert i[0].tolist() == [1, 3, 4, 0]


def test_rounding_matches_ieee(oracle):
    rng = np.random.default_rng(5)
    x = np.concatenate([
        rng.standard_normal(20000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 20000),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5,
                  np.inf, -np.inf, 1.0009765625, 1.00048828125, 1.001464844], np.float32)])
    got = oracle.round_storage(x, O.STORAGE_F16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).astype(np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # bf16: (bits + 0x7FFF + lsb) >> 16 (src/MetalIndexFlat.mm:231-234) == torch's RNE
    import torch
    want_bf = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    got_bf = oracle.round_storage(x, O.STORAGE_BF16)
    assert np.array_equal(got_bf.view(np.uint32), want_bf.view(np.uint32))
    # fp16 reconstruct tolerance of the reference: 2e-3 abs on uniform(-1,1) (tests/test_metal_flat.mm:259-265)
    u = H.uniform_pm1(100, 128, 42)
    assert np.abs(oracle.round_storage(u, O.STORAGE_F16) - u).max() < 2e-3


def test_merge_equals_unsharded(oracle):
    xb = H.uniform_pm1(900, 24, 3)
    xq = H.uniform_pm1(11, 24, 4)
    for metric in (O.METRIC_L2, O.METRIC_INNER_PRODUCT):
        for k in (1, 7, 400):
            full_d, full_i, _ = oracle.search(metric, xb, xq, k)
            P = 3
            per = 300
            dists, ids, base = [], [], []
            for p in range(P):
                d_, i_, _ = oracle.search(metric, xb[p * per:(p + 1) * per], xq, k)
                dists.append(d_)
                ids.append(i_)
                base.append(p * per)
            md, mi = oracle.merge(metric, np.stack(dists), np.stack(ids), np.array(base))
            assert np.array_equal(mi, full_i)
            np.testing.assert_array_equal(md, full_d)


def test_blas_search_agrees(oracle):
    xb = H.uniform01(5000, 64, 1)
    xq = H.uniform01(33, 64, 2)
    for metric in (O.METRIC_L2, O.METRIC_INNER_PRODUCT):
        d_ref, i_ref, d64 = oracle.search(metric, xb, xq, 10)
        d_b, i_b = oracle.blas_search(metric, xb, xq, 10, block=1024)
        true_d = oracle.rescore(metric, xb, xq, i_b)
        r = oracle.compare_results(metric, d_b, i_b, d64, i_ref, true_d, 1e-4, eps=1e-3)
        assert oracle.passed(r), r


def test_golden_vectors(oracle):
    g = np.load(GOLDEN)
    for name in ("l2", "ip"):
        metric = O.METRIC_L2 if name == "l2" else O.METRIC_INNER_PRODUCT
        d, i, _ = oracle.search(metric, g["xb"], g["xq"], int(g["k"]))
        assert np.array_equal(i, g[name + "_labels"])
        np.testing.assert_allclose(d, g[name + "_dist"], rtol=1e-6)
    for s, name in ((O.STORAGE_F16, "f16"), (O.STORAGE_BF16, "bf16")):
        assert np.array_equal(oracle.to_bits16(g["xb"][:8], s), g[name + "_bits"])


def test_comparator_flags_errors(oracle):
    xb = H.uniform_pm1(200, 16, 8)
    xq = H.uniform_pm1(4, 16, 9)
    d, i, d64 = oracle.search(O.METRIC_L2, xb, xq, 5)
    ok = oracle.compare_results(O.METRIC_L2, d, i, d64, i, oracle.rescore(O.METRIC_L2, xb, xq, i), 1e-4)
    assert oracle.passed(ok)
    bad_i = i.copy()
    bad_i[0, 0] = (i[0, 0] + 57) % 200
    r = oracle.compare_results(O.METRIC_L2, d, bad_i, d64, i, oracle.rescore(O.METRIC_L2, xb, xq, bad_i), 1e-4)
    assert not oracle.passed(r) and r["label_bad"] >= 1
    bad_d = d.copy()
    bad_d[1, 2] *= 1.01
    r = oracle.compare_results(O.METRIC_L2, bad_d, i, d64, i, oracle.rescore(O.METRIC_L2, xb, xq, i), 1e-4)
    assert r["dist"] == 1
    dup = i.copy()
    dup[2, 1] = dup[2, 0]
    r = oracle.compare_results(O.METRIC_L2, d, dup, d64, i, oracle.rescore(O.METRIC_L2, xb, xq, dup), 1e-4)
    assert r["duplicates"] == 1

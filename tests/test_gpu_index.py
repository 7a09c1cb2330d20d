"""GPU parity tests of the plugin surface through the handle-based C-ABI, modelled on
tests/test_metal_flat.mm of the reference (same cases, plus the gaps it leaves:
k > 10, BF16, fused path, k > ntotal, growth, ties, ranks 2..k)."""
import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

PATH_SCAN, PATH_TENSOR = 1, 2


def make_index(fm, res, xb, metric, storage, path=0):
    idx = fm.B200IndexFlat(res, xb.shape[1], metric, storage)
    idx.add(xb)
    if path:
        idx.set_path(path)
    return idx


# (nv, nq, d, k) of the reference's test_flat_l2 (tests/test_metal_flat.mm:477-490)
REFERENCE_CASES = [(1000, 10, 32, 5), (1000, 10, 128, 10), (500, 5, 768, 5), (500, 5, 1536, 5), (100, 1, 32, 1)]


@pytest.mark.parametrize("path", [PATH_SCAN, PATH_TENSOR])
@pytest.mark.parametrize("storage", [0, 1, 2])
@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nv,nq,d,k", REFERENCE_CASES)
def test_flat_reference_cases(fm, res, path, storage, metric, nv, nq, d, k):
    xb = H.uniform_pm1(nv, d, 42)
    xq = H.uniform_pm1(nq, d, 43)
    idx = make_index(fm, res, xb, metric, storage, path)
    assert idx.ntotal == nv
    D, I = idx.search(xq, k)
    H.check_against_oracle(metric, storage, path == PATH_TENSOR, xb, xq, k, D, I)
    # the reference's own assertion: top-1 labels equal CPU results (tests/test_metal_flat.mm:52-58)
    _, ref_i, ref_d = O.search(metric, *H.effective_operands(storage, path == PATH_TENSOR, xb, xq), min(2, nv))
    if ref_i.shape[1] == 2:   # except where rank 1 and rank 2 are closer than fp32 accumulation noise
        clear = np.abs(ref_d[:, 1] - ref_d[:, 0]) > 1e-4 * np.maximum(np.abs(ref_d[:, 0]), 1e-3)
    else:
        clear = np.ones(nq, dtype=bool)
    assert np.array_equal(np.asarray(I)[clear, 0], ref_i[clear, 0])
    idx.close()


@pytest.mark.parametrize("path", [0, PATH_SCAN, PATH_TENSOR])
@pytest.mark.parametrize("nv,nq,d,k,storage,metric", [
    (3000, 33, 96, 32, 0, O.METRIC_L2),
    (3000, 130, 64, 17, 2, O.METRIC_L2),
    (2500, 7, 200, 32, 1, O.METRIC_INNER_PRODUCT),
    (777, 3, 70, 20, 2, O.METRIC_INNER_PRODUCT),   # d not a multiple of 8: padded pitch
    (1500, 2, 33, 9, 0, O.METRIC_L2),
])
def test_flat_more_shapes(fm, res, path, nv, nq, d, k, storage, metric):
    xb = H.uniform_pm1(nv, d, 7)
    xq = H.uniform_pm1(nq, d, 8)
    idx = make_index(fm, res, xb, metric, storage, path)
    D, I = idx.search(xq, k)
    # automatic choice: scan up to 4 queries on fp32 rows and up to 8 on 16-bit rows (these shards
    # are too small for the streaming kernel, so the scan multiplies unrounded fp32 queries)
    tensor = (path == PATH_TENSOR) or (path == 0 and nq > (4 if storage == 0 else 8))
    H.check_against_oracle(metric, storage, tensor, xb, xq, k, D, I)
    idx.close()


@pytest.mark.parametrize("storage", [1, 2])
@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nv,nq,d,k", [(60_000, 5, 64, 10), (60_000, 8, 128, 32), (60_000, 7, 200, 3), (2_000, 8, 64, 10)])
def test_automatic_path_five_to_eight_queries(fm, res, storage, metric, nv, nq, d, k):
    # 16-bit rows, 5 - 8 queries: one pass of the streaming scan on large shards (queries rounded
    # to the storage format, like the tensor path), two passes of the plain scan on small ones
    xb = H.uniform_pm1(nv, d, 71)
    xq = H.uniform_pm1(nq, d, 72)
    idx = make_index(fm, res, xb, metric, storage)
    D, I = idx.search(xq, k)
    H.check_against_oracle(metric, storage, nv >= 20_000, xb, xq, k, D, I)
    # same labels as the tensor path up to ties inside the tolerance: compare with the oracle only
    idx.close()


@pytest.mark.parametrize("path", [PATH_SCAN, PATH_TENSOR])
@pytest.mark.parametrize("k", [33, 100, 1024, 4096])
@pytest.mark.parametrize("storage,metric", [(0, O.METRIC_L2), (1, O.METRIC_INNER_PRODUCT)])
def test_large_k(fm, res, select_mode, path, k, storage, metric):
    # block_select range of the reference (k up to 4096, src/MetalSelect.mm:65-70), which its
    # tests never check
    nv, nq, d = 6000, 6, 48
    xb = H.uniform_pm1(nv, d, 11)
    xq = H.uniform_pm1(nq, d, 12)
    idx = make_index(fm, res, xb, metric, storage, path)
    D, I = idx.search(xq, k)
    H.check_against_oracle(metric, storage, path == PATH_TENSOR, xb, xq, k, D, I)
    idx.close()


@pytest.mark.parametrize("path", [PATH_SCAN, PATH_TENSOR])
@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("k", [5, 40])
def test_k_larger_than_ntotal(fm, res, path, metric, k):
    # tail (+/-INF, -1): src/MetalIndexFlat.mm:387-399
    xb = H.uniform_pm1(3, 16, 1)
    xq = H.uniform_pm1(6, 16, 2)
    idx = make_index(fm, res, xb, metric, 0, path)
    D, I = idx.search(xq, k)
    assert (I[:, :3] >= 0).all() and (I[:, 3:] == -1).all()
    assert (np.isposinf(D[:, 3:]) if metric == O.METRIC_L2 else np.isneginf(D[:, 3:])).all()
    H.check_against_oracle(metric, 0, path == PATH_TENSOR, xb, xq, k, D, I)
    idx.close()


@pytest.mark.parametrize("path", [PATH_SCAN, PATH_TENSOR])
def test_ties_lower_label_first(fm, res, path):
    rng = np.random.default_rng(0)
    base = rng.integers(-3, 4, size=(40, 16)).astype(np.float32)  # exactly representable everywhere
    xb = np.concatenate([base] * 25)  # every row appears 25 times
    xq = base[:9].copy()
    for storage in (0, 1, 2):
        for metric in (O.METRIC_L2, O.METRIC_INNER_PRODUCT):
            idx = make_index(fm, res, xb, metric, storage, path)
            D, I = idx.search(xq, 32)
            _, ref_i, ref_d = O.search(metric, xb, xq, 32)
            assert np.array_equal(I, ref_i)
            np.testing.assert_allclose(D, ref_d, rtol=1e-6, atol=1e-6)
            idx.close()


@pytest.mark.parametrize("k", [10, 32, 100])
def test_ties_lower_label_first_large_shard(fm, res, select_mode, k):
    # shard large enough for the threshold filter: every row appears three times, values are
    # small integers (exact in every storage format), so equal keys are common inside the k best
    rng = np.random.default_rng(5)
    base = rng.integers(-3, 4, size=(25_000, 24)).astype(np.float32)
    xb = np.concatenate([base, base, base])
    xq = base[rng.permutation(25_000)[:150]].copy()
    for storage in (0, 2):
        for metric in (O.METRIC_L2, O.METRIC_INNER_PRODUCT):
            idx = make_index(fm, res, xb, metric, storage, PATH_TENSOR)
            D, I = idx.search(xq, k)
            _, ref_i, ref_d = O.search(metric, xb, xq, k)
            assert np.array_equal(I, ref_i)
            np.testing.assert_allclose(D, ref_d, rtol=1e-6, atol=1e-6)
            idx.close()


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("storage", [0, 1, 2])
@pytest.mark.parametrize("nv,nq,d,k", [(40_000, 1, 64, 10), (40_000, 4, 128, 32), (40_001, 3, 200, 7),
                                       (5_000, 2, 1536, 32), (150_000, 1, 128, 10), (40_000, 1, 100, 1)])
def test_scan_streaming_pipeline(fm, res, metric, storage, nv, nq, d, k):
    # shards large enough for the streaming ring of the scan path (small ones use the plain
    # kernel); with 16-bit storage that kernel multiplies queries rounded to the storage format
    xb = H.uniform_pm1(nv, d, 17)
    xb[nv // 2::997] = xb[5]  # a few exact duplicates: ties by label
    xq = H.uniform_pm1(nq, d, 18)
    idx = make_index(fm, res, xb, metric, storage, PATH_SCAN)
    D, I = idx.search(xq, k)
    H.check_against_oracle(metric, storage, storage != 0, xb, xq, k, D, I)
    idx.close()


@pytest.mark.parametrize("k,storage,metric", [(100, 1, O.METRIC_INNER_PRODUCT), (1024, 0, O.METRIC_L2)])
def test_large_k_many_queries_deterministic(fm, res, select_mode, k, storage, metric):
    # more queries than selection CTAs (each CTA walks several rows) and enough columns for
    # repeated buffer compaction; two runs must agree bit for bit and match the oracle
    nv, nq, d = 40_000, 5_000, 32
    xb = H.gaussian(nv, d, 21)
    xq = H.gaussian(nq, d, 22)
    idx = make_index(fm, res, xb, metric, storage, PATH_TENSOR)
    D1, I1 = idx.search(xq, k)
    D2, I2 = idx.search(xq, k)
    assert np.array_equal(I1, I2) and np.array_equal(D1, D2)
    H.check_against_oracle(metric, storage, True, xb, xq, k, D1, I1, loose=False)
    idx.close()

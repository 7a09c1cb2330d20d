"""GPU tests of the MetalIndexFlat contract other than search parity: reset,
reconstruct, async tokens, empty index, growth, error behaviour
(tests/test_metal_flat.mm:132-462 of the reference)."""
import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu


def test_reset(fm, res):
    # tests/test_metal_flat.mm:178-196: 100 -> 0 -> 50
    idx = fm.B200IndexFlat(res, 32, O.METRIC_L2, 0)
    idx.add(H.uniform_pm1(100, 32, 1))
    assert idx.ntotal == 100
    idx.reset()
    assert idx.ntotal == 0
    xb = H.uniform_pm1(50, 32, 2)
    idx.add(xb)
    assert idx.ntotal == 50
    D, I = idx.search(xb[:3], 1)
    assert I[:, 0].tolist() == [0, 1, 2]
    idx.close()


@pytest.mark.parametrize("storage", [0, 1, 2])
def test_reconstruct(fm, res, storage):
    # fp32 bit-exact (tests/test_metal_flat.mm:198-221); fp16 within 2e-3 abs (:259-265)
    xb = H.uniform_pm1(10, 64, 5)
    idx = fm.B200IndexFlat(res, 64, O.METRIC_L2, storage)
    idx.add(xb)
    want = O.round_storage(xb, storage)
    for key in (0, 3, 9):
        r = idx.reconstruct(key)
        assert np.array_equal(r.view(np.uint32), want[key].view(np.uint32))
        if storage == 0:
            assert np.array_equal(r, xb[key])
        elif storage == 1:
            assert np.abs(r - xb[key]).max() < 2e-3
    assert np.array_equal(idx.reconstruct_n(2, 5), want[2:7])
    for bad in (-1, 10, 1 << 40):
        with pytest.raises(fm.B200Error) as e:
            idx.reconstruct(bad)
        assert e.value.status == 8  # B200F_ERR_RANGE (src/MetalIndexFlat.mm:509-511 throws)
    idx.close()


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
def test_empty_index_and_empty_query(fm, res, metric):
    # src/MetalIndexFlat.mm:328-334; tests/test_metal_flat.mm:439-462
    idx = fm.B200IndexFlat(res, 16, metric, 0)
    xq = H.uniform_pm1(3, 16, 1)
    D, I = idx.search(xq, 5)
    assert (I == -1).all()
    assert (np.isposinf(D) if metric == O.METRIC_L2 else np.isneginf(D)).all()
    D0, I0 = idx.search(np.zeros((0, 16), np.float32), 5)
    assert D0.shape == (0, 5)
    # async on the empty index and with n == 0
    d = np.zeros((3, 5), np.float32)
    i = np.zeros((3, 5), np.int64)
    t = idx.search_async(xq, 5, d, i)
    t.wait()
    assert (i == -1).all()
    t0 = idx.search_async(np.zeros((0, 16), np.float32), 5, np.zeros((0, 5), np.float32), np.zeros((0, 5), np.int64))
    assert t0.is_ready()
    t0.wait()
    idx.close()


def test_search_argument_errors(fm, res):
    idx = fm.B200IndexFlat(res, 8, O.METRIC_L2, 0)
    idx.add(H.uniform_pm1(20, 8, 1))
    xq = H.uniform_pm1(2, 8, 2)
    with pytest.raises(fm.B200Error) as e:   # k must be > 0 (src/MetalIndexFlat.mm:321)
        idx.search(xq, 0)
    assert e.value.status == 1
    with pytest.raises(fm.B200Error) as e:   # k above the selection limit (src/MetalSelect.mm:65-70)
        idx.search(xq, 4097)
    assert e.value.status == 2
    D, I = idx.search(xq, 4096)              # the limit itself is served
    assert (I[:, :20] >= 0).all() and (I[:, 20:] == -1).all()
    idx.close()


def test_search_async_matches_sync(fm, res):
    # tests/test_metal_flat.mm:309-347: async == sync bit-exact
    xb = H.uniform_pm1(1000, 128, 42)
    xq = H.uniform_pm1(10, 128, 43)
    idx = fm.B200IndexFlat(res, 128, O.METRIC_L2, 0)
    idx.add(xb)
    D, I = idx.search(xq, 10)
    d = np.zeros_like(D)
    i = np.zeros_like(I)
    t = idx.search_async(xq, 10, d, i)
    t.wait()
    assert np.array_equal(d, D) and np.array_equal(i, I)
    idx.close()


def test_search_async_multiple_in_flight(fm, res):
    # tests/test_metal_flat.mm:349-401: 3 tokens, waited in reverse order
    xb = H.uniform_pm1(2000, 64, 1)
    idx = fm.B200IndexFlat(res, 64, O.METRIC_L2, 1)
    idx.add(xb)
    qs = [H.uniform_pm1(5, 64, 10 + j) for j in range(3)]
    sync = [idx.search(q, 5) for q in qs]
    outs = [(np.zeros((5, 5), np.float32), np.zeros((5, 5), np.int64)) for _ in range(3)]
    toks = [idx.search_async(q.copy(), 5, o[0], o[1]) for q, o in zip(qs, outs)]
    for j in (2, 1, 0):
        toks[j].wait()
        assert np.array_equal(outs[j][0], sync[j][0]) and np.array_equal(outs[j][1], sync[j][1])
    idx.close()


def test_search_async_is_ready(fm, res):
    # tests/test_metal_flat.mm:403-437
    import time
    xb = H.uniform_pm1(1000, 32, 3)
    idx = fm.B200IndexFlat(res, 32, O.METRIC_L2, 0)
    idx.add(xb)
    d = np.zeros((1, 3), np.float32)
    i = np.zeros((1, 3), np.int64)
    t = idx.search_async(H.uniform_pm1(1, 32, 4), 3, d, i)
    t0 = time.time()
    while not t.is_ready():
        assert time.time() - t0 < 30
    t.wait()
    assert ((i >= 0) & (i < 1000)).all()
    t.close()
    idx.close()


@pytest.fixture(params=["in_place", "copying"])
def growth_mode(request):
    # in_place: rows are mapped into a reserved address range as the index grows (no copies);
    # copying: plain allocations with the reference's allocate-copy-free growth
    return request.param


@pytest.mark.parametrize("storage", [0, 2])
@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
def test_growth_over_many_adds(fm, res, growth_mode, storage, metric):
    # capacity rule max(new, 2*cap, 1024) (src/MetalIndexFlat.mm:196-208)
    d = 40
    xb = H.uniform_pm1(5000, d, 9)
    idx = fm.B200IndexFlat(res, d, metric, storage)
    idx.set_growth_mode(1 if growth_mode == "copying" else 0)
    base0 = None
    pos = 0
    for n in (1, 7, 1000, 30, 2500, 1462):
        idx.add(xb[pos:pos + n])
        pos += n
        if base0 is None:
            base0 = idx.device_rows()
        elif growth_mode == "in_place":
            assert idx.device_rows() == base0   # the array never moves
    assert pos == 5000 and idx.ntotal == 5000
    assert np.array_equal(idx.reconstruct_n(0, 5000), O.round_storage(xb, storage))
    xq = H.uniform_pm1(9, d, 10)
    D, I = idx.search(xq, 10)
    H.check_against_oracle(metric, storage, True, xb, xq, 10, D, I)
    # reset drops the storage; the index can be filled again
    idx.reset()
    assert idx.ntotal == 0
    idx.add(xb[:1500])
    D, I = idx.search(xq, 10)
    H.check_against_oracle(metric, storage, True, xb[:1500], xq, 10, D, I)
    idx.close()


def test_large_growth_in_place_keeps_rows(fm, res, growth_mode):
    # 300,000 rows of d = 256 in bf16 (158 MB) added in uneven pieces, with reserve() in the middle
    d = 256
    xb = H.gaussian(300_000, d, 33, scale=0.05)
    idx = fm.B200IndexFlat(res, d, O.METRIC_L2, 2)
    idx.set_growth_mode(1 if growth_mode == "copying" else 0)
    idx.add(xb[:10])
    idx.add(xb[10:70_000])
    idx.reserve(250_000)
    idx.add(xb[70_000:240_000])
    idx.add(xb[240_000:])
    assert idx.ntotal == 300_000
    back = idx.reconstruct_n(0, 300_000)
    assert np.array_equal(back, O.round_storage(xb, 2))
    xq = H.gaussian(33, d, 34, scale=0.05)
    D, I = idx.search(xq, 10)
    H.check_against_oracle(O.METRIC_L2, 2, True, xb, xq, 10, D, I)
    idx.close()


def test_device_pointers_in_and_out(fm, res):
    import torch
    xb = H.uniform_pm1(3000, 64, 21)
    xq = H.uniform_pm1(40, 64, 22)
    idx = fm.B200IndexFlat(res, 64, O.METRIC_L2, 2)
    idx.add(torch.from_numpy(xb).cuda())          # device-resident add
    Dh, Ih = idx.search(xq, 10)                   # host in / host out
    Dd, Id = idx.search(torch.from_numpy(xq).cuda(), 10)  # device in / device out
    assert np.array_equal(Dd.cpu().numpy(), Dh) and np.array_equal(Id.cpu().numpy(), Ih)
    H.check_against_oracle(O.METRIC_L2, 2, True, xb, xq, 10, Dh, Ih)
    idx.close()


def test_capabilities(fm, res):
    caps = fm.device_caps(0)
    assert caps["supported"] == 1 and caps["cc_major"] == 10 and caps["sm_count"] > 0
    assert caps["max_smem_per_block"] >= 227 * 1024

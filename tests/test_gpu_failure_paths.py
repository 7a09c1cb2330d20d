"""Error paths of the device code, exercised without any fault, trap or hang: a bounded wait
that is made to run out (a barrier nothing signals, limit of about a millisecond), the status
word it leaves, the status code the host maps it to, and the debug canaries around the scratch
slices."""
import ctypes

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

LIMIT = 2_000_000   # SM clocks: about a millisecond


def test_bounded_wait_expires_and_sets_the_status_word(fm, res):
    status = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    fm.abi.check_op(fm.lib().b200f_debug_wait_expiry(ctypes.c_void_p(status.data_ptr()), LIMIT, st), "wait_expiry")
    t1.record()
    torch.cuda.synchronize()                      # the kernel returned by itself
    assert status.cpu().tolist()[0] == 1          # kDevErrBarrierWait
    assert 0.2 < t0.elapsed_time(t1) < 200.0      # gave up after about the limit, not after a second
    # bad limits are refused on the host
    assert fm.lib().b200f_debug_wait_expiry(ctypes.c_void_p(status.data_ptr()), 0, st) == fm.abi.ERR_BAD_ARG
    assert fm.lib().b200f_debug_wait_expiry(None, LIMIT, st) == fm.abi.ERR_BAD_ARG


def test_expired_wait_maps_to_device_wait_and_the_next_search_is_fine(fm, res):
    xb = H.uniform_pm1(3000, 64, 1)
    xq = H.uniform_pm1(20, 64, 2)
    idx = fm.B200IndexFlat(res, 64, O.METRIC_L2, 2)
    idx.add(xb)
    D0, I0 = idx.search(xq, 10)
    fm.abi.check(fm.lib().b200f_index_debug_wait_expiry(idx._h, LIMIT), "debug_wait_expiry")
    with pytest.raises(fm.B200Error) as e:
        idx.synchronize()
    assert e.value.status == fm.abi.ERR_DEVICE_WAIT
    assert "device status 1" in str(e.value)
    # same stream, same index: the next search clears the word and gives the same result
    D1, I1 = idx.search(xq, 10)
    assert np.array_equal(I1, I0) and np.array_equal(D1, D0)
    idx.synchronize()
    idx.close()


def test_canary_checker_selftest(fm, res):
    buf = torch.zeros(8192, dtype=torch.uint8, device="cuda:0")
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    L = fm.lib()
    status = torch.zeros(4, dtype=torch.int32, device="cuda:0")
    fm.abi.check_op(L.b200f_debug_canary_selftest(ctypes.c_void_p(buf.data_ptr()), 8192, 0,
                                                  ctypes.c_void_p(status.data_ptr()), st), "selftest")
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0, 0, 0]
    fm.abi.check_op(L.b200f_debug_canary_selftest(ctypes.c_void_p(buf.data_ptr()), 8192, 1,
                                                  ctypes.c_void_p(status.data_ptr()), st), "selftest")
    torch.cuda.synchronize()
    got = status.cpu().tolist()
    assert got[0] == 8 and got[2] == 2            # kDevErrCanary, second guard


@pytest.fixture
def canaries(fm):
    assert fm.lib().b200f_set_debug_canaries(1) == 0
    yield
    assert fm.lib().b200f_set_debug_canaries(0) == 0


@pytest.mark.parametrize("nq,k,storage,metric", [(3, 10, 1, O.METRIC_L2), (3, 100, 0, O.METRIC_L2),
                                                 (200, 32, 2, O.METRIC_L2), (150, 100, 1, O.METRIC_INNER_PRODUCT),
                                                 (130, 1024, 0, O.METRIC_L2), (40, 2000, 2, O.METRIC_INNER_PRODUCT)])
def test_no_kernel_writes_past_its_scratch_slice(fm, res, canaries, select_mode, nq, k, storage, metric):
    # every slice of the search scratch is followed by a guard that is compared after the search;
    # a guard that changed would surface as status bit 8 -> B200F_ERR_DEVICE_CHECK
    nb, d = 70_000, 72
    xb = H.gaussian(nb, d, 5, scale=0.3)
    xq = H.gaussian(nq, d, 6, scale=0.3)
    idx = fm.B200IndexFlat(res, d, metric, storage)
    idx.add(xb)
    D, I = idx.search(xq, k)
    assert idx.last_device_status == 0
    if nq * nb <= 15_000_000:
        tensor = nq > (4 if storage == 0 else 8)
        H.check_against_oracle(metric, storage, tensor, xb, xq, k, D, I, loose=False)
    idx.close()


@pytest.mark.parametrize("storage,metric,k", [(1, O.METRIC_L2, 10), (0, O.METRIC_INNER_PRODUCT, 32), (2, O.METRIC_L2, 100)])
def test_graph_replay_equals_call_by_call(fm, res, storage, metric, k):
    # searches of <= 8 queries with host buffers: first call eager, second captured, later replayed
    nb, d = 60_000, 96
    xb = H.uniform_pm1(nb, d, 7)
    idx = fm.B200IndexFlat(res, d, metric, storage)
    idx.add(xb[:50_000])
    plain = fm.B200IndexFlat(res, d, metric, storage)
    plain.set_use_graphs(False)
    plain.add(xb[:50_000])
    for nq in (1, 4, 1, 1, 4, 8, 1):
        for rep in range(3):
            xq = H.uniform_pm1(nq, d, 100 + 10 * nq + rep)
            D, I = idx.search(xq, k)
            Dp, Ip = plain.search(xq, k)
            assert np.array_equal(I, Ip) and np.array_equal(D, Dp), (nq, rep)
    # the index changes: graphs captured for the old rows must not be replayed
    idx.add(xb[50_000:])
    plain.add(xb[50_000:])
    xq = H.uniform_pm1(1, d, 999)
    for rep in range(3):
        D, I = idx.search(xq, k)
        Dp, Ip = plain.search(xq, k)
        assert np.array_equal(I, Ip) and np.array_equal(D, Dp)
    tensor = False if storage == 0 else True   # 16-bit rows, shard large enough: the streaming kernel rounds the query
    H.check_against_oracle(metric, storage, tensor, xb, xq, k, D, I, loose=True, strict=False)
    idx.set_label_base(1000)
    D2, I2 = idx.search(xq, k)
    assert np.array_equal(I2, I + 1000)
    idx.close()
    plain.close()


def test_ingest_pipeline_pinned_and_pageable(fm, res):
    # three 32 MiB chunks and a ragged tail through the double-buffered add, from pageable and
    # from pinned memory; rows read back through the pipelined reconstruct_n, into both kinds
    n, d = 230_000, 100
    xb = H.gaussian(n, d, 11)
    pinned = torch.empty((n, d), dtype=torch.float32, pin_memory=True)
    pinned.copy_(torch.from_numpy(xb))
    want = O.round_storage(xb, 1)
    for src in (xb, pinned.numpy()):
        idx = fm.B200IndexFlat(res, d, O.METRIC_L2, 1)
        idx.add(src[:200_000])
        idx.add(src[200_000:])
        assert idx.ntotal == n
        assert np.array_equal(idx.reconstruct_n(0, n), want)
        out_pin = torch.empty((n - 5, d), dtype=torch.float32, pin_memory=True)
        idx.reconstruct_n(5, n - 5, out_pin.numpy())
        assert np.array_equal(out_pin.numpy(), want[5:])
        idx.close()


def test_many_async_tokens_in_flight(fm, res):
    # sixteen tokens of different sizes queued back to back: uploads, kernels and downloads of
    # neighbouring tokens overlap on the three streams; every token must hold exactly what the
    # synchronous search gives for its queries, whatever the order they are waited for in
    nb, d = 120_000, 128
    xb = H.gaussian(nb, d, 3, scale=0.05)
    idx = fm.B200IndexFlat(res, d, O.METRIC_L2, 2)
    idx.add(xb)
    sizes = [1, 700, 3, 2000, 64, 9, 1500, 2, 300, 5000, 1, 17, 1024, 8, 256, 33]
    k = 10
    queries = [H.gaussian(n, d, 100 + i, scale=0.05) for i, n in enumerate(sizes)]
    outs = [(np.full((n, k), np.nan, np.float32), np.full((n, k), -7, np.int64)) for n in sizes]
    for rounds in range(2):                      # the second round runs entirely on recycled buffers
        tokens = [idx.search_async(q, k, o[0], o[1]) for q, o in zip(queries, outs)]
        for t in reversed(tokens):
            t.wait()
        for q, (D, I) in zip(queries, outs):
            Ds, Is = idx.search(q, k)
            assert np.array_equal(I, Is) and np.array_equal(D, Ds)
            D.fill(np.nan)
            I.fill(-7)
    idx.close()

"""The sharded index classes (C++ B200ShardedIndexFlat through the C-ABI): block-cyclic
placement, label mapping, query slicing, candidate exchange and merge.  On one GPU several
shards share the device and exchange with device copies; with two or more GPUs the same tests
run over NCCL, in one process (MultiGpuIndexFlat) and with one process per GPU
(ShardedIndexFlat)."""
import os
import socket
import sys

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def assert_same(D, I, Df, If):
    """Sharded against unsharded: distances bit-equal; labels equal, except that rows whose final
    fp32 distances are EQUAL may swap places (the single index orders by the raw key, which can
    still differ in the last bit before ||q||^2 is added; the merge sees only the distance and
    orders equal ones by label)."""
    D, I, Df, If = (np.asarray(a) for a in (D, I, Df, If))
    assert np.array_equal(D, Df)
    for q, j in np.argwhere(I != If):
        run = np.flatnonzero(Df[q] == Df[q, j])
        assert run.size > 1 and sorted(I[q, run].tolist()) == sorted(If[q, run].tolist()), (q, j)


def unsharded(fm, res, xb, xq, k, metric, storage):
    idx = fm.B200IndexFlat(res, xb.shape[1], metric, storage)
    idx.add(xb)
    D, I = idx.search(xq, k)
    idx.close()
    return D, I


@pytest.mark.parametrize("shards", [2, 5])
@pytest.mark.parametrize("k,storage,metric,nq", [(32, 2, O.METRIC_L2, 64), (100, 1, O.METRIC_INNER_PRODUCT, 64),
                                                 (10, 0, O.METRIC_L2, 3), (1500, 2, O.METRIC_L2, 9)])
def test_shards_on_one_gpu_equal_unsharded(fm, res, shards, k, storage, metric, nq):
    nb, d = 30_000, 64
    xb = H.gaussian(nb, d, 31, scale=0.05)
    xb[500:560] = xb[20_000:20_060]          # exact duplicates on different shards: ties by label
    xq = H.gaussian(nq, d, 32, scale=0.05)
    Df, If = unsharded(fm, res, xb, xq, k, metric, storage)
    idx = fm.MultiGpuIndexFlat([res] * shards, d, metric, storage, block_rows=1000)
    assert idx.num_shards == shards
    idx.add(xb[:7])                           # a partial block
    idx.add(xb[7:12_345])
    idx.add(xb[12_345:])
    assert idx.ntotal == nb
    D, I = idx.search(xq, k)                  # host queries, host results
    assert_same(D, I, Df, If)
    Dd, Id = idx.search(torch.from_numpy(xq).cuda(), k)   # device in / device out
    assert_same(Dd.cpu().numpy(), Id.cpu().numpy(), Df, If)
    for key in (0, 999, 1000, 1001, 12_344, 12_345, nb - 1):
        assert np.array_equal(idx.reconstruct(key), O.round_storage(xb[key:key + 1], storage)[0])
    with pytest.raises(fm.B200Error) as e:
        idx.reconstruct(nb)
    assert e.value.status == fm.abi.ERR_RANGE
    idx.reset()
    assert idx.ntotal == 0
    D0, I0 = idx.search(xq, 5)
    assert (I0 == -1).all()
    idx.close()


def test_query_batches_and_slices(fm, res):
    # more queries than one launch takes (k <= 1024: 16384), a query count that does not divide by
    # the number of parts, and d * 4 bytes not a multiple of 16 (slices are then not exchanged)
    nb = 9_000
    for d, nq, k in ((33, 17_000, 5), (20, 101, 40)):
        xb = H.uniform_pm1(nb, d, 3)
        xq = H.uniform_pm1(nq, d, 4)
        Df, If = unsharded(fm, res, xb, xq, k, O.METRIC_L2, 0)
        idx = fm.MultiGpuIndexFlat([res] * 3, d, O.METRIC_L2, 0, block_rows=512)
        idx.add(xb)
        D, I = idx.search(xq, k)
        assert_same(D, I, Df, If)
        idx.close()


def test_rank_form_world_one(fm, res):
    xb = H.gaussian(20_000, 64, 41, scale=0.05)
    xq = H.gaussian(50, 64, 42, scale=0.05)
    idx = fm.B200IndexFlat(res, 64, O.METRIC_L2, 2)
    idx.add(xb)
    idx.set_label_base(7)
    D, I = idx.search(xq, 10)
    sh = fm.ShardedIndexFlat(idx, 0, 1)
    D1, I1 = sh.search(xq, 10)
    assert np.array_equal(I1, I) and np.array_equal(D1, D) and I1.min() >= 7
    assert sh.search(xq, 10, want_result=False) == (None, None)
    sh.close()
    idx.close()


needs_two_gpus = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two or more GPUs")


@needs_two_gpus
@pytest.mark.parametrize("k,storage,metric", [(32, 2, O.METRIC_L2), (100, 1, O.METRIC_INNER_PRODUCT)])
def test_one_process_several_gpus(fm, res, k, storage, metric):
    n = torch.cuda.device_count()
    rs = [res] + [fm.StandardB200Resources(i) for i in range(1, n)]
    nb, d, nq = 200_000, 128, 300
    xb = H.gaussian(nb, d, 51, scale=0.05)
    xq = H.gaussian(nq, d, 52, scale=0.05)
    Df, If = unsharded(fm, res, xb, xq, k, metric, storage)
    idx = fm.MultiGpuIndexFlat(rs, d, metric, storage, block_rows=4096)
    idx.add(xb[:100_000])
    idx.add(xb[100_000:])
    for _ in range(2):
        D, I = idx.search(xq, k)
        assert_same(D, I, Df, If)
    Dd, Id = idx.search(torch.from_numpy(xq).cuda(0), k)
    assert_same(Dd.cpu().numpy(), Id.cpu().numpy(), Df, If)
    idx.close()
    for r in rs[1:]:
        r.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_worker(rank, world, port, out_dir):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    from test_gpu_sharded import assert_same
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch.distributed as dist

    import faiss_metal_b200 as fm
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)   # only carries the communicator id
    try:
        nb, d, nq = 120_000, 96, 130
        xb = H.gaussian(nb, d, 61, scale=0.05)
        xq = H.gaussian(nq, d, 62, scale=0.05)
        res = fm.StandardB200Resources(rank)
        lo, hi = fm.shard_range(nb, rank, world)
        for k, storage, metric in ((32, 2, O.METRIC_L2), (100, 1, O.METRIC_INNER_PRODUCT), (10, 1, O.METRIC_L2)):
            idx = fm.B200IndexFlat(res, d, metric, storage)
            idx.add(xb[lo:hi])
            idx.set_label_base(lo)
            sh = fm.ShardedIndexFlat(idx, rank, world)
            full = None
            if rank == 0:
                full = fm.B200IndexFlat(res, d, metric, storage)
                full.set_use_graphs(False)
                full.add(xb)
            # a batch, then single queries: the second single query captures the whole call
            # (exchange included) into a graph, the following ones replay it
            for first, n_queries in ((0, nq), (0, 1), (1, 1), (2, 1), (3, 1), (0, 3), (3, 3), (6, 3)):
                q = xq[first:first + n_queries]
                D, I = sh.search(q, k, want_result=(rank == 0))          # host queries
                Dd, Id = sh.search_device(torch.from_numpy(q).cuda(), k)  # device queries, every rank merges
                if rank == 0:
                    Df, If = full.search(q, k)
                    assert_same(D, I, Df, If)
                    assert_same(Dd.cpu().numpy(), Id.cpu().numpy(), Df, If)
                else:
                    assert D is None and I is None
            enq, wait = sh.read_trace()
            assert enq.size == 0                       # tracing is off unless asked for
            sh.trace(True)
            sh.search(xq[:1], k, want_result=(rank == 0))
            enq, wait = sh.read_trace()
            assert enq.size == 1 and enq[0] > 0 and wait[0] >= 0
            sh.trace(False)
            if full is not None:
                full.close()
            sh.close()
            idx.close()
        res.close()
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@needs_two_gpus
def test_one_process_per_gpu(tmp_path):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    mp.spawn(_rank_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / ("ok%d" % r)).exists()

"""CPU tests (gloo, world_size 2 and 3) of the multi-GPU host logic: shard ranges, label
bases, candidate packing, the all-gather exchange and the merge order.  The shard-local
search is played by the CPU oracle here (there is no GPU in this test), the device merge
by the oracle's merge."""
import os
import socket
import sys

import numpy as np
import pytest

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


class OracleLocalIndex:
    """Stands in for B200IndexFlat on a rank without a GPU."""

    def __init__(self, xb, metric):
        self.xb = xb
        self.metric_type = metric
        self.base = 0

    def set_label_base(self, base):
        self.base = base

    def search(self, x, k):
        from oracle import flat_oracle as O
        d, i, _ = O.search(self.metric_type, self.xb, np.asarray(x), k)
        return d, np.where(i >= 0, i + self.base, -1)


def _worker(rank, world, port, metric, k, nb, out_dir):
    sys.path.insert(0, REPO)
    sys.path.insert(0, os.path.join(REPO, "tests"))
    import torch.distributed as dist

    import faiss_metal_b200 as fm
    import helpers as H
    from oracle import flat_oracle as O

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        xb = H.uniform_pm1(nb, 24, 5)
        xb[3::17] = xb[1]  # ties across shards
        xq = H.uniform_pm1(13, 24, 6)
        lo, hi = fm.shard_range(nb, rank, world)
        local = OracleLocalIndex(xb[lo:hi], metric)

        def host_merge(m, d_all, l_all):
            return O.merge(m, d_all, l_all, np.zeros(d_all.shape[0], np.int64))

        sh = fm.ShardedIndexFlat(local, rank, world, merge_fn=host_merge)
        sh.set_shard(lo)
        D, I = sh.search(xq, k)
        fd, fi, _ = O.search(metric, xb, xq, k)
        assert np.array_equal(np.asarray(I), fi), (rank, "labels")
        assert np.array_equal(np.asarray(D), fd), (rank, "distances")
        open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,metric,k,nb", [(2, 1, 10, 500), (2, 0, 64, 300), (3, 1, 7, 100), (2, 1, 40, 31)])
def test_sharded_search_gloo(tmp_path, world, metric, k, nb):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(world, port, metric, k, nb, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / ("ok%d" % r)).exists()


def test_shard_range_covers_everything():
    sys.path.insert(0, REPO)
    import faiss_metal_b200 as fm
    for nb in (0, 1, 7, 100, 10_000_000):
        for world in (1, 2, 3, 8):
            spans = [fm.shard_range(nb, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == nb
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(s for s in sizes if s >= 0) <= (nb + world - 1) // world


def test_pack_roundtrip():
    import torch
    sys.path.insert(0, REPO)
    from faiss_metal_b200 import sharded
    d = torch.randn(5, 7)
    l = torch.randint(-1, 1 << 40, (5, 7))
    buf = sharded.pack_candidates(d, l)
    dd, ll = sharded.unpack_candidates(torch.stack([buf, buf]))
    assert torch.equal(dd[1], d) and torch.equal(ll[0], l)

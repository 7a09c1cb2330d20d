"""GPU parity on inputs with the shapes and value distributions of the benchmark
configurations (seeded synthetic data stands in for them), at sizes the CPU oracle
finishes in seconds, plus the single-GPU emulation of the row-sharded search."""
import ctypes

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu


def run_case(fm, res, xb, xq, metric, storage, k, path=0):
    idx = fm.B200IndexFlat(res, xb.shape[1], metric, storage)
    idx.add(xb)
    if path:
        idx.set_path(path)
    D, I = idx.search(xq, k)
    tensor = (path == 2) or (path == 0 and xq.shape[0] > 4)
    r = H.check_against_oracle(metric, storage, tensor, xb, xq, k, D, I)
    idx.close()
    return r


def test_config1_l2_fp32_full_size(fm, res, select_mode):
    # IndexFlatL2 FP32, nb=100,000, nq=1,000, d=128, U[0,1), k=10 -- full size
    xb = H.uniform01(100_000, 128, 1)
    xq = H.uniform01(1_000, 128, 2)
    r = run_case(fm, res, xb, xq, O.METRIC_L2, 0, 10)
    assert r["loose"]["max_rel_dist_err"] < 1e-4


def test_config2_ip_fp16_scaled(fm, res, select_mode):
    # IndexFlatIP FP16, d=768, unit-norm gaussian rows, k=100 (nb, nq scaled down)
    xb = H.gaussian(70_000, 768, 3, normalise=True)
    xq = H.gaussian(200, 768, 4, normalise=True)
    run_case(fm, res, xb, xq, O.METRIC_INNER_PRODUCT, 1, 100)


def test_config3_l2_bf16_scaled(fm, res, select_mode):
    # IndexFlatL2 BF16, d=1536, N(0,1)*0.05, k=32 (nb, nq scaled down); fused GEMM + top-k
    xb = H.gaussian(70_000, 1536, 5, scale=0.05)
    xq = H.gaussian(300, 1536, 6, scale=0.05)
    run_case(fm, res, xb, xq, O.METRIC_L2, 2, 32)


def test_config4_l2_fp32_large_k_scaled(fm, res, select_mode):
    # IndexFlatL2 FP32, d=96, mixture of 1,000 gaussians, k=1024 (nb, nq scaled down)
    rng = np.random.default_rng(7)
    centres = rng.uniform(-1, 1, size=(1000, 96)).astype(np.float32)
    xb = H.mixture(150_000, 96, 8, centres)
    xq = H.mixture(48, 96, 9, centres)
    run_case(fm, res, xb, xq, O.METRIC_L2, 0, 1024)


def test_config5_l2_fp16_single_query_scaled(fm, res):
    # IndexFlatL2 FP16, d=128, U[0,1), stream of single queries, k=10 (nb scaled down)
    xb = H.uniform01(1_000_000, 128, 10)
    idx = fm.B200IndexFlat(res, 128, O.METRIC_L2, 1)
    idx.add(xb)
    for s in range(4):
        xq = H.uniform01(1, 128, 100 + s)
        D, I = idx.search(xq, 10)
        H.check_against_oracle(O.METRIC_L2, 1, True, xb, xq, 10, D, I)  # streaming scan rounds q to fp16
    idx.close()


@pytest.mark.parametrize("G", [2, 8])
@pytest.mark.parametrize("k,storage,metric", [(32, 2, O.METRIC_L2), (100, 1, O.METRIC_INNER_PRODUCT)])
def test_sharded_emulation_equals_unsharded(fm, res, G, k, storage, metric):
    """G row shards searched one after the other on one GPU, lists merged by the k-way
    merge kernel: labels must equal the unsharded search bit for bit."""
    import torch
    nb, nq, d = 40_000, 64, 128
    xb = H.gaussian(nb, d, 31, scale=0.05)
    xq = H.gaussian(nq, d, 32, scale=0.05)
    full = fm.B200IndexFlat(res, d, metric, storage)
    full.add(xb)
    Df, If = full.search(xq, k)
    full.close()
    dists, labels = [], []
    for g in range(G):
        lo, hi = fm.shard_range(nb, g, G)
        sh = fm.B200IndexFlat(res, d, metric, storage)
        sh.add(xb[lo:hi])
        sh.set_label_base(lo)
        Dg, Ig = sh.search(xq, k)
        dists.append(Dg)
        labels.append(Ig)
        sh.close()
    dd = torch.from_numpy(np.stack(dists)).cuda()
    ll = torch.from_numpy(np.stack(labels)).cuda()
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda:0")
    fm.abi.check_op(fm.lib().b200f_merge_lists(
        ctypes.c_void_p(dd.data_ptr()), ctypes.c_void_p(ll.data_ptr()), G, nq, k, metric,
        ctypes.c_void_p(out_d.data_ptr()), ctypes.c_void_p(out_l.data_ptr()),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "merge")
    torch.cuda.synchronize()
    assert np.array_equal(out_l.cpu().numpy(), If)
    assert np.array_equal(out_d.cpu().numpy(), Df)


def test_sharded_device_path_single_rank(fm, res):
    """ShardedIndexFlat.search_device (enqueue-only search + strided merge entry point) against the
    plain search; world 1 exercises the enqueue path, the strided merge is checked directly."""
    import torch
    xb = H.gaussian(30_000, 64, 41, scale=0.05)
    xq = H.gaussian(50, 64, 42, scale=0.05)
    idx = fm.B200IndexFlat(res, 64, O.METRIC_L2, 2)
    idx.add(xb)
    D, I = idx.search(xq, 10)
    ext = torch.cuda.ExternalStream(res.stream)
    with torch.cuda.stream(ext):
        sh = fm.ShardedIndexFlat(idx, 0, 1)
        Dd, Id = sh.search_device(torch.from_numpy(xq).cuda(), 10)
        assert np.array_equal(Id.cpu().numpy(), I) and np.array_equal(Dd.cpu().numpy(), D)
        # strided merge of two interleaved [distances | labels] rank buffers
        nq, k = 50, 10
        dist_bytes = (nq * k * 4 + 15) // 16 * 16
        rank_bytes = (dist_bytes + nq * k * 8 + 15) // 16 * 16
        buf = torch.zeros(2 * rank_bytes, dtype=torch.uint8, device="cuda")
        halves = []
        for r, (lo, hi) in enumerate([(0, 15_000), (15_000, 30_000)]):
            s = fm.B200IndexFlat(res, 64, O.METRIC_L2, 2)
            s.add(xb[lo:hi])
            s.set_label_base(lo)
            Ds, Is = s.search(xq, k)
            halves.append((Ds, Is))
            off = r * rank_bytes
            buf[off: off + nq * k * 4].view(torch.float32).copy_(torch.from_numpy(Ds).flatten())
            buf[off + dist_bytes: off + dist_bytes + nq * k * 8].view(torch.int64).copy_(torch.from_numpy(Is).flatten())
            s.close()
        out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda")
        out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda")
        fm.abi.check_op(fm.lib().b200f_merge_lists_strided(
            ctypes.c_void_p(buf.data_ptr()), ctypes.c_void_p(buf.data_ptr() + dist_bytes), rank_bytes // 4,
            rank_bytes // 8, 2, nq, k, O.METRIC_L2, ctypes.c_void_p(out_d.data_ptr()),
            ctypes.c_void_p(out_l.data_ptr()), ctypes.c_void_p(ext.cuda_stream)), "merge strided")
        ext.synchronize()
        assert np.array_equal(out_l.cpu().numpy(), I) and np.array_equal(out_d.cpu().numpy(), D)
        del Dd, Id, buf, out_d, out_l, sh
    idx.close()

"""GPU parity tests of the op-level C-ABI entry points (device pointers), modelled on
tests/test_metal_distance.mm of the reference."""
import ctypes

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def vp(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def cur_stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class Stored:
    """Rows stored on the device through b200f_store_rows."""

    def __init__(self, fm, xb, storage, l2=True):
        L = fm.lib()
        self.nb, self.d = xb.shape
        self.storage = storage
        es = 4 if storage == 0 else 2
        # 8 norm columns after round_up(d, 8) in the 16-bit row / split plane 0
        self.pitch = (self.d + 3) // 4 * 4 if storage == 0 else (self.d + 7) // 8 * 8 + 8
        self.ppitch = (self.d + 7) // 8 * 8 + 8
        dev = torch.device("cuda:0")
        self.rows = torch.zeros(max(1, self.nb) * self.pitch * es, dtype=torch.uint8, device=dev)
        self.planes = torch.zeros(3 * max(1, self.nb) * self.ppitch, dtype=torch.int16, device=dev) if storage == 0 else None
        self.norms = torch.zeros(max(1, self.nb), dtype=torch.float32, device=dev)
        src = torch.from_numpy(xb).to(dev)
        fm.abi.check_op(L.b200f_store_rows(vp(src), self.nb, self.d, storage, vp(self.rows), self.pitch,
                                           vp(self.planes), self.ppitch, max(1, self.nb) * self.ppitch,
                                           vp(self.norms), 1, cur_stream()), "store_rows")
        torch.cuda.synchronize()

    def args(self, fm, xq_dev, metric, k, path, out_d=None, out_l=None):
        L = fm.lib()
        a = fm.abi.SearchArgs()
        nq = xq_dev.shape[0]
        a.queries = xq_dev.data_ptr()
        a.nq = nq
        a.d = self.d
        a.storage = self.storage
        a.rows = self.rows.data_ptr()
        a.row_pitch = self.pitch
        a.planes = self.planes.data_ptr() if self.planes is not None else None
        a.plane_pitch = self.ppitch
        a.plane_stride = max(1, self.nb) * self.ppitch
        a.norms = self.norms.data_ptr()
        a.nb = self.nb
        a.metric = metric
        a.k = k
        a.label_base = 0
        a.out_dist = out_d.data_ptr() if out_d is not None else None
        a.out_labels = out_l.data_ptr() if out_l is not None else None
        nbytes = L.b200f_search_scratch_bytes(nq, self.nb, self.d, k, self.storage, path)
        assert nbytes > 0
        self.scratch = torch.empty(nbytes, dtype=torch.uint8, device=xq_dev.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=xq_dev.device)
        a.scratch = self.scratch.data_ptr()
        a.scratch_bytes = nbytes
        a.status = self.status.data_ptr()
        a.stream = torch.cuda.current_stream().cuda_stream
        a.path = path
        a.norm_cols = 1
        return a


@pytest.mark.parametrize("storage", [0, 1, 2])
@pytest.mark.parametrize("n,d", [(100, 128), (10, 1536), (37, 70), (5, 3)])
def test_row_norms_and_store(fm, res, storage, n, d):
    # tests/test_metal_distance.mm:17-96 (100x128 abs 1e-3; 10x1536 rel 1e-4)
    seed = 42 if d == 128 else 123
    xb = H.uniform_pm1(n, d, seed)
    st = Stored(fm, xb, storage)
    want = O.row_norms(O.round_storage(xb, storage))
    got = st.norms[:n].cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6)
    # standalone norm kernel on the stored rows
    out = torch.zeros(n, dtype=torch.float32, device="cuda:0")
    fm.abi.check_op(fm.lib().b200f_row_norms(vp(st.rows), storage, n, d, st.pitch, vp(out), cur_stream()), "row_norms")
    np.testing.assert_allclose(out.cpu().numpy(), want, rtol=1e-5, atol=1e-6)
    # stored bits: bit-exact against the oracle's rounding; load_rows inverts them
    back = torch.zeros(n, d, dtype=torch.float32, device="cuda:0")
    fm.abi.check_op(fm.lib().b200f_load_rows(vp(st.rows), storage, n, d, st.pitch, vp(back), cur_stream()), "load_rows")
    assert np.array_equal(back.cpu().numpy().view(np.uint32), O.round_storage(xb, storage).view(np.uint32))
    if storage == 0:
        # the three bf16 planes sum back to the fp32 value to within 2^-24 relative
        planes = st.planes.view(torch.bfloat16).reshape(3, n, st.ppitch).to(torch.float64)
        pl = planes[:, :, :d].sum(0).cpu().numpy()
        np.testing.assert_allclose(pl, xb.astype(np.float64), rtol=2.0 ** -22, atol=1e-30)
        ncols = planes[0, :, st.ppitch - 8:].sum(1).cpu().numpy()     # scales are 1 for bf16
        np.testing.assert_allclose(ncols, -0.5 * want.astype(np.float64), rtol=2.0 ** -21)
    else:
        # norm columns: sum_i S_i * c_i == -||x||^2 / 2 to >= 21 bits
        d8 = (d + 7) // 8 * 8
        view = st.rows.view(torch.float16 if storage == 1 else torch.bfloat16).reshape(n, st.pitch)
        pieces = view[:, d8:d8 + 8].to(torch.float64).cpu().numpy()
        scales = np.array([4096.0, 2.0, 2.0 ** -10, 2.0 ** -21, 0, 0, 0, 0]) if storage == 1 else \
            np.array([1.0, 1.0, 1.0, 0, 0, 0, 0, 0])
        np.testing.assert_allclose(pieces @ scales, -0.5 * want.astype(np.float64), rtol=2.0 ** -21)


@pytest.mark.parametrize("path", [1, 2])
@pytest.mark.parametrize("storage", [0, 1, 2])
@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nq,nb,d", [(5, 50, 64), (130, 700, 200), (3, 1000, 1536)])
def test_pairwise_matrix(fm, res, path, storage, metric, nq, nb, d):
    # tests/test_metal_distance.mm:98-230: full matrix against the inline CPU loops
    xb = H.uniform_pm1(nb, d, 99)
    xq = H.uniform_pm1(nq, d, 77)
    st = Stored(fm, xb, storage)
    xq_dev = torch.from_numpy(xq).cuda()
    out = torch.full((nq, nb), float("nan"), dtype=torch.float32, device="cuda:0")
    a = st.args(fm, xq_dev, metric, 1, path)
    fm.abi.check_op(fm.lib().b200f_pairwise(ctypes.byref(a), vp(out), nb), "pairwise")
    torch.cuda.synchronize()
    assert int(st.status[0]) == 0
    got = out.cpu().numpy().astype(np.float64)
    xb_eff, xq_eff = H.effective_operands(storage, path == 2, xb, xq)
    want = O.pairwise(metric, xb_eff, xq_eff)
    if metric == O.METRIC_L2 and xq_eff is not xq:
        want = want + (np.sum(xq.astype(np.float64) ** 2, 1) - np.sum(xq_eff.astype(np.float64) ** 2, 1))[:, None]
    scale = np.abs(want).max()
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 2e-5 * scale, np.abs(got - want).max() / scale
    # north-star tolerance against the unrounded fp32 operands
    want32 = O.pairwise(metric, xb, xq)
    tol = H.TOL_NORTH_STAR[storage]
    assert np.abs(got - want32).max() <= tol * scale


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nq,ncols,k", [(7, 1000, 10), (3, 50000, 100), (2, 20000, 1024), (1, 9000, 4096),
                                        (4, 33, 40), (5, 64, 1)])
def test_select_rows(fm, res, metric, nq, ncols, k):
    rng = np.random.default_rng(nq * 1000 + k)
    scores = rng.standard_normal((nq, ncols)).astype(np.float32)
    scores[:, ::7] = scores[:, 3:4]  # plenty of exact ties
    s_dev = torch.from_numpy(scores).cuda()
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda:0")
    fm.abi.check_op(fm.lib().b200f_select_rows(vp(s_dev), nq, ncols, ncols, metric, k, vp(out_d), vp(out_l),
                                               None, 0, cur_stream()), "select_rows")
    torch.cuda.synchronize()
    key = scores if metric == O.METRIC_L2 else -scores
    kk = min(k, ncols)
    for r in range(nq):
        order = np.lexsort((np.arange(ncols), key[r]))[:kk]
        assert np.array_equal(out_l[r, :kk].cpu().numpy(), order)
        assert np.array_equal(out_d[r, :kk].cpu().numpy(), scores[r][order])
        assert (out_l[r, kk:].cpu().numpy() == -1).all()
        pad = out_d[r, kk:].cpu().numpy()
        assert (np.isposinf(pad) if metric == O.METRIC_L2 else np.isneginf(pad)).all()


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("P,nq,k", [(2, 9, 10), (8, 100, 32), (8, 5, 100), (4, 3, 1024), (3, 2, 4096), (8, 1, 1)])
def test_merge_lists(fm, res, metric, P, nq, k):
    # per-shard oracle lists -> device merge == oracle merge (bit-exact)
    per = max(40, k // 2 + 7)
    d = 16
    xb = H.uniform_pm1(P * per, d, 3)
    xb[5::11] = xb[2]  # duplicates across shards: ties resolved by the lower label
    xq = H.uniform_pm1(nq, d, 4)
    dists, labels, base = [], [], []
    for p in range(P):
        d_, i_, _ = O.search(metric, xb[p * per:(p + 1) * per], xq, k)
        dists.append(d_)
        labels.append(np.where(i_ >= 0, i_ + p * per, -1))
        base.append(0)
    want_d, want_i = O.merge(metric, np.stack(dists), np.stack(labels), np.array(base))
    dd = torch.from_numpy(np.stack(dists)).cuda()
    ll = torch.from_numpy(np.stack(labels)).cuda()
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda:0")
    fm.abi.check_op(fm.lib().b200f_merge_lists(vp(dd), vp(ll), P, nq, k, metric, vp(out_d), vp(out_l), cur_stream()),
                    "merge_lists")
    torch.cuda.synchronize()
    assert np.array_equal(out_l.cpu().numpy(), want_i)
    assert np.array_equal(out_d.cpu().numpy(), want_d)


@pytest.mark.parametrize("dist_kind", [0, 1, 2, 3])
def test_fill_synthetic(fm, res, dist_kind):
    n, d = 4096, 96
    a = torch.empty((n, d), dtype=torch.float32, device="cuda:0")
    b = torch.empty((n // 2, d), dtype=torch.float32, device="cuda:0")
    L = fm.lib()
    fm.abi.check_op(L.b200f_fill_synthetic(vp(a), n, d, 0, 7, dist_kind, 0.05, cur_stream()), "fill")
    fm.abi.check_op(L.b200f_fill_synthetic(vp(b), n // 2, d, n // 2, 7, dist_kind, 0.05, cur_stream()), "fill")
    torch.cuda.synchronize()
    assert torch.equal(a[n // 2:], b)  # rows depend on (seed, global row, col) only
    x = a.cpu().numpy().astype(np.float64)
    if dist_kind == 0:
        assert x.min() >= 0 and x.max() < 1 and abs(x.mean() - 0.5) < 0.01 and abs(x.var() - 1 / 12) < 0.005
    elif dist_kind == 1:
        assert abs(x.mean()) < 1e-3 and abs(x.std() - 0.05) < 1e-3
    elif dist_kind == 2:
        np.testing.assert_allclose(np.linalg.norm(x, axis=1), 1.0, rtol=1e-5)
    else:
        # sigma = 0 leaves the bare centres: at most 1,000 distinct rows inside [-1,1]^d, the same
        # set for every seed; with sigma = 0.05 the rows scatter around them by N(0, 0.05^2)
        c7 = torch.empty((n, d), dtype=torch.float32, device="cuda:0")
        c8 = torch.empty((n, d), dtype=torch.float32, device="cuda:0")
        fm.abi.check_op(L.b200f_fill_synthetic(vp(c7), n, d, 0, 7, dist_kind, 0.0, cur_stream()), "fill")
        fm.abi.check_op(L.b200f_fill_synthetic(vp(c8), n, d, 0, 8, dist_kind, 0.0, cur_stream()), "fill")
        torch.cuda.synchronize()
        u7 = {r.tobytes() for r in c7.cpu().numpy()}
        u8 = {r.tobytes() for r in c8.cpu().numpy()}
        assert 900 < len(u7) <= 1000 and 900 < len(u8) <= 1000 and len(u7 & u8) > 850
        assert len(u7 | u8) <= 1000
        assert float(c7.abs().max()) <= 1.0
        noise = x - c7.cpu().numpy().astype(np.float64)
        assert abs(noise.mean()) < 1e-3 and abs(noise.std() - 0.05) < 1e-3


def run_search(fm, st, xq, metric, k, path):
    xq_dev = torch.from_numpy(xq).cuda()
    nq = xq.shape[0]
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda:0")
    a = st.args(fm, xq_dev, metric, k, path, out_d, out_l)
    fm.abi.check_op(fm.lib().b200f_search(ctypes.byref(a)), "search")
    torch.cuda.synchronize()
    status = st.status.cpu().numpy()
    assert status[0] == 0
    return out_d.cpu().numpy(), out_l.cpu().numpy(), int(status[1])


@pytest.mark.parametrize("storage,metric,k,nq,nb", [(2, O.METRIC_L2, 100, 300, 70_000),
                                                    (1, O.METRIC_INNER_PRODUCT, 100, 130, 70_000),
                                                    (0, O.METRIC_L2, 1024, 40, 70_000),
                                                    (2, O.METRIC_L2, 33, 257, 70_000),
                                                    (1, O.METRIC_INNER_PRODUCT, 500, 9, 70_000),
                                                    (2, O.METRIC_L2, 10, 600, 70_000),
                                                    (0, O.METRIC_L2, 32, 100, 70_000),
                                                    (1, O.METRIC_L2, 1024, 300, 140_000),
                                                    (2, O.METRIC_INNER_PRODUCT, 200, 50, 140_000)])
def test_optimistic_selection_random_rows(fm, res, select_mode, storage, metric, k, nq, nb):
    # Tensor path, k <= 1024.  filter: threshold filter from 64k rows (k <= 128) / 128k rows up,
    # else selection from the fused kernel's 32-entry lists; no_filter: lists (fused kernel for
    # k <= 32); matrix_or_fused: key matrix.  With rows in random order no stage has to give up,
    # so no row is redone (status word 1 counts them), and all modes agree with the oracle.
    d = 64
    xb = H.gaussian(nb, d, 51)
    xq = H.gaussian(nq, d, 52)
    st = Stored(fm, xb, storage)
    D, I, redone = run_search(fm, st, xq, metric, k, 2)
    assert redone == 0
    H.check_against_oracle(metric, storage, True, xb, xq, k, D, I, loose=False)


@pytest.mark.parametrize("storage,metric,k", [(2, O.METRIC_L2, 100), (0, O.METRIC_L2, 200),
                                              (1, O.METRIC_INNER_PRODUCT, 64), (2, O.METRIC_L2, 20)])
@pytest.mark.parametrize("nq,near", [(300, 150), (700, 700), (130, 1)])
def test_optimistic_selection_redoes_rows(fm, res, select_mode, storage, metric, k, nq, near):
    # The k nearest rows of `near` queries are the first rows of the database.  They sit next
    # to each other (one 32-entry list cannot hold them all) and inside the first column tile,
    # which the pilot pass samples (its threshold then admits fewer than k rows): exactly these
    # queries must be found and redone; the others keep the optimistic result.
    nb, d = 70_000, 32
    rng = np.random.default_rng(61)
    xb = H.gaussian(nb, d, 62)
    # a cluster far from everything else, wide enough that ||q||^2 + ||x||^2 - 2 q.x does not
    # cancel to nothing inside it
    centre = np.full(d, 2.0, dtype=np.float32)
    xb[:250] = centre + 0.3 * rng.standard_normal((250, d)).astype(np.float32)
    xq = H.gaussian(nq, d, 63)
    rows = rng.permutation(nq)[:near]
    xq[rows] = centre + 0.3 * rng.standard_normal((near, d)).astype(np.float32)
    st = Stored(fm, xb, storage)
    D, I, redone = run_search(fm, st, xq, metric, k, 2)
    optimistic = select_mode == "filter" or (select_mode == "no_filter" and k > 32)
    if not optimistic:
        assert redone == 0
    elif metric == O.METRIC_L2:
        assert redone == near
    else:
        assert redone >= near  # a long query also favours the cluster's direction
    H.check_against_oracle(metric, storage, True, xb, xq, k, D, I, loose=False)
    # the redone rows are counted and compacted on the device: a second run agrees bit for bit
    D2, I2, _ = run_search(fm, st, xq, metric, k, 2)
    assert np.array_equal(I, I2) and np.array_equal(D, D2)


@pytest.fixture
def force_filter(fm):
    L = fm.lib()
    old = L.b200f_get_selection_mode()
    assert L.b200f_set_selection_mode(fm.abi.SELECT_FILTER) == 0
    yield
    L.b200f_set_selection_mode(old)


@pytest.mark.parametrize("k", [10, 100])
def test_threshold_filter_overflow_is_redone(fm, res, force_filter, k):
    # 30,000 copies of one row: for a query next to it every copy lies under any threshold, the
    # candidate buffer overflows, and the row must be redone (ties resolved by the lower label)
    nb, d = 80_000, 32
    xb = H.gaussian(nb, d, 81)
    xb[10_000:40_000] = xb[7]
    xq = H.gaussian(40, d, 82)
    xq[3] = xb[7] + 0.01
    xq[17] = xb[7] - 0.01
    st = Stored(fm, xb, 2)
    D, I, redone = run_search(fm, st, xq, O.METRIC_L2, k, 2)
    assert 2 <= redone < 10  # a random query may also have the copied row among its k best
    H.check_against_oracle(O.METRIC_L2, 2, True, xb, xq, k, D, I, loose=False)
    assert I[3, 0] == 7 and list(I[3, 1:k]) == list(range(10_000, 10_000 + k - 1))


def test_list_selection_small_shard_uses_matrix(fm, res):
    # too few column ranges for lists to hold 4 k candidates: plain key-matrix path, nothing redone
    xb = H.gaussian(3_000, 48, 71)
    xq = H.gaussian(20, 48, 72)
    st = Stored(fm, xb, 2)
    D, I, redone = run_search(fm, st, xq, O.METRIC_L2, 500, 2)
    assert redone == 0
    H.check_against_oracle(O.METRIC_L2, 2, True, xb, xq, 500, D, I, loose=False)


@pytest.mark.parametrize("nq,nb,k,path", [(300, 70_000, 10, 2), (40, 70_000, 100, 2), (1, 200_000, 10, 1),
                                          (20, 5_000, 64, 2)])
def test_search_is_enqueue_only_cuda_graph(fm, res, force_filter, nq, nb, k, path):
    # b200f_search only enqueues work (rows to redo are counted on the device, nothing is read
    # back): the whole search can be captured into a CUDA graph and replayed on new queries
    d = 64
    xb = H.gaussian(nb, d, 91)
    st = Stored(fm, xb, 2)
    xq_dev = torch.from_numpy(H.gaussian(nq, d, 92)).cuda()
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda:0")
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        a = st.args(fm, xq_dev, O.METRIC_L2, k, path, out_d, out_l)
        a.stream = side.cuda_stream
        fm.abi.check_op(fm.lib().b200f_search(ctypes.byref(a)), "warm-up search")  # one-time attribute calls
        side.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            fm.abi.check_op(fm.lib().b200f_search(ctypes.byref(a)), "captured search")
        for seed in (93, 94):
            xq = H.gaussian(nq, d, seed)
            xq_dev.copy_(torch.from_numpy(xq))
            out_l.fill_(-7)
            g.replay()
            side.synchronize()
            assert int(st.status[0]) == 0
            H.check_against_oracle(O.METRIC_L2, 2, True, xb, xq, k, out_d.cpu().numpy(), out_l.cpu().numpy(),
                                   loose=False)
    torch.cuda.synchronize()

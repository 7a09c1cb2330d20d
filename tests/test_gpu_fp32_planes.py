"""FP32 storage on the tensor path: the two split-plane formats (three bf16 planes / two fp16
planes of the rows scaled by a power of two), the index's choice of scale, its fall-back when rows
leave fp16's range, and per-row query scaling.  The contract is 1e-4 relative on distances and
labels equal to the oracle's up to proven ties, for both formats."""
import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

BF16X3, FP16X2 = 0, 1


def build(fm, res, xb, metric, fmt=None, pieces=1):
    idx = fm.B200IndexFlat(res, xb.shape[1], metric, 0)
    if fmt is not None:
        idx.set_fp32_planes(fmt)
    idx.set_path(fm.PATH_TENSOR)
    step = (xb.shape[0] + pieces - 1) // pieces
    for r0 in range(0, xb.shape[0], step):
        idx.add(xb[r0:r0 + step])
    return idx


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nb,nq,d,k", [(20_000, 200, 96, 10), (70_000, 300, 128, 100), (5_000, 37, 33, 1024)])
def test_both_formats_hold_the_fp32_contract(fm, res, metric, nb, nq, d, k):
    centres = np.random.default_rng(1).uniform(-1, 1, size=(50, d)).astype(np.float32)
    xb = H.mixture(nb, d, 2, centres)          # clustered: near neighbours, heavy cancellation in L2
    xq = H.mixture(nq, d, 3, centres)
    results = {}
    for fmt in (FP16X2, BF16X3):
        idx = build(fm, res, xb, metric, fmt, pieces=3)
        assert idx.fp32_planes == fmt
        D, I = idx.search(xq, k)
        H.check_against_oracle(metric, 0, True, xb, xq, k, D, I)
        results[fmt] = (D, I)
        idx.close()
    # the two formats agree far inside the tolerance
    a, b = results[FP16X2][0], results[BF16X3][0]
    fin = np.isfinite(a)
    scale = np.abs(b[fin]).max()
    assert np.abs(a[fin] - b[fin]).max() <= 5e-5 * scale


def test_default_is_two_fp16_planes_and_any_magnitude_works(fm, res):
    # the scale comes from the data: rows of order 1e-6, 1 and 1e5 give the same neighbours
    d = 64
    base = H.gaussian(30_000, d, 5)
    q = H.gaussian(100, d, 6)
    want = None
    for mag in (1e-6, 1.0, 1e5):
        idx = build(fm, res, (base * np.float32(mag)).astype(np.float32), O.METRIC_L2)
        assert idx.fp32_planes == FP16X2
        xq = (q * np.float32(mag)).astype(np.float32)
        D, I = idx.search(xq, 10)
        H.check_against_oracle(O.METRIC_L2, 0, True, (base * np.float32(mag)).astype(np.float32), xq, 10, D, I)
        if want is None:
            want = I
        else:
            assert (I == want).mean() > 0.999      # same geometry, power-of-two-free scaling: ties aside
        idx.close()


def test_queries_are_scaled_per_row(fm, res):
    # query rows nine orders of magnitude apart in one batch, and an all-zero query
    d = 48
    xb = H.gaussian(40_000, d, 7)
    xq = H.gaussian(90, d, 8)
    xq[0::3] *= np.float32(1e-4)
    xq[1::3] *= np.float32(3e4)
    xq[5] = 0
    for metric in (O.METRIC_L2, O.METRIC_INNER_PRODUCT):
        idx = build(fm, res, xb, metric)
        assert idx.fp32_planes == FP16X2
        D, I = idx.search(xq, 20)
        H.check_against_oracle(metric, 0, True, xb, xq, 20, D, I)
        idx.close()


def test_rows_outside_fp16_range_fall_back_to_bf16_planes(fm, res):
    d = 40
    xb = H.gaussian(30_000, d, 9)
    xq = H.gaussian(64, d, 10)
    # (1) a later add 5,000 times larger than the scale was made for
    big = xb.copy()
    big[20_000:] *= np.float32(5000.0)
    idx = build(fm, res, big, O.METRIC_L2, pieces=3)
    assert idx.fp32_planes == BF16X3
    D, I = idx.search(xq, 10)
    H.check_against_oracle(O.METRIC_L2, 0, True, big, xq, 10, D, I)
    idx.close()
    # (2) rows 1e-5 of the others: their low plane would go subnormal
    tiny = xb.copy()
    tiny[100:200] *= np.float32(1e-5)
    idx = build(fm, res, tiny, O.METRIC_L2)
    assert idx.fp32_planes == BF16X3
    qt = (xq * np.float32(1e-5)).astype(np.float32)     # queries among the tiny rows
    D, I = idx.search(qt, 10)
    H.check_against_oracle(O.METRIC_L2, 0, True, tiny, qt, 10, D, I)
    # reset forgets scale and format
    idx.reset()
    idx.add(xb)
    assert idx.fp32_planes == FP16X2
    D, I = idx.search(xq, 10)
    H.check_against_oracle(O.METRIC_L2, 0, True, xb, xq, 10, D, I)
    idx.close()
    # (3) zeros first: the scale waits for the first non-zero rows
    z = np.concatenate([np.zeros((2000, d), np.float32), xb[:8000]])
    idx = build(fm, res, z, O.METRIC_INNER_PRODUCT, pieces=5)
    assert idx.fp32_planes == FP16X2
    D, I = idx.search(xq, 10)
    H.check_against_oracle(O.METRIC_INNER_PRODUCT, 0, True, z, xq, 10, D, I)
    idx.close()


def test_format_can_only_be_chosen_on_an_empty_index(fm, res):
    idx = fm.B200IndexFlat(res, 16, O.METRIC_L2, 0)
    idx.set_fp32_planes(BF16X3)
    idx.add(H.gaussian(100, 16, 1))
    with pytest.raises(fm.B200Error) as e:
        idx.set_fp32_planes(FP16X2)
    assert e.value.status == fm.abi.ERR_STATE
    with pytest.raises(fm.B200Error) as e:
        fm.B200IndexFlat(res, 16, O.METRIC_L2, 0).set_fp32_planes(7)
    assert e.value.status == fm.abi.ERR_BAD_ARG
    idx.close()


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
def test_op_level_fp16_planes_pairwise_and_search(fm, res, metric):
    """The op-level entry points with the FP16X2 plane format: b200f_rows_absmax gives the scale,
    b200f_store_rows_fp32 writes the planes, b200f_pairwise (keys scaled back per query row in the
    store epilogue) and b200f_search multiply them."""
    import ctypes

    import torch
    from test_gpu_ops import Stored, cur_stream, vp
    L = fm.lib()
    nb, nq, d = 3000, 150, 72
    xb = (H.gaussian(nb, d, 21) * np.float32(37.0)).astype(np.float32)
    xq = (H.gaussian(nq, d, 22) * np.float32(0.02)).astype(np.float32)
    xq[::2] *= np.float32(500.0)
    st = Stored(fm, xb, 0)                                  # allocates rows / planes / norms (bf16x3 content)
    src = torch.from_numpy(xb).cuda()
    bits = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    fm.abi.check_op(L.b200f_rows_absmax(vp(src), nb, d, d, vp(bits), cur_stream()), "rows_absmax")
    amax = np.array([int(bits.cpu()[0])], dtype=np.uint32).view(np.float32)[0]
    assert amax == np.abs(xb).max()
    lg = 7 - int(np.frexp(amax)[1])
    flag = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    fm.abi.check_op(L.b200f_store_rows_fp32(vp(src), d, nb, d, vp(st.rows), st.pitch, vp(st.planes), st.ppitch,
                                            max(1, nb) * st.ppitch, fm.abi.PLANES_FP16X2, lg, vp(flag), vp(st.norms), 1,
                                            cur_stream()), "store_rows_fp32")
    torch.cuda.synchronize()
    assert int(flag.cpu()[0]) == 0
    # plane 0 + plane 1 reproduce 2^lg * x to 22 bits
    planes = st.planes.view(torch.float16).reshape(3, nb, st.ppitch).to(torch.float64)
    back = (planes[0, :, :d] + planes[1, :, :d]).cpu().numpy() / 2.0 ** lg
    np.testing.assert_allclose(back, xb.astype(np.float64), rtol=2.0 ** -21, atol=2.0 ** (-25 - lg))
    xq_dev = torch.from_numpy(xq).cuda()
    out = torch.full((nq, nb), float("nan"), dtype=torch.float32, device="cuda:0")
    a = st.args(fm, xq_dev, metric, 1, 2)
    a.plane_format = fm.abi.PLANES_FP16X2
    a.plane_scale_log2 = lg
    fm.abi.check_op(L.b200f_pairwise(ctypes.byref(a), vp(out), nb), "pairwise")
    torch.cuda.synchronize()
    got = out.cpu().numpy().astype(np.float64)
    want = O.pairwise(metric, xb, xq)
    if metric == O.METRIC_L2:
        assert (np.abs(got - want) <= 1e-4 * np.maximum(want, 1e-3 * want.max())).all()
    else:
        # relative to |q| |x| of each pair's query row (rows differ by 500x in magnitude)
        bound = 1e-5 * np.linalg.norm(xq, axis=1)[:, None] * np.linalg.norm(xb, axis=1)[None, :]
        assert (np.abs(got - want) <= bound).all()
    k = 40
    out_d = torch.empty((nq, k), dtype=torch.float32, device="cuda:0")
    out_l = torch.empty((nq, k), dtype=torch.int64, device="cuda:0")
    a = st.args(fm, xq_dev, metric, k, 2, out_d, out_l)
    a.plane_format = fm.abi.PLANES_FP16X2
    a.plane_scale_log2 = lg
    fm.abi.check_op(L.b200f_search(ctypes.byref(a)), "search")
    torch.cuda.synchronize()
    assert int(st.status[0]) == 0
    H.check_against_oracle(metric, 0, True, xb, xq, k, out_d.cpu().numpy(), out_l.cpu().numpy())
    # a row that does not fit raises the flag
    xb2 = xb.copy()
    xb2[7] *= np.float32(1e4)
    src2 = torch.from_numpy(xb2).cuda()
    fm.abi.check_op(L.b200f_store_rows_fp32(vp(src2), d, nb, d, vp(st.rows), st.pitch, vp(st.planes), st.ppitch,
                                            max(1, nb) * st.ppitch, fm.abi.PLANES_FP16X2, lg, vp(flag), vp(st.norms), 1,
                                            cur_stream()), "store_rows_fp32")
    torch.cuda.synchronize()
    assert int(flag.cpu()[0]) == 1
    # bad arguments
    assert L.b200f_store_rows_fp32(vp(src), d, nb, d, vp(st.rows), st.pitch, vp(st.planes), st.ppitch,
                                   max(1, nb) * st.ppitch, 5, lg, None, None, 1, cur_stream()) == fm.abi.ERR_BAD_ARG
    assert L.b200f_rows_absmax(vp(src), nb, d, d, None, cur_stream()) == fm.abi.ERR_BAD_ARG

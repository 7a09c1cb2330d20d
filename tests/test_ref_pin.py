"""Pins the oracle to the reference's OWN CPU code.

tests/golden/ref_loops.npz holds what the reference's inline CPU loops compute on the
reference's own seeded inputs (tests/test_metal_distance.mm:23-54,65-93,105-153,164-227 and the
generator of tests/test_metal_flat.mm:64-70 for the shapes of :477-490); it is produced by
tests/golden/make_ref_golden.py, which compiles those lines out of the reference tree.  The
reference accumulates in fp32, the oracle in double: they must agree to fp32 accumulation
noise (1e-5 relative here; the reference's own tolerances are 1e-3 absolute / 1e-4 relative
for norms and 5e-2 relative for distances).

What this pins: squared norms, squared-L2 and inner-product values, and rank 1 (the only rank
the reference asserts on, tests/test_metal_flat.mm:52-58, tests/test_metal_distance.mm:206-227).
Ranks >= 2 are pinned against the selection the reference's distance values imply (stable sort
of its fp32 matrix), which the reference itself never checks.
"""
import os

import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_loops.npz")
FLAT_CASES = ["flat_l2_1000x32", "flat_l2_1000x128", "flat_l2_500x768", "flat_l2_500x1536", "flat_l2_100x32",
              "flat_ip_1000x128"]
REL = 1e-5


@pytest.fixture(scope="module")
def ref():
    return np.load(FIX)


def flat_inputs(ref, tag):
    """Regenerates the inputs of a flat case from the reference's seed (42: vectors first, then
    queries) and checks them against the checksum the reference-side generator left."""
    nv, nq, d, k, chk = (int(x) for x in ref[tag + "_meta"])
    draws = H.mt19937_uniform_pm1(42, nv * d + nq * d)
    xb = draws[: nv * d].reshape(nv, d)
    xq = draws[nv * d:].reshape(nq, d)
    assert H.fnv1a64_half(xb, xq) == chk, "regenerated inputs differ from the reference generator's"
    return xb, xq, k


def test_generator_restatement_is_bit_exact(ref):
    # the numpy restatement of std::mt19937 + uniform_real_distribution<float>(-1, 1)
    assert np.array_equal(H.mt19937_uniform_pm1(42, 100 * 128).reshape(100, 128), ref["norm_small_x"])
    assert np.array_equal(H.mt19937_uniform_pm1(123, 10 * 1536).reshape(10, 1536), ref["norm_large_x"])
    draws = H.mt19937_uniform_pm1(99, 5 * 64 + 50 * 64)   # queries first, then vectors (:112-115)
    assert np.array_equal(draws[: 5 * 64].reshape(5, 64), ref["l2_q"])
    assert np.array_equal(draws[5 * 64:].reshape(50, 64), ref["l2_x"])


@pytest.mark.parametrize("case", ["norm_small", "norm_large"])
def test_row_norms_match_reference_loop(oracle, ref, case):
    got = oracle.row_norms(ref[case + "_x"])
    np.testing.assert_allclose(got, ref[case + "_out"], rtol=REL, atol=0)


def test_l2_matrix_matches_reference_loop(oracle, ref):
    got = oracle.pairwise(O.METRIC_L2, ref["l2_x"], ref["l2_q"])
    np.testing.assert_allclose(got, ref["l2_out"], rtol=REL, atol=0)


def test_ip_matrix_and_top1_match_reference_loop(oracle, ref):
    got = oracle.pairwise(O.METRIC_INNER_PRODUCT, ref["ip_x"], ref["ip_q"])
    scale = float(np.abs(ref["ip_out"]).max())
    assert np.abs(got - ref["ip_out"]).max() <= REL * scale
    # the reference's CPU top-1 (:206-227).  Its running best starts from a value that is not
    # row 0's inner product (:211-212 multiplies by vectors[0] for every k); that only matters
    # when row 0 is the best row, which the comparison below would expose.
    _, lab, _ = oracle.search(O.METRIC_INNER_PRODUCT, ref["ip_x"], ref["ip_q"], 1)
    assert np.array_equal(lab[:, 0], ref["ip_top1"])
    assert np.array_equal(np.argmax(ref["ip_out"], axis=1), ref["ip_top1"])


@pytest.mark.parametrize("tag", FLAT_CASES)
def test_flat_shapes_match_reference_loops(oracle, ref, tag):
    xb, xq, k = flat_inputs(ref, tag)
    metric = O.METRIC_INNER_PRODUCT if "_ip_" in tag else O.METRIC_L2
    want = ref[tag + "_out"].astype(np.float64)
    got = oracle.pairwise(metric, xb, xq)
    scale = np.abs(want).max() if metric == O.METRIC_INNER_PRODUCT else np.abs(want)
    assert (np.abs(got - want) <= REL * scale).all()
    # selection implied by the reference's values: best first, ties to the lower row
    key = want if metric == O.METRIC_L2 else -want
    order = np.stack([np.lexsort((np.arange(key.shape[1]), key[i]))[:k] for i in range(key.shape[0])])
    d32, lab, d64 = oracle.search(metric, xb, xq, k)
    assert np.array_equal(lab[:, 0], order[:, 0]), "rank 1 differs from the reference's CPU values"
    ref_d = np.take_along_axis(want, order, axis=1)
    true_d = oracle.rescore(metric, xb, xq, lab)
    r = oracle.compare_results(metric, d32, lab, ref_d, order, true_d, REL, eps=1e-3)
    assert oracle.passed(r), r
    assert r["label_diff"] == 0   # no fp32-noise tie among the first k of these cases


def test_fixture_regenerates_bit_for_bit(oracle, ref, tmp_path):
    """Where the reference checkout is present, the committed recipe reproduces the fixture."""
    import subprocess
    binary = oracle.build_ref()
    if binary is None:
        pytest.skip("reference checkout not present: the committed fixture is used as it is")
    manifest = subprocess.check_output([binary, str(tmp_path)], text=True)
    names = []
    for line in manifest.splitlines():
        f = line.split()
        a = np.fromfile(str(tmp_path / (f[0] + ".bin")), dtype={"f32": np.float32, "i64": np.int64}[f[1]])
        assert np.array_equal(a.reshape(tuple(int(x) for x in f[2:])), ref[f[0]]), f[0]
        names.append(f[0])
    assert sorted(names) == sorted(ref.files)

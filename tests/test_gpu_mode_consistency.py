"""The tensor path has three ways to select the k best (threshold filter, 32-entry lists, key
matrix).  All of them see the same keys (the same GEMM kernel produces them), so their results
must agree bit for bit on any input; one of them (the key matrix) is also checked against the
oracle on the smaller shapes.  Seeded random shapes: odd dimensions, partial tiles, k from 1 to
1024, several query blocks, all storage types and both metrics."""
import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu

MODES = {"filter": 1, "no_filter": 2, "matrix_or_fused": 3}   # B200F_SELECT_*


def search_in_mode(fm, idx, xq, k, mode):
    L = fm.lib()
    old = L.b200f_get_selection_mode()
    assert L.b200f_set_selection_mode(MODES[mode]) == 0
    try:
        return idx.search(xq, k)
    finally:
        L.b200f_set_selection_mode(old)


def random_shapes(seed, count):
    rng = np.random.default_rng(seed)
    shapes = []
    for _ in range(count):
        nb = int(rng.choice([66_000, 70_001, 131_072, 140_000, 263_000]))
        nq = int(rng.choice([5, 33, 128, 129, 257, 700, 1500]))
        d = int(rng.choice([8, 24, 33, 64, 100, 129, 200]))
        k = int(rng.choice([1, 7, 32, 33, 100, 128, 129, 500, 1024]))
        storage = int(rng.integers(0, 3))
        metric = int(rng.choice([O.METRIC_L2, O.METRIC_INNER_PRODUCT]))
        dup = bool(rng.integers(0, 2))
        shapes.append((nb, nq, d, k, storage, metric, dup))
    return shapes


@pytest.mark.parametrize("nb,nq,d,k,storage,metric,dup", random_shapes(2024, 32))
def test_selection_modes_agree(fm, res, nb, nq, d, k, storage, metric, dup):
    rng = np.random.default_rng(nb + nq + d + k)
    xb = rng.standard_normal((nb, d), dtype=np.float32)
    if dup:
        # blocks of exact copies next to each other and far apart: ties inside the k best, lists
        # that overflow, thresholds that admit too few rows
        xb[1000:1300] = xb[17]
        xb[nb // 2::501] = xb[17]
        xb[:200] = xb[3] + 0.25 * rng.standard_normal((200, d), dtype=np.float32)
    xq = rng.standard_normal((nq, d), dtype=np.float32)
    xq[::7] = xb[17] + 0.05
    # exact copies of a STORED row (a query that is only rounded on the device would make the
    # exact ||q||^2 and the rounded dot product disagree: a slightly negative distance, clamped)
    xq[1::7] = O.round_storage(xb[3:4], storage)[0]
    idx = fm.B200IndexFlat(res, d, metric, storage)
    idx.add(xb)
    idx.set_path(2)
    results = {mode: search_in_mode(fm, idx, xq, k, mode) for mode in MODES}
    D0, I0 = results["matrix_or_fused"]
    for mode in ("filter", "no_filter"):
        Dm, Im = results[mode]
        assert np.array_equal(Im, I0), (mode, int((Im != I0).sum()))
        assert np.array_equal(Dm, D0), mode
    if nq * nb <= 30_000_000:
        H.check_against_oracle(metric, storage, True, xb, xq, k, D0, I0, loose=False)
    idx.close()

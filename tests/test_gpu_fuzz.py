"""Seeded random shapes through the public index surface (automatic path choice, adds in pieces,
one to three shards on the GPU) against the oracle at the north-star tolerance: odd dimensions,
k from 1 to beyond the number of rows, single queries (graph replay) up to several query blocks,
every storage type and both metrics."""
import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu


def cases(seed, count):
    rng = np.random.default_rng(seed)
    out = []
    for i in range(count):
        nb = int(rng.choice([1, 7, 300, 2_000, 9_000, 40_000, 90_000]))
        nq = int(rng.choice([1, 1, 2, 3, 5, 8, 9, 17, 130, 300]))
        d = int(rng.choice([1, 3, 8, 17, 32, 50, 96, 128, 200, 257]))
        k = int(rng.choice([1, 2, 10, 32, 33, 50, 100, 300, 1024, 1100]))
        storage = int(rng.integers(0, 3))
        metric = int(rng.choice([O.METRIC_L2, O.METRIC_INNER_PRODUCT]))
        shards = int(rng.choice([1, 1, 2, 3]))
        pieces = int(rng.choice([1, 2, 4]))
        scale = float(rng.choice([0.05, 1.0, 30.0]))
        out.append((i, nb, nq, d, k, storage, metric, shards, pieces, scale))
    return out


@pytest.mark.parametrize("i,nb,nq,d,k,storage,metric,shards,pieces,scale", cases(77, 40))
def test_random_shapes_against_oracle(fm, res, i, nb, nq, d, k, storage, metric, shards, pieces, scale):
    if nq * nb * d > 3e9:
        nq = max(1, int(3e9 / (nb * d)))
    xb = H.gaussian(nb, d, 1000 + i, scale=scale)
    xq = H.gaussian(nq, d, 2000 + i, scale=scale)
    if nb > 10:
        xb[nb // 2] = xb[1]                      # an exact duplicate
        xq[0] = xb[nb // 3]                      # a query that is a stored row
    if shards == 1:
        idx = fm.B200IndexFlat(res, d, metric, storage)
    else:
        idx = fm.MultiGpuIndexFlat([res] * shards, d, metric, storage, block_rows=256)
    step = (nb + pieces - 1) // pieces
    for r0 in range(0, nb, step):
        idx.add(xb[r0:r0 + step])
    assert idx.ntotal == nb
    for rep in range(3 if nq <= 8 else 1):       # small searches: eager, captured, replayed
        D, I = idx.search(xq, k)
        # tolerance of the storage type; the denominator floor keeps scores that cross zero sane
        _, ref_i, ref_d = O.search(metric, xb, xq, k)
        true_d = O.rescore(metric, xb, xq, I)
        fin = np.isfinite(ref_d)
        eps = max(1e-1 * float(np.abs(ref_d[fin]).max()) if fin.any() else 1e-6, 1e-6)
        xn = np.einsum("ij,ij->i", xb, xb)
        qn = np.einsum("ij,ij->i", xq, xq)
        if metric == O.METRIC_L2:
            # ||q||^2 + ||x||^2 - 2 q.x cancels: an error is relative to the norms, not to a
            # distance that may be a million times smaller (d = 1: neighbours 1e-4 apart)
            eps = max(eps, 0.25 * float(np.median(xn) + qn.max()))
        else:
            # a dot product of random vectors is small against |q| |x|, which is what rounding
            # errors of 16-bit storage are relative to
            eps = max(eps, 0.25 * float(np.sqrt(np.median(xn) * qn.max())))
        r = O.compare_results(metric, D, I, ref_d, ref_i, true_d, H.TOL_NORTH_STAR[storage], eps=eps)
        assert O.passed(r), (rep, r, D[:2, :6], ref_d[:2, :6], I[:2, :6], ref_i[:2, :6])
    idx.close()

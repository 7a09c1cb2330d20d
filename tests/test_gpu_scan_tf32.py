"""Five to eight queries on FP32 rows take the streaming scan that multiplies a tf32 split of the
staged rows (scan_tf32_kernel).  Checked against the oracle on the stored operands (strict
tolerance), for both metrics, dimensions that are not a multiple of the 16-column chunk, ties, more
than one query group (scan path forced) and shards with a partial last stage."""
import numpy as np
import pytest

import helpers as H
from oracle import flat_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("metric", [O.METRIC_L2, O.METRIC_INNER_PRODUCT])
@pytest.mark.parametrize("nb,nq,d,k,force_scan", [
    (70_000, 5, 64, 10, False),
    (70_001, 8, 128, 32, False),
    (66_000, 6, 100, 1, False),       # d not a multiple of 16: the last chunk is partly padding
    (131_077, 7, 33, 7, False),       # padded row pitch, partial last stage
    (90_000, 13, 48, 10, True),       # groups of 8 and 5
    (200_000, 8, 16, 32, False),      # a single chunk per row
    (66_000, 8, 768, 10, False),      # the widest rows the kernel takes: three stages of 16 rows
    (66_000, 6, 1024, 5, False),      # wider: these queries go to the tensor path
    (5_000, 3, 64, 10, False),        # a shard of a few stages: fewer CTAs than SMs
])
def test_tf32_scan_against_oracle(fm, res, metric, nb, nq, d, k, force_scan):
    rng = np.random.default_rng(nb + nq + d)
    xb = rng.standard_normal((nb, d), dtype=np.float32)
    xb[1000:1040] = xb[17]                 # exact ties: lower label first
    xb[nb - 5:] = xb[17]                   # in the last (partial) stage too
    xq = rng.standard_normal((nq, d), dtype=np.float32)
    if d <= 128:
        # a near copy of a stored row (at large d the fp32 cancellation in ||q||^2 + ||x||^2 - 2 q.x,
        # terms of ~d each, is all such a distance consists of, on any kernel)
        xq[0] = xb[17] + 0.01
    idx = fm.B200IndexFlat(res, d, metric, fm.abi.STORAGE_F32)
    idx.add(xb)
    if force_scan:
        idx.set_path(1)
    D, I = idx.search(xq, k)
    H.check_against_oracle(metric, fm.abi.STORAGE_F32, False, xb, xq, k, D, I, loose=True)
    # the same queries four at a time run on the FMA kernel: same labels, distances to 1e-4
    D4 = np.empty_like(D)
    I4 = np.empty_like(I)
    for q0 in range(0, nq, 4):
        D4[q0:q0 + 4], I4[q0:q0 + 4] = idx.search(xq[q0:q0 + 4], k)
    # an L2 distance is ||q||^2 + ||x||^2 - 2 q.x: its error scales with the norms, not with itself
    scale = np.abs(D4).max()
    if metric == O.METRIC_L2:
        scale = max(scale, float((xq ** 2).sum(1).max() + (xb[:1000] ** 2).sum(1).max()))
    err = np.abs(D - D4) / np.maximum(np.abs(D4), scale)
    assert err.max() < 1e-4, err.max()
    differ = I != I4
    if differ.any():
        # only where neighbouring distances are within the two kernels' rounding of each other
        assert (np.abs(D[differ] - D4[differ]) <= 1e-4 * scale).all()
    idx.close()

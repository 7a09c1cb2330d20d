"""Generates tests/golden/flat_small.npz: a small seeded case with the oracle's outputs.

The reference ships no golden vectors and cannot be run here (Objective-C++ / Metal,
CPU FAISS not installed), so these vectors pin the ORACLE against accidental change:
they were produced by oracle/flat_oracle.c after it was cross-checked against the pure
numpy restatement (tests/test_oracle.py::test_c_matches_numpy).
Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import flat_oracle as O  # noqa: E402


def main():
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, size=(64, 16)).astype(np.float32)
    xq = rng.uniform(-1, 1, size=(4, 16)).astype(np.float32)
    k = 5
    out = {"xb": xb, "xq": xq, "k": np.int64(k)}
    for name, metric in (("l2", O.METRIC_L2), ("ip", O.METRIC_INNER_PRODUCT)):
        d, i, _ = O.search(metric, xb, xq, k)
        dn, i_n, _ = O.numpy_search(metric, xb, xq, k)
        assert np.array_equal(i, i_n)
        out[name + "_dist"] = d
        out[name + "_labels"] = i
    out["f16_bits"] = O.to_bits16(xb[:8], O.STORAGE_F16)
    out["bf16_bits"] = O.to_bits16(xb[:8], O.STORAGE_BF16)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "flat_small.npz"), **out)


if __name__ == "__main__":
    main()

"""Shared helpers of the parity tests: seeded inputs with the shapes and value
distributions of the benchmark configurations, and the strict / loose comparison
against the CPU oracle."""
import numpy as np

from oracle import flat_oracle as O

TOL_NORTH_STAR = {O.STORAGE_F32: 1e-4, O.STORAGE_F16: 2e-2, O.STORAGE_BF16: 2e-2}
TOL_STRICT = 2e-4  # GPU vs oracle on the SAME (rounded) operands: only fp32 accumulation differs


def uniform_pm1(n, d, seed):
    """The reference's test data: uniform(-1, 1) (tests/test_metal_flat.mm:64-70)."""
    rng = np.random.default_rng(seed)
    return rng.uniform(-1.0, 1.0, size=(n, d)).astype(np.float32)


def mt19937_uniform_pm1(seed, count):
    """`count` draws of std::uniform_real_distribution<float>(-1, 1) from std::mt19937(seed), in
    order: the reference's test-data generator (tests/test_metal_distance.mm:26-31,
    tests/test_metal_flat.mm:64-70) restated for numpy.  std::mt19937(seed) is the standard
    init_genrand seeding, which numpy's legacy RandomState(seed) uses too; the distribution
    takes one 32-bit output per value: float(raw) / 2^32 (a value that rounds up to 1 becomes
    the float below 1), then 2 * u - 1, all in fp32.  Bit-exact against the fixture made from
    the reference's code (tests/golden/ref_loops.npz)."""
    raw = np.random.RandomState(seed)._bit_generator.random_raw(count).astype(np.uint32)
    u = raw.astype(np.float32) / np.float32(4294967296.0)
    u = np.where(u >= np.float32(1.0), np.nextafter(np.float32(1.0), np.float32(0.0)), u).astype(np.float32)
    return (np.float32(2.0) * u + np.float32(-1.0)).astype(np.float32)


def fnv1a64_half(*arrays):
    """Checksum the fixture keeps of inputs too large to commit (FNV-1a 64 over the bytes of the
    arrays in order, shifted right once to fit int64): oracle/ref_loops.cpp, flat_case."""
    h = 1469598103934665603
    for a in arrays:
        for b in np.ascontiguousarray(a).view(np.uint8).ravel().tolist():
            h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h >> 1


def uniform01(n, d, seed):
    rng = np.random.default_rng(seed)
    return rng.random(size=(n, d), dtype=np.float32)


def gaussian(n, d, seed, scale=1.0, normalise=False):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(size=(n, d), dtype=np.float32)
    if normalise:
        x /= np.linalg.norm(x, axis=1, keepdims=True)
    return (x * np.float32(scale)).astype(np.float32)


def mixture(n, d, seed, centres, sigma=0.1):
    rng = np.random.default_rng(seed)
    c = rng.integers(0, centres.shape[0], size=n)
    return (centres[c] + sigma * rng.standard_normal(size=(n, d), dtype=np.float32)).astype(np.float32)


def effective_operands(storage, tensor_path, xb, xq):
    """Operands the GPU path really multiplies: the stored (rounded) database and, on the
    tensor path with 16-bit storage, the queries rounded to the same format."""
    xb_eff = O.round_storage(xb, storage)
    xq_eff = O.round_storage(xq, storage) if (tensor_path and storage != O.STORAGE_F32) else xq
    return xb_eff, xq_eff


def check_against_oracle(metric, storage, tensor_path, xb, xq, k, got_d, got_i, strict=True, loose=True):
    """Runs both comparisons; returns dict of the two result dicts and asserts they pass."""
    out = {}
    got_d = np.asarray(got_d)
    got_i = np.asarray(got_i)
    if strict:
        xb_eff, xq_eff = effective_operands(storage, tensor_path, xb, xq)
        _, ref_i, ref_d = O.search(metric, xb_eff, xq_eff, k)
        true_d = O.rescore(metric, xb_eff, xq_eff, got_i)
        if metric == O.METRIC_L2 and xq_eff is not xq:
            # the kernel adds the exact ||q||^2, the oracle on rounded queries has ||q~||^2
            corr = (np.einsum("ij,ij->i", xq.astype(np.float64), xq.astype(np.float64))
                    - np.einsum("ij,ij->i", xq_eff.astype(np.float64), xq_eff.astype(np.float64)))
            ref_d = ref_d + corr[:, None]
            true_d = true_d + corr[:, None]
        eps = 1e-2 * float(np.nanmax(np.abs(ref_d[np.isfinite(ref_d)]))) if np.isfinite(ref_d).any() else 1e-6
        r = O.compare_results(metric, got_d, got_i, ref_d, ref_i, true_d, TOL_STRICT, eps=max(eps, 1e-6))
        out["strict"] = r
        assert O.passed(r), ("strict", r)
    if loose:
        _, ref_i, ref_d = O.search(metric, xb, xq, k)
        true_d = O.rescore(metric, xb, xq, got_i)
        # relative error is meaningless for scores that cross zero (inner product, large k):
        # the denominator is floored at 10 % of the largest score of the result
        eps = 1e-1 * float(np.nanmax(np.abs(ref_d[np.isfinite(ref_d)]))) if np.isfinite(ref_d).any() else 1e-6
        r = O.compare_results(metric, got_d, got_i, ref_d, ref_i, true_d, TOL_NORTH_STAR[storage], eps=max(eps, 1e-6))
        out["loose"] = r
        assert O.passed(r), ("loose", r)
    # best-first order
    finite = np.isfinite(got_d)
    dd = np.where(finite, got_d, np.nan)
    diffs = np.diff(dd, axis=1)
    if metric == O.METRIC_L2:
        assert not (diffs < -1e-6 * np.maximum(1.0, np.abs(dd[:, 1:]))).any(), "distances not ascending"
    else:
        assert not (diffs > 1e-6 * np.maximum(1.0, np.abs(dd[:, 1:]))).any(), "scores not descending"
    return out

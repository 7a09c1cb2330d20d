"""Generates tests/golden/ref_loops.npz from the reference's own CPU code.

The reference's unit tests hold the only CPU implementation of this path inside the reference
project: seeded std::mt19937 generators and inline fp32 loops for squared norms, squared L2
distances, inner products and the inner-product top-1 (tests/test_metal_distance.mm:23-54,
65-93,105-153,164-227), and the generator of the index tests (tests/test_metal_flat.mm:64-70).
`make -C oracle ref` cuts those lines out of the reference tree and compiles them inside
oracle/ref_loops.cpp; this script runs the binary and packs what it wrote.

It needs the reference checkout (make variable REF) and is therefore run where that tree
exists; the tests only read the committed .npz.

    python tests/golden/make_ref_golden.py

The fixture is reproducible bit for bit: the binary is deterministic (fp32 arithmetic in source
order, no FMA contraction) and numpy's savez stores raw arrays.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
ORACLE = os.path.join(ROOT, "oracle")
DTYPES = {"f32": np.float32, "i64": np.int64}


def main():
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.check_call(["make", "-C", ORACLE, "-s", "ref"], env=env)
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        manifest = subprocess.check_output([os.path.join(ORACLE, "_ref", "ref_loops"), tmp], text=True)
        for line in manifest.splitlines():
            f = line.split()
            name, dtype, dims = f[0], DTYPES[f[1]], tuple(int(x) for x in f[2:])
            a = np.fromfile(os.path.join(tmp, name + ".bin"), dtype=dtype)
            out[name] = a.reshape(dims)
    path = os.path.join(HERE, "ref_loops.npz")
    np.savez(path, **out)
    print("wrote %s: %d arrays, %d bytes" % (path, len(out), os.path.getsize(path)))


if __name__ == "__main__":
    sys.exit(main())

"""Benchmark of the flat k-NN search path.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (config.workload "c3"): IndexFlatL2, BF16 storage, nb = 10,000,000 database
rows, d = 1536, nq = 4,096 fp32 queries, k = 32, components N(0,1) * 0.05 (seeded
synthetic data generated on the device).  The database is row-sharded over the N GPUs
(one process per GPU, launched by torch.distributed.run for N > 1); one step = one
search of all 4,096 queries: shard-local fused GEMM + top-k, NCCL all-gather of the
per-GPU candidates, k-way merge.  Metric: queries per second of the whole job.

value   device-resident: queries and results stay in HBM; timed with CUDA events on the
        stream the kernels run on, max over ranks.
e2e     through the index's public search() with pinned HOST buffers: the host->device
        copy of the queries and the device->host copy of distances + labels are inside
        the timed region.
roofline  tensor-core bound: algorithmic FLOPs (2 * nq * nb_local * d) per launch of the
        fused GEMM kernel / its average duration, measured live with CUDA events around
        each launch in the timed region, against the measured dense BF16 peak.
cpu_baseline / --impl reference  the CPU algorithm of the reference's oracle (sgemm +
        partial select, fp32, all host threads) on a bounded sample of the workload,
        projected to the full database size (cost is linear in nb).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: nb, nq, d, k, storage (0 f32, 1 f16, 2 bf16), metric (1 L2, 0 IP), dist kind, scale
    "c3": dict(nb=10_000_000, nq=4096, d=1536, k=32, storage=2, metric=1, dist=1, scale=0.05,
               desc="IndexFlatL2 BF16 nb=10M nq=4096 d=1536 k=32"),
    "c2": dict(nb=1_000_000, nq=10_000, d=768, k=100, storage=1, metric=0, dist=2, scale=1.0,
               desc="IndexFlatIP FP16 nb=1M nq=10000 d=768 k=100"),
    "c1": dict(nb=100_000, nq=1000, d=128, k=10, storage=0, metric=1, dist=0, scale=1.0,
               desc="IndexFlatL2 FP32 nb=100k nq=1000 d=128 k=10"),
    "c4": dict(nb=5_000_000, nq=2048, d=96, k=1024, storage=0, metric=1, dist=1, scale=1.0,
               desc="IndexFlatL2 FP32 nb=5M nq=2048 d=96 k=1024"),
    "c5": dict(nb=50_000_000, nq=1, d=128, k=10, storage=1, metric=1, dist=0, scale=1.0,
               desc="IndexFlatL2 FP16 nb=50M nq=1 d=128 k=10"),
}
DTYPE_NAME = {0: "f32 (3 x bf16 split, fp32 accumulate)", 1: "f16", 2: "bf16"}
ELEM_BYTES = {0: 4, 1: 2, 2: 2}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            p = json.load(open(path))
            return dict(hbm_gbs=float(p["hbm_gbs"]), bf16_tflops=float(p["bf16_tflops"]),
                        bf16_tflops_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                        source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "samples": len(sm), "reasons": sorted(reasons)}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--nb", type=int, default=0, help="override database rows (not the headline config)")
    ap.add_argument("--nq", type=int, default=0, help="override queries per step (not the headline config)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


# ---------------------------------------------------------------------------------------
# CPU arm: the reference's CPU algorithm (oracle port) on a bounded sample
# ---------------------------------------------------------------------------------------
def cpu_sample_shape(w):
    """Bounded sample: about a second of sgemm per step on a 16-core host."""
    nb_s = min(w["nb"], max(20_000, int(4.0e8 / w["d"])))     # ~1.6 GB of fp32 rows at most
    nq_s = min(w["nq"], 512)
    return nb_s, nq_s


def cpu_make_data(w, nb_s, nq_s):
    import numpy as np
    rng = np.random.default_rng(1)
    if w["dist"] == 0:
        xb = rng.random((nb_s, w["d"]), dtype=np.float32)
        xq = rng.random((nq_s, w["d"]), dtype=np.float32)
    else:
        xb = rng.standard_normal((nb_s, w["d"]), dtype=np.float32)
        xq = rng.standard_normal((nq_s, w["d"]), dtype=np.float32)
        if w["dist"] == 2:
            xb /= np.linalg.norm(xb, axis=1, keepdims=True)
            xq /= np.linalg.norm(xq, axis=1, keepdims=True)
        else:
            xb *= np.float32(w["scale"])
            xq *= np.float32(w["scale"])
    return xb, xq


def cpu_time_steps(w, steps, warmup):
    """Returns (projected QPS on the full workload, ms per step, cores, sample text)."""
    import numpy as np

    from oracle import flat_oracle as O
    nb_s, nq_s = cpu_sample_shape(w)
    xb, xq = cpu_make_data(w, nb_s, nq_s)
    norms = np.einsum("ij,ij->i", xb, xb) if w["metric"] == 1 else None
    cores = os.cpu_count() or 1
    for _ in range(max(1, warmup)):
        O.blas_search(w["metric"], xb, xq, w["k"], xb_norms=norms)
    t0 = time.perf_counter()
    for _ in range(steps):
        O.blas_search(w["metric"], xb, xq, w["k"], xb_norms=norms)
    dt = (time.perf_counter() - t0) / steps
    # cost is linear in the number of database rows: project the sample to the full nb
    qps = nq_s / (dt * (w["nb"] / nb_s))
    sample = ("%d queries x %d of %d rows per step (fp32 sgemm + partial select, OpenBLAS, %d threads), "
              "time scaled by nb/sample rows" % (nq_s, nb_s, w["nb"], cores))
    return qps, dt * 1e3, cores, sample


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    qps, ms, cores, sample = cpu_time_steps(w, args.steps, args.warmup)
    line = {
        "impl": "reference",
        "metric": "QPS (flat kNN %s)" % w["desc"],
        "value": qps, "unit": "queries/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "desc": w["desc"], "nb": w["nb"], "nq": w["nq"], "d": w["d"],
                   "k": w["k"], "note": "CPU FAISS is not installed; this is the oracle's sgemm port"},
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)

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
    "c4": dict(nb=5_000_000, nq=2048, d=96, k=1024, storage=0, metric=1, dist=3, scale=0.1,
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
    ap.add_argument("--storage", type=int, default=-1, help="override the storage type 0/1/2 (not the headline config)")
    ap.add_argument("--ingest", type=float, default=0.0, metavar="GIB",
                    help="only time add() of this many GiB of host rows against a plain pinned copy")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-label-check", action="store_true", help="skip the full-shard oracle label check")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no c5 / c2 / c4 legs)")
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
    elif w["dist"] == 3:
        centres = rng.uniform(-1.0, 1.0, size=(1000, w["d"])).astype(np.float32)
        xb = centres[rng.integers(0, 1000, size=nb_s)] + np.float32(w["scale"]) * rng.standard_normal((nb_s, w["d"]), dtype=np.float32)
        xq = centres[rng.integers(0, 1000, size=nq_s)] + np.float32(w["scale"]) * rng.standard_normal((nq_s, w["d"]), dtype=np.float32)
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
    # torchrun exports OMP_NUM_THREADS=1: give BLAS all host cores back
    cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=cores)
    except Exception:
        pass
    nb_s, nq_s = cpu_sample_shape(w)
    xb, xq = cpu_make_data(w, nb_s, nq_s)
    norms = np.einsum("ij,ij->i", xb, xb) if w["metric"] == 1 else None
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
        # the same keys and values as the B200 arm's config for this N: it names the workload, not the arm
        "config": {"workload": args.workload, "desc": w["desc"], "nb": w["nb"], "nq": w["nq"], "d": w["d"],
                   "k": w["k"], "rows_per_gpu": (w["nb"] + world - 1) // world,
                   "parallelism": "row-sharded x%d, NCCL all-gather + k-way merge" % world,
                   "l2_policy": "inputs larger than L2 (database shard %.1f GB streams every step)"
                                % ((w["nb"] + world - 1) // world * w["d"] * ELEM_BYTES[w["storage"]] / 1e9),
                   "seeds": {"database": 1, "queries": 2},
                   "headline": not (args.nb or args.nq or args.storage >= 0)},
        "note": "the reference's own CPU comparison is CPU FAISS, which is not installed and whose "
                "Metal shaders cannot run here; this arm times the oracle's sgemm + partial-select "
                "port (the algorithm CPU FAISS uses for query batches) on all host cores of this box, "
                "whatever the number of GPUs",
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ---------------------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------------------
def build_shard(fm, torch, res, w, lo, hi, seed):
    """Generates rows [lo, hi) of the synthetic database on the device and adds them."""
    import ctypes
    idx = fm.B200IndexFlat(res, w["d"], w["metric"], w["storage"])
    n = hi - lo
    idx.reserve(max(n, 1))
    chunk = max(1, min(n, (256 << 20) // (w["d"] * 4)))
    buf = torch.empty((chunk, w["d"]), dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for r0 in range(0, n, chunk):
        nr = min(chunk, n - r0)
        fm.abi.check_op(fm.lib().b200f_fill_synthetic(ctypes.c_void_p(buf.data_ptr()), nr, w["d"], lo + r0, seed,
                                                      w["dist"], w["scale"], stream), "fill_synthetic")
        torch.cuda.current_stream().synchronize()
        idx.add(buf[:nr])
    idx.set_label_base(lo)
    del buf
    return idx


TOL_STRICT = 2e-4   # GPU against the oracle on the SAME (stored) operands: only fp32 accumulation differs


def exact_shard_topk(fm, torch, O, w, index_local, lo, hi, xq_sel, rounds_query):
    """The oracle over the WHOLE shard for a few queries, outside the timed region.

    The stored rows are streamed back chunk by chunk (reconstruct_n: the dequantised rows the
    kernels multiply), each chunk goes through the oracle's sgemm search for 2k candidates per
    query, and the union of candidates is re-scored exactly in float64 from the same rows.
    Returns (ref_d float64 [n, k], ref_i int64 [n, k] global labels, fetch) where fetch(labels)
    gives the exact float64 score of arbitrary (query, local-or-global label) pairs of this shard.
    """
    import numpy as np
    d, k, metric = w["d"], w["k"], w["metric"]
    n = xq_sel.shape[0]
    nb = hi - lo
    xq_eff = O.round_storage(xq_sel, w["storage"]) if rounds_query else xq_sel
    kk = min(2 * k, max(nb, 1))
    chunk_rows = max(1, min(nb, (256 << 20) // (d * 4)))
    stage = torch.empty((chunk_rows, d), dtype=torch.float32, pin_memory=True).numpy()
    cand_key = np.empty((n, 0), dtype=np.float32)
    cand_id = np.empty((n, 0), dtype=np.int64)
    for r0 in range(0, nb, chunk_rows):
        nr = min(chunk_rows, nb - r0)
        rows = index_local.reconstruct_n(r0, nr, stage[:nr])
        cd, ci = O.blas_search(metric, rows, xq_eff, min(kk, nr))
        key = cd if metric == O.METRIC_L2 else -cd
        cand_key = np.concatenate([cand_key, key], axis=1)
        cand_id = np.concatenate([cand_id, np.where(ci >= 0, ci + r0, -1)], axis=1)
        if cand_key.shape[1] > 8 * kk:
            sel = np.argpartition(cand_key, kk - 1, axis=1)[:, :kk]
            cand_key = np.take_along_axis(cand_key, sel, axis=1)
            cand_id = np.take_along_axis(cand_id, sel, axis=1)
    if cand_key.shape[1] > kk:
        sel = np.argpartition(cand_key, kk - 1, axis=1)[:, :kk]
        cand_id = np.take_along_axis(cand_id, sel, axis=1)

    q64 = xq_eff.astype(np.float64)
    # the kernel adds the exact ||q||^2 of the unrounded query to -2 q~.x + ||x||^2
    corr = (np.einsum("ij,ij->i", xq_sel.astype(np.float64), xq_sel.astype(np.float64))
            - np.einsum("ij,ij->i", q64, q64)) if (metric == O.METRIC_L2 and rounds_query) else np.zeros(n)
    cache = {}

    def row64(local):
        r = cache.get(local)
        if r is None:
            r = index_local.reconstruct(int(local)).astype(np.float64)
            cache[local] = r
        return r

    def fetch(labels_global):
        out = np.full(labels_global.shape, np.inf if metric == O.METRIC_L2 else -np.inf, dtype=np.float64)
        for qi in range(labels_global.shape[0]):
            for j in range(labels_global.shape[1]):
                lab = int(labels_global[qi, j])
                if lo <= lab < hi:
                    r = row64(lab - lo)
                    out[qi, j] = (((q64[qi] - r) ** 2).sum() + corr[qi]) if metric == O.METRIC_L2 else (q64[qi] * r).sum()
        return out

    pad = np.inf if metric == O.METRIC_L2 else -np.inf
    ref_d = np.full((n, k), pad, dtype=np.float64)
    ref_i = np.full((n, k), -1, dtype=np.int64)
    for qi in range(n):
        ids = np.unique(cand_id[qi][cand_id[qi] >= 0])
        if ids.size == 0:
            continue
        exact = np.array([(((q64[qi] - row64(i)) ** 2).sum() + corr[qi]) if metric == O.METRIC_L2
                          else (q64[qi] * row64(i)).sum() for i in ids])
        key = exact if metric == O.METRIC_L2 else -exact
        order = np.lexsort((ids, key))[:k]
        ref_i[qi, :order.size] = ids[order] + lo
        ref_d[qi, :order.size] = exact[order]
    return ref_d, ref_i, fetch


def label_check(fm, torch, dist, O, w, index_local, lo, hi, rank, world, xq_host, D_host, I_host, nsample=16):
    """Label parity at the size the step ran on: for `nsample` of the step's queries the merged
    GPU result must equal the oracle's exact top-k over the whole database (strict tolerance:
    same stored rows, same rounded queries; a differing label must be a proven tie).  With
    several ranks each rank also checks its own shard's list against the oracle over its
    shard, and rank 0 merges the ranks' exact lists on the host."""
    import numpy as np
    nq, k, metric = xq_host.shape[0], w["k"], w["metric"]
    sel = np.unique(np.linspace(0, nq - 1, num=min(nsample, nq)).astype(np.int64))
    xq_sel = np.ascontiguousarray(xq_host[sel])
    # 16-bit rows: the tensor path and the streaming scan multiply the query rounded to the storage format
    rounds_query = w["storage"] != 0 and (nq > 8 or (hi - lo) >= 65536)
    t0 = time.perf_counter()
    ref_d, ref_i, fetch = exact_shard_topk(fm, torch, O, w, index_local, lo, hi, xq_sel, rounds_query)
    out = {"label_queries": int(sel.size), "labels_checked": int(sel.size * k), "label_tolerance": TOL_STRICT}
    finite = np.isfinite(ref_d)
    eps = max(1e-2 * float(np.abs(ref_d[finite]).max()) if finite.any() else 1e-6, 1e-6)
    if world > 1:
        # this rank's own list over its shard
        Dl, Il = index_local.search(xq_sel, k)
        r = O.compare_results(metric, Dl, Il, ref_d, ref_i, fetch(Il), TOL_STRICT, eps=eps)
        local_bad = 0 if O.passed(r) else 1
        gathered = [None] * world
        dist.all_gather_object(gathered, (ref_d, ref_i, local_bad, r))
        out["shard_lists_bad"] = int(sum(g[2] for g in gathered))
        if rank == 0:
            d_all = np.stack([g[0] for g in gathered])
            i_all = np.stack([g[1] for g in gathered])
            key = d_all if metric == O.METRIC_L2 else -d_all
            key = np.transpose(key, (1, 0, 2)).reshape(sel.size, -1)
            ids = np.transpose(i_all, (1, 0, 2)).reshape(sel.size, -1)
            key = np.where(ids >= 0, key, np.inf)
            order = np.stack([np.lexsort((ids[q], key[q]))[:k] for q in range(sel.size)])
            ref_i = np.take_along_axis(ids, order, axis=1)
            ref_d = np.take_along_axis(np.transpose(d_all, (1, 0, 2)).reshape(sel.size, -1), order, axis=1)
        # exact scores of the labels the merged result holds: each rank scores the labels that
        # are rows of its shard (+/-INF elsewhere), rank 0 combines
        share = [I_host[sel] if rank == 0 else None]
        dist.broadcast_object_list(share, src=0)
        box = [None] * world
        dist.all_gather_object(box, fetch(share[0]))
        if rank == 0:
            true_d = np.min(np.stack(box), axis=0) if metric == O.METRIC_L2 else np.max(np.stack(box), axis=0)
    else:
        true_d = fetch(I_host[sel])
    if rank == 0:
        r = O.compare_results(metric, D_host[sel], I_host[sel], ref_d, ref_i, true_d, TOL_STRICT, eps=eps)
        out.update({"label_diff": r["label_diff"], "label_bad": r["label_bad"], "dist_bad": r["dist"],
                    "pad_mismatch": r["pad_mismatch"], "duplicates": r["duplicates"],
                    "max_rel_dist_err_vs_stored_operands": r["max_rel_dist_err"],
                    "label_check_seconds": round(time.perf_counter() - t0, 2),
                    "label_check": "GPU top-k of %d queries against the oracle's exact top-k over all %d rows "
                            "(stored rows read back, float64 re-score)" % (sel.size, w["nb"])})
        if not O.passed(r) or out.get("shard_lists_bad", 0):
            raise AssertionError("label check failed: %r" % (out,))
    return out


def spot_check(fm, torch, w, index_local, lo, hi, xq_host, D, I, nsample=8):
    """Outside the timed region: exact re-score (float64, from the stored rows) of the labels
    returned for a few queries that fall in this rank's shard against the UNROUNDED queries:
    the north-star distance tolerance (1e-4 FP32 storage, 2e-2 16-bit storage) and the order."""
    import numpy as np
    worst = 0.0
    checked = 0
    for qi in range(min(nsample, xq_host.shape[0])):
        prev = None
        for j in range(I.shape[1]):
            lab = int(I[qi, j])
            if lab < 0:
                continue
            dist = float(D[qi, j])
            if prev is not None:
                assert (dist >= prev - 1e-5 * abs(prev)) if w["metric"] == 1 else (dist <= prev + 1e-5 * abs(prev)), \
                    "results are not best-first"
            prev = dist
            if not (lo <= lab < hi):
                continue
            row = index_local.reconstruct(lab - lo).astype(np.float64)
            q = xq_host[qi].astype(np.float64)
            exact = float(((q - row) ** 2).sum()) if w["metric"] == 1 else float((q * row).sum())
            err = abs(exact - dist) / max(abs(exact), 1e-6)
            worst = max(worst, err)
            checked += 1
    tol = 1e-4 if w["storage"] == 0 else 2e-2
    assert worst <= tol, "distance error %g above tolerance %g" % (worst, tol)
    return {"pairs_rescored": checked, "max_rel_dist_err": worst, "tolerance": tol}


def run_workload(ctx, name, w, steps, warmup, headline, with_e2e=True, with_label_check=True):
    """Builds the workload's index on this rank's shard, times it, checks it, frees it.
    Returns the dict of everything measured (rank 0) or None."""
    import ctypes

    import numpy as np

    fm, torch, dist, O = ctx["fm"], ctx["torch"], ctx["dist"], ctx["O"]
    rank, world, local_rank, res, ext, peaks = (ctx[k] for k in ("rank", "world", "local_rank", "res", "ext", "peaks"))
    L = fm.lib()
    lo, hi = fm.shard_range(w["nb"], rank, world)
    nq, d, k = w["nq"], w["d"], w["k"]
    root = rank == 0

    with torch.cuda.stream(ext):
        index = build_shard(fm, torch, res, w, lo, hi, seed=1)
        sharded = fm.ShardedIndexFlat(index, rank, world)
        xq_dev = torch.empty((nq, d), dtype=torch.float32, device="cuda")
        fm.abi.check_op(L.b200f_fill_synthetic(ctypes.c_void_p(xq_dev.data_ptr()), nq, d, 0, 2, w["dist"], w["scale"],
                                               ctypes.c_void_p(ext.cuda_stream)), "fill queries")
        ext.synchronize()
        xq_pin = torch.empty((nq, d), dtype=torch.float32, pin_memory=True)
        xq_pin.copy_(xq_dev)
        d_pin = torch.empty((nq, k), dtype=torch.float32, pin_memory=True)
        l_pin = torch.empty((nq, k), dtype=torch.int64, pin_memory=True)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        batch = 16384 if k <= 1024 else 1024   # queries per launch of the library

        def step_device():
            # queries and results resident in HBM; every launch of a step queued back to back,
            # one host synchronisation per step; only rank 0 merges
            if nq <= batch:
                return sharded.search_device(xq_dev, k, want_result=root)
            return sharded.search(xq_dev, k, want_result=root)

        def step_e2e():
            # the public call with HOST buffers: each rank uploads its slice of the queries, the
            # slices are all-gathered over NVLink, rank 0 alone merges and downloads the result
            if world == 1:
                index.search(xq_pin.numpy(), k, d_pin.numpy(), l_pin.numpy())
            elif root:
                sharded.search(xq_pin.numpy(), k, d_pin.numpy(), l_pin.numpy())
            else:
                sharded.search(xq_pin.numpy(), k, want_result=False)

        # ---- device-resident timing ------------------------------------------------------
        sampler = ClockSampler(local_rank)
        if root:
            sampler.start()  # started before the warm-up so that its own start-up is not timed
        for _ in range(max(warmup, 3)):
            step_device()
        barrier()
        L.b200f_profile_enable(1)
        L.b200f_profile_read(None, None, None, 1)
        sampler.lines.clear()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        barrier()
        evs[0].record(ext)
        for i in range(steps):
            D_dev, I_dev = step_device()
            evs[i + 1].record(ext)
        barrier()
        clocks = sampler.stop() if root else None
        ms_total = evs[0].elapsed_time(evs[-1])
        step_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
        launches = ctypes.c_int64(0)
        main_launches = ctypes.c_int64(0)
        main_ms = ctypes.c_double(0.0)
        L.b200f_profile_read(ctypes.byref(launches), ctypes.byref(main_launches), ctypes.byref(main_ms), 1)
        L.b200f_profile_enable(0)
        t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item()) / steps
        # the dominant kernel's time per step on every rank: a step ends when the slowest shard
        # has been searched (the exchange waits for it), so the spread between the GPUs (clocks
        # under the power cap) shows up as waiting time on the faster ranks
        kernel_ms_by_rank = None
        if world > 1:
            km = torch.zeros(world, dtype=torch.float64, device="cuda")
            km[rank] = main_ms.value / max(1, steps)
            dist.all_reduce(km, op=dist.ReduceOp.SUM)
            kernel_ms_by_rank = [round(v, 4) for v in km.cpu().tolist()]

        # ---- end-to-end timing -------------------------------------------------------------
        e2e = None
        if with_e2e:
            for _ in range(3):
                step_e2e()
            barrier()
            t0 = time.perf_counter()
            for _ in range(steps):
                step_e2e()
            barrier()
            dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            e2e_s = float(dt.item()) / steps
            e2e = {"value": nq / e2e_s, "unit": "queries/s", "ms_per_step": e2e_s * 1e3,
                   "h2d_bytes_per_step": nq * d * 4, "d2h_bytes_per_step": nq * k * 12,
                   "what": "index search() with pinned host buffers; each GPU uploads 1/%d of the queries, "
                           "GPU 0 alone downloads the merged result" % world}

        # ---- latency distribution of a stream of single searches (small-nq workloads) ------
        latency = None
        if nq <= 4 and with_e2e:
            # 10,000 calls unless that would take much longer than ~25 s
            ncalls = max(1000, min(10000, int(25000.0 / max(ms_step, 0.05))))
            qbank = torch.empty((64 * nq, d), dtype=torch.float32, device="cuda")
            fm.abi.check_op(L.b200f_fill_synthetic(ctypes.c_void_p(qbank.data_ptr()), 64 * nq, d, 0, 3, w["dist"],
                                                   w["scale"], ctypes.c_void_p(ext.cuda_stream)), "fill query bank")
            ext.synchronize()
            qbank_pin = torch.empty((64 * nq, d), dtype=torch.float32, pin_memory=True)
            qbank_pin.copy_(qbank)
            qb = qbank_pin.numpy()
            lat = []
            lat_sampler = ClockSampler(local_rank)
            if root:
                lat_sampler.start()
            for i in range(4):   # the second call of a shape captures its graph: keep that out of the record
                (index.search(qb[:nq], k, d_pin.numpy(), l_pin.numpy()) if world == 1 else
                 sharded.search(qb[:nq], k, d_pin.numpy() if root else None, l_pin.numpy() if root else None,
                                want_result=root))
            if world > 1:
                sharded.trace(True)
            barrier()
            for i in range(ncalls):
                j = (i % 64) * nq
                t0 = time.perf_counter()
                if world == 1:
                    index.search(qb[j:j + nq], k, d_pin.numpy(), l_pin.numpy())
                elif root:
                    sharded.search(qb[j:j + nq], k, d_pin.numpy(), l_pin.numpy())
                else:
                    sharded.search(qb[j:j + nq], k, want_result=False)
                lat.append((time.perf_counter() - t0) * 1e3)
            trace = None
            if world > 1:
                # Where does a slow call lose its time?  Per call and rank: microseconds on the host
                # until everything was enqueued, then microseconds waiting for the device.  A call
                # is only as fast as its slowest rank (the all-gather waits for every shard), so
                # one rank that is late on the host shows as a long device wait on all the others.
                enq, wait = sharded.read_trace()
                sharded.trace(False)
                per_rank = [None] * world
                dist.all_gather_object(per_rank, (enq[:ncalls].tolist(), wait[:ncalls].tolist()))
                if root:
                    enq_all = np.array([p[0] for p in per_rank])      # [world, calls]
                    wait_all = np.array([p[1] for p in per_rank])
                    total = (enq_all + wait_all).max(axis=0)
                    med = float(np.median(total))
                    slow = total > 1.5 * med
                    late_host = enq_all.max(axis=0) > np.median(enq_all) + 50.0   # some rank enqueued > 50 us late
                    trace = {"calls": int(total.size), "median_call_us": med,
                             "median_enqueue_us": float(np.median(enq_all)),
                             "p99_enqueue_us_worst_rank": float(np.percentile(enq_all.max(axis=0), 99)),
                             "slow_calls": int(slow.sum()),
                             "slow_calls_with_a_rank_late_on_the_host": int((slow & late_host).sum()),
                             "slow_calls_per_rank_latest": np.bincount(enq_all[:, slow].argmax(axis=0), minlength=world).tolist()
                             if slow.any() else [0] * world,
                             "what": "slow = call longer than 1.5 x the median; late = a rank took > 50 us longer than "
                                     "the median to enqueue its work"}
            lat_t = torch.tensor(lat, dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(lat_t, op=dist.ReduceOp.MAX)   # a call ends when the slowest rank has it
            lat_all = lat_t.cpu().tolist()
            lat_s = sorted(lat_all)
            head, tail = sorted(lat_all[:500]), sorted(lat_all[-500:])
            latency = {"calls": ncalls, "p50_ms": lat_s[len(lat_s) // 2], "p99_ms": lat_s[int(len(lat_s) * 0.99)],
                       "max_ms": lat_s[-1], "p50_first_500_ms": head[len(head) // 2], "p50_last_500_ms": tail[len(tail) // 2],
                       "clocks": lat_sampler.stop() if root else None, "trace": trace,
                       "what": "host-timed search() with host buffers, one query batch per call"}
            qbank = qbank_pin = lat_t = None
            step_e2e()   # leaves the benchmark queries' result in the pinned arrays again

        # ---- checks outside the timed region ---------------------------------------------
        D_host = D_dev.cpu().numpy() if root else None
        I_host = I_dev.cpu().numpy() if root else None
        check = None
        if root:
            check = spot_check(fm, torch, w, index, lo, hi, xq_pin.numpy(), D_host, I_host)
            if with_e2e:
                assert np.array_equal(l_pin.numpy(), I_host), "end-to-end labels differ from device-resident labels"
        if with_label_check:
            lc = label_check(fm, torch, dist, O, w, index, lo, hi, rank, world, xq_pin.numpy(), D_host, I_host)
            if root:
                check.update(lc)

    # every torch tensor that lived on the library's stream must be released before that stream
    # is destroyed (torch records an event on the allocation stream when it frees a block)
    D_dev = I_dev = xq_dev = xq_pin = d_pin = l_pin = t = evs = None  # noqa: F841
    sharded.close()
    index.close()
    import gc
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    if not root:
        return None

    nb_local = hi - lo
    # DRAM bytes of the dominant kernel from ncu captures on smaller shards of the same workload
    # (dram__bytes_read.sum + dram__bytes_write.sum of one launch), scaled by the rows a full
    # launch scans: the traffic of both kernels grows in proportion to the rows of the shard.
    #   c3: filter-mode gemm_topk_kernel, 1,250,000 rows: 4,694.8 MB + 25.2 MB
    #   c5: scan_mma_kernel, 8,000,000 rows: 2,176 MB + 3.7 MB
    traffic = None
    if name == "c3" and w["nq"] == WORKLOADS["c3"]["nq"]:
        traffic = (4694.8e6 + 25.2e6) / 1_250_000 * nb_local
    elif name == "c5":
        traffic = (2176.0e6 + 3.7e6) / 8_000_000 * nb_local
    flops_per_launch = 2.0 * nq * nb_local * d
    bytes_per_launch = nb_local * d * ELEM_BYTES[w["storage"]] + nq * d * 4 + nq * k * 12
    n_main = max(1, main_launches.value)
    main_avg_ms = main_ms.value / n_main
    tensor_bound = nq > 64
    if tensor_bound:
        # a step may launch the kernel several times (pilot pass, filter pass, query batches):
        # credit the step's algorithmic FLOPs against the summed duration of its launches
        launches_per_step = max(1.0, main_launches.value / max(1, steps))
        achieved = flops_per_launch / (main_avg_ms * launches_per_step * 1e-3) / 1e12 if main_avg_ms > 0 else 0.0
        peak = peaks["bf16_tflops_sustained"] if ms_step * steps > 1000 else peaks["bf16_tflops"]
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak, "traffic": traffic, "traffic_unit": "bytes per step (scaled from an ncu capture)", "kernel": "gemm_topk_kernel",
                    "kernel_ms_avg": main_avg_ms, "kernel_launches": main_launches.value,
                    "kernel_launches_per_step": launches_per_step,
                    "peak_source": peaks["source"] + (" sustained" if peak == peaks["bf16_tflops_sustained"] else " burst"),
                    "frac_of_burst_peak": achieved / peaks["bf16_tflops"],
                    "frac_of_nominal_2250": achieved / 2250.0}
    else:
        achieved = bytes_per_launch / (main_avg_ms * 1e-3) / 1e9 if main_avg_ms > 0 else 0.0
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_unit": "bytes per launch (scaled from an ncu capture)",
                    "kernel": "scan_mma_kernel" if w["storage"] != 0 else "scan_kernel",
                    "kernel_ms_avg": main_avg_ms, "kernel_launches": main_launches.value,
                    "peak_source": peaks["source"], "frac_of_nominal_8000": achieved / 8000.0}
    return {
        "metric": "QPS (flat kNN %s)" % w["desc"],
        "value": nq / (ms_step * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": steps,
        "warmup": max(warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE_NAME[w["storage"]].split(" ")[0], "data": "synthetic",
        "config": {"workload": name, "desc": w["desc"], "nb": w["nb"], "nq": nq, "d": d, "k": k,
                   "rows_per_gpu": nb_local, "parallelism": "row-sharded x%d, NCCL all-gather + k-way merge" % world,
                   "l2_policy": "inputs larger than L2 (database shard %.1f GB streams every step)"
                                % (nb_local * d * ELEM_BYTES[w["storage"]] / 1e9),
                   "seeds": {"database": 1, "queries": 2},
                   "headline": headline},
        "roofline": dict(roofline, kernel_ms_per_step_by_rank=kernel_ms_by_rank), "e2e": e2e,
        "gpu_launches": int(launches.value),
        "latency": latency, "clocks": clocks, "check": check, "step_ms": [round(x, 3) for x in step_ms],
    }


def run_ingest(ctx, w, gib=4.0):
    """Host -> index throughput of add() (the ingest pipeline: pinned or pageable host rows, 32 MiB
    chunks, upload overlapped with the conversion kernel) against a plain pinned cudaMemcpyAsync
    of the same bytes.  Rows are fp32 on the host, as a caller of add() has them."""
    import numpy as np
    fm, torch, res, ext = ctx["fm"], ctx["torch"], ctx["res"], ctx["ext"]
    d = w["d"]
    n = int(gib * (1 << 30) / (d * 4))
    nbytes = n * d * 4
    out = {"rows": n, "bytes": nbytes, "storage": DTYPE_NAME[w["storage"]].split(" ")[0]}
    with torch.cuda.stream(ext):
        pinned = torch.empty((n, d), dtype=torch.float32, pin_memory=True)
        pinned.normal_(0.0, 0.05)
        dev = torch.empty((n, d), dtype=torch.float32, device="cuda")
        # the yardstick: one asynchronous copy from pinned memory
        best = 1e9
        for _ in range(3):
            ext.synchronize()
            t0 = time.perf_counter()
            dev.copy_(pinned, non_blocking=True)
            ext.synchronize()
            best = min(best, time.perf_counter() - t0)
        out["pinned_memcpy_gbs"] = nbytes / best / 1e9
        del dev
        pageable = pinned.numpy().copy()
        for name, src in (("pinned", pinned.numpy()), ("pageable", pageable)):
            best = 1e9
            for _ in range(2):
                idx = fm.B200IndexFlat(res, d, w["metric"], w["storage"])
                idx.reserve(n)
                ext.synchronize()
                t0 = time.perf_counter()
                idx.add(src)
                best = min(best, time.perf_counter() - t0)
                idx.close()
            out["add_from_%s_gbs" % name] = nbytes / best / 1e9
            out["add_from_%s_vs_memcpy" % name] = out["add_from_%s_gbs" % name] / out["pinned_memcpy_gbs"]
        del pinned, pageable
    torch.cuda.empty_cache()
    return out


def run_b200(args, w, rank, world, local_rank):
    import torch
    import torch.distributed as dist

    import faiss_metal_b200 as fm
    from oracle import flat_oracle as O   # the checker of the label checks and the CPU baseline leg

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    res = fm.StandardB200Resources(local_rank)
    ext = torch.cuda.ExternalStream(res.stream, device=torch.device("cuda", local_rank))
    ctx = {"fm": fm, "torch": torch, "dist": dist, "O": O, "rank": rank, "world": world, "local_rank": local_rank,
           "res": res, "ext": ext, "peaks": load_peaks()}
    headline = not (args.nb or args.nq or args.storage >= 0)
    if args.ingest:
        if rank == 0:
            emit({"ingest": run_ingest(ctx, w, args.ingest), "config": {"workload": args.workload, "d": w["d"]}})
        res.close()
        return
    line = run_workload(ctx, args.workload, w, args.steps, args.warmup, headline, with_e2e=not args.no_e2e,
                        with_label_check=not args.no_label_check)

    # The other north-star configurations, a few steps each, attached to the same line: the
    # headline keys above are untouched.
    extras = {}
    if headline and args.workload == "c3" and not args.no_extras:
        for name in ("c5", "c2", "c4"):
            try:
                extras[name] = run_workload(ctx, name, dict(WORKLOADS[name]), max(3, min(args.steps, 10)), 3, False,
                                            with_e2e=not args.no_e2e, with_label_check=not args.no_label_check)
            except Exception as e:   # an extra must never take the headline down with it
                # (checks raise after a workload's last collective call, so the ranks stay in step)
                extras[name] = {"error": "%s: %s" % (type(e).__name__, e)}
        if world == 1:
            try:
                extras["ingest"] = run_ingest(ctx, w)
            except Exception as e:
                extras["ingest"] = {"error": "%s: %s" % (type(e).__name__, e)}

    def teardown():
        torch.cuda.synchronize()
        res.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    if rank != 0:
        teardown()
        return
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        qps_c, ms_c, cores, sample = cpu_time_steps(w, 3, 1)
        cpu = {"value": qps_c, "unit": "queries/s", "cores": cores, "kind": "port", "sample": sample}
    line["cpu_baseline"] = cpu
    if extras:
        line["extra_configs"] = extras
    emit(line)
    teardown()


_RESULT_FD = None


def emit(line: dict):
    """The one JSON line of the run, on the process's original stdout."""
    text = json.dumps(line) + "\n"
    if _RESULT_FD is not None:
        os.write(_RESULT_FD, text.encode())
    else:
        sys.stdout.write(text)
        sys.stdout.flush()


def main():
    # Libraries may print to stdout on their own (NCCL writes its version line there when the
    # first communicator is created): everything but the result line goes to stderr.
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    args = parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.nb:
        w["nb"] = args.nb
    if args.nq:
        w["nq"] = args.nq
    if args.storage >= 0:
        w["storage"] = args.storage
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if world != args.gpus:
        if args.gpus > 1 and world == 1:
            raise SystemExit("--gpus %d needs one process per GPU: launch with "
                             "python -m torch.distributed.run --nproc-per-node %d bench.py ..." % (args.gpus, args.gpus))
    run_b200(args, w, rank, world, local_rank)


if __name__ == "__main__":
    main()

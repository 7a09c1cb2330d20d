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
        "config": {"workload": args.workload, "desc": w["desc"], "nb": w["nb"], "nq": w["nq"], "d": w["d"],
                   "k": w["k"], "seeds": {"database": 1, "queries": 2}, "headline": not (args.nb or args.nq),
                   "note": "the reference's own CPU comparison is CPU FAISS, which is not installed and whose "
                           "Metal shaders cannot run here; this arm times the oracle's sgemm + partial-select "
                           "port (the algorithm CPU FAISS uses for query batches) on all host cores"},
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


def spot_check(fm, torch, w, index_local, lo, hi, xq_host, D, I, nsample=8):
    """Outside the timed region: exact re-score (float64, from the stored rows) of the labels
    returned for a few queries that fall in this rank's shard, order and tolerance check."""
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


def run_b200(args, w, rank, world, local_rank):
    import ctypes

    import numpy as np
    import torch
    import torch.distributed as dist

    import faiss_metal_b200 as fm

    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks()
    res = fm.StandardB200Resources(local_rank)
    ext = torch.cuda.ExternalStream(res.stream, device=torch.device("cuda", local_rank))
    lo, hi = fm.shard_range(w["nb"], rank, world)
    L = fm.lib()

    with torch.cuda.stream(ext):
        index = build_shard(fm, torch, res, w, lo, hi, seed=1)
        sharded = fm.ShardedIndexFlat(index, rank, world)
        nq, d, k = w["nq"], w["d"], w["k"]
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

        single_batch = nq <= (16384 if k <= 32 else 1024)

        def step_device():
            if single_batch:   # queued back to back on one stream, one host sync per step
                return sharded.search_device(xq_dev, k)
            return sharded.search(xq_dev, k)

        def step_e2e():
            # public API with HOST buffers: H2D of the queries and D2H of the results inside
            if world == 1:
                index.search(xq_pin.numpy(), k, d_pin.numpy(), l_pin.numpy())
            else:
                if single_batch:
                    dd, ll = sharded.search_device(xq_dev.copy_(xq_pin, non_blocking=True), k, sync=False)
                else:
                    dd, ll = sharded.search(xq_dev.copy_(xq_pin, non_blocking=True), k)
                d_pin.copy_(dd, non_blocking=True)
                l_pin.copy_(ll, non_blocking=True)
                index.synchronize()

        # ---- device-resident timing ------------------------------------------------------
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()  # started before the warm-up so that its own start-up is not timed
        for _ in range(max(args.warmup, 3)):
            step_device()
        barrier()
        L.b200f_profile_enable(1)
        L.b200f_profile_read(None, None, None, 1)
        sampler.lines.clear()
        evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        barrier()
        evs[0].record(ext)
        for i in range(args.steps):
            D_dev, I_dev = step_device()
            evs[i + 1].record(ext)
        barrier()
        clocks = sampler.stop() if rank == 0 else None
        ms_total = evs[0].elapsed_time(evs[-1])
        step_ms = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
        launches = ctypes.c_int64(0)
        main_launches = ctypes.c_int64(0)
        main_ms = ctypes.c_double(0.0)
        L.b200f_profile_read(ctypes.byref(launches), ctypes.byref(main_launches), ctypes.byref(main_ms), 1)
        L.b200f_profile_enable(0)
        t = torch.tensor([ms_total], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step = float(t.item()) / args.steps

        # ---- end-to-end timing -------------------------------------------------------------
        e2e = None
        if not args.no_e2e:
            for _ in range(2):
                step_e2e()
            barrier()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                step_e2e()
            barrier()
            dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            e2e_s = float(dt.item()) / args.steps
            e2e = {"value": nq / e2e_s, "unit": "queries/s", "ms_per_step": e2e_s * 1e3,
                   "h2d_bytes_per_step": world * nq * d * 4, "d2h_bytes_per_step": world * nq * k * 12}

        # ---- latency distribution of a stream of single searches (small-nq workloads) ------
        latency = None
        if nq <= 4 and not args.no_e2e:
            # 10,000 calls unless that would take much longer than ~25 s
            ncalls = max(1000, min(10000, int(25000.0 / max(ms_step, 0.05))))
            qbank = torch.empty((64 * nq, d), dtype=torch.float32, device="cuda")
            fm.abi.check_op(L.b200f_fill_synthetic(ctypes.c_void_p(qbank.data_ptr()), 64 * nq, d, 0, 3, w["dist"],
                                                   w["scale"], ctypes.c_void_p(ext.cuda_stream)), "fill query bank")
            ext.synchronize()
            qbank_pin = torch.empty((64 * nq, d), dtype=torch.float32, pin_memory=True)
            qbank_pin.copy_(qbank)
            lat = []
            barrier()
            for i in range(ncalls):
                j = (i % 64) * nq
                t0 = time.perf_counter()
                if world == 1:
                    index.search(qbank_pin[j:j + nq].numpy(), k, d_pin.numpy(), l_pin.numpy())
                else:
                    dd, ll = sharded.search_device(xq_dev.copy_(qbank_pin[j:j + nq], non_blocking=True), k, sync=False)
                    d_pin.copy_(dd, non_blocking=True)
                    l_pin.copy_(ll, non_blocking=True)
                    index.synchronize()
                lat.append((time.perf_counter() - t0) * 1e3)
            lat_t = torch.tensor(lat, dtype=torch.float64, device="cuda")
            if world > 1:
                dist.all_reduce(lat_t, op=dist.ReduceOp.MAX)   # a call ends when the slowest rank has it
            lat_s = sorted(lat_t.cpu().tolist())
            latency = {"calls": ncalls, "p50_ms": lat_s[len(lat_s) // 2], "p99_ms": lat_s[int(len(lat_s) * 0.99)],
                       "max_ms": lat_s[-1], "what": "host-timed search() with host buffers, one query batch per call"}
            qbank = qbank_pin = lat_t = None
            # restore the benchmark queries for the checks below
            fm.abi.check_op(L.b200f_fill_synthetic(ctypes.c_void_p(xq_dev.data_ptr()), nq, d, 0, 2, w["dist"],
                                                   w["scale"], ctypes.c_void_p(ext.cuda_stream)), "fill queries")
            ext.synchronize()
            D_dev, I_dev = step_device()
            step_e2e()

        # ---- checks outside the timed region ---------------------------------------------
        D_host = D_dev.cpu().numpy()
        I_host = I_dev.cpu().numpy()
        check = spot_check(fm, torch, w, index, lo, hi, xq_pin.numpy(), D_host, I_host)
        if not args.no_e2e:
            assert np.array_equal(l_pin.numpy(), I_host), "end-to-end labels differ from device-resident labels"

    # every torch tensor that lived on the library's stream must be released before that stream
    # is destroyed (torch records an event on the allocation stream when it frees a block)
    D_dev = I_dev = xq_dev = xq_pin = d_pin = l_pin = t = dt = sharded = evs = ev_unused = None  # noqa: F841
    import gc
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()

    def teardown():
        # ordered: index, resources, then the process group
        torch.cuda.synchronize()
        index.close()
        res.close()
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()

    if rank != 0:
        teardown()
        return

    nb_local = hi - lo
    # DRAM bytes of the dominant kernel from ncu captures on smaller shards of the same workload
    # (dram__bytes_read.sum + dram__bytes_write.sum of one launch), scaled by the rows a full
    # launch scans: the traffic of both kernels grows in proportion to the rows of the shard.
    #   c3: filter-mode gemm_topk_kernel, 1,250,000 rows: 4,694.8 MB + 25.2 MB
    #   c5: scan_mma_kernel, 8,000,000 rows: 2,176 MB + 3.7 MB
    traffic = None
    if args.workload == "c3" and w["nq"] == WORKLOADS["c3"]["nq"]:
        traffic = (4694.8e6 + 25.2e6) / 1_250_000 * nb_local
    elif args.workload == "c5":
        traffic = (2176.0e6 + 3.7e6) / 8_000_000 * nb_local
    flops_per_launch = 2.0 * nq * nb_local * d
    bytes_per_launch = nb_local * d * ELEM_BYTES[w["storage"]] + nq * d * 4 + nq * k * 12
    n_main = max(1, main_launches.value)
    main_avg_ms = main_ms.value / n_main
    tensor_bound = nq > 64
    if tensor_bound:
        # a step may launch the kernel several times (column chunks, query batches): credit the
        # step's algorithmic FLOPs against the summed duration of its launches
        launches_per_step = max(1.0, main_launches.value / max(1, args.steps))
        achieved = flops_per_launch / (main_avg_ms * launches_per_step * 1e-3) / 1e12 if main_avg_ms > 0 else 0.0
        peak = peaks["bf16_tflops_sustained"] if ms_step * args.steps > 1000 else peaks["bf16_tflops"]
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
                    "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "traffic_unit": "bytes per launch (scaled from an ncu capture)", "kernel": "scan_mma_kernel",
                    "kernel_ms_avg": main_avg_ms, "kernel_launches": main_launches.value,
                    "peak_source": peaks["source"], "frac_of_nominal_8000": achieved / 8000.0}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        qps_c, ms_c, cores, sample = cpu_time_steps(w, 3, 1)
        cpu = {"value": qps_c, "unit": "queries/s", "cores": cores, "kind": "port", "sample": sample}

    line = {
        "metric": "QPS (flat kNN %s)" % w["desc"],
        "value": nq / (ms_step * 1e-3), "unit": "queries/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE_NAME[w["storage"]].split(" ")[0], "data": "synthetic",
        "config": {"workload": args.workload, "desc": w["desc"], "nb": w["nb"], "nq": nq, "d": d, "k": k,
                   "rows_per_gpu": nb_local, "parallelism": "row-sharded x%d, NCCL all-gather + k-way merge" % world,
                   "l2_policy": "inputs larger than L2 (database shard %.1f GB streams every step)"
                                % (nb_local * d * ELEM_BYTES[w["storage"]] / 1e9),
                   "seeds": {"database": 1, "queries": 2},
                   "headline": not (args.nb or args.nq)},
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches.value),
        "latency": latency, "clocks": clocks, "check": check, "step_ms": [round(x, 3) for x in step_ms],
    }
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

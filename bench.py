#!/usr/bin/env python
"""Benchmark of the IVF-PQ search path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the deep-embedding-shaped configuration -- 10,000,000 x 96 fp32 L2-normalised
draws from a 4,096-component anisotropic Gaussian mixture (seed 1), 10,000 queries, n_lists 50,000,
pq_dim 48, pq_bits 8, k = 10, fp16 look-up table, fp32 internal distances, n_probes swept over
{20, 50, 100, 200}, one batch of 10,000 queries per step.  The public dataset this imitates is not
available offline; the seeded synthetic generator below stands in for it.

A step = one search of the whole query batch.  `value` is queries/s with queries resident in HBM;
`e2e` is the same through the C interface with pinned host buffers and the copies inside the timed
region.  Times come from CUDA events on the stream the library launches on (torch's current
stream); the code-scan kernel is timed by the library's own events around its launch.

--impl reference times the CPU oracle (the port of the reference search arithmetic, all host
threads) on a bounded sample of the same queries against the same index.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(name="deep-embedding-shaped L2, 10M x 96 f32", n_rows=10_000_000, dim=96,
                n_components=4096, seed=1, n_queries=10_000, n_lists=50_000, pq_dim=48, pq_bits=8,
                k=10, probes=(20, 50, 100, 200), lut="float16", internal="float32",
                kmeans_n_iters=10, kmeans_trainset_fraction=0.1, refine_ratio=2)
# A second, optional workload (--workload sift): the SIFT-shaped integer configuration in miniature
# (one GPU's share of it): long lists, 8-bit look-up table, k = 100 -- the regime where the code scan
# rather than the look-up-table build dominates.  Not the headline; used for the scan roofline.
SIFT_WORKLOAD = dict(name="SIFT-shaped L2, 20M x 128 u8", kind="sift", n_rows=20_000_000, dim=128,
                     n_components=16384, seed=2, n_queries=10_000, n_lists=20_000, pq_dim=64,
                     pq_bits=8, k=100, probes=(64,), lut="uint8", internal="float32",
                     kmeans_n_iters=10, kmeans_trainset_fraction=0.1, refine_ratio=1)
METRIC = "IVF-PQ search QPS @ recall@10>=0.95"
FALLBACK_HBM_GBS = 6650.0


def log(*a):
    if int(os.environ.get("RANK", "0")) == 0:
        print(*a, file=sys.stderr, flush=True)


# --------------------------------------------------------------------------------------------
# synthetic data (seeded per chunk, so any prefix or shard can be regenerated independently)
# --------------------------------------------------------------------------------------------
def mixture_model(wl, device):
    import torch
    g = torch.Generator(device="cpu").manual_seed(wl["seed"] * 7919 + 17)
    if wl.get("kind") == "sift":
        # centres in [0, 120] plus a per-dimension exponential offset (mean 20): mass skewed to 0-40
        centers = torch.rand(wl["n_components"], wl["dim"], generator=g) * 60.0
        centers = centers + torch.empty(wl["n_components"], wl["dim"]).exponential_(1.0 / 20.0, generator=g)
        scales = torch.full((wl["n_components"], wl["dim"]), 12.0)
        return centers.to(device), scales.to(device)
    centers = torch.randn(wl["n_components"], wl["dim"], generator=g)
    lo, hi = np.log(0.05), np.log(0.5)
    scales = torch.exp(torch.rand(wl["n_components"], wl["dim"], generator=g) * (hi - lo) + lo)
    # per-component scale is relative to the centre norm, so clusters keep their identity after
    # the rows are L2-normalised
    scales = scales * (centers.norm(dim=1, keepdim=True) / np.sqrt(wl["dim"]))
    return centers.to(device), scales.to(device)


def gen_rows(wl, model, start, count, device, stream_id=0):
    import torch
    centers, scales = model
    g = torch.Generator(device=device).manual_seed(wl["seed"] * 1_000_003 + start + stream_id * 977)
    comp = torch.randint(0, wl["n_components"], (count,), generator=g, device=device)
    x = centers[comp] + scales[comp] * torch.randn(count, wl["dim"], generator=g, device=device)
    if wl.get("kind") == "sift":
        return x.round_().clamp_(0, 255).to(torch.uint8)
    return torch.nn.functional.normalize(x, dim=1)


def gen_dataset(wl, device):
    import torch
    model = mixture_model(wl, device)
    x = torch.empty((wl["n_rows"], wl["dim"]), device=device,
                    dtype=torch.uint8 if wl.get("kind") == "sift" else torch.float32)
    step = 1_000_000
    for s in range(0, wl["n_rows"], step):
        c = min(step, wl["n_rows"] - s)
        x[s:s + c] = gen_rows(wl, model, s, c, device)
    q = gen_rows(wl, model, 0, wl["n_queries"], device, stream_id=1)
    return x, q


def ground_truth(x, q, k):
    """Exact top-k by squared L2 distance, fp32, in row chunks."""
    import torch
    q = q.float()
    qn = (q * q).sum(1, keepdim=True)
    best_d = torch.full((q.shape[0], k), float("inf"), device=q.device)
    best_i = torch.zeros((q.shape[0], k), dtype=torch.int64, device=q.device)
    step = 200_000
    for s in range(0, x.shape[0], step):
        xb = x[s:s + step].float()
        d = qn + (xb * xb).sum(1)[None, :] - 2.0 * (q @ xb.T)
        dd, ii = torch.topk(d, k, dim=1, largest=False)
        cat_d = torch.cat([best_d, dd], 1)
        cat_i = torch.cat([best_i, ii + s], 1)
        best_d, sel = torch.topk(cat_d, k, dim=1, largest=False)
        best_i = torch.gather(cat_i, 1, sel)
    return best_i


def recall_at_k(found, truth):
    import torch
    hits = (found.unsqueeze(2) == truth.unsqueeze(1)).any(2).sum().item()
    return hits / truth.numel()


# --------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.samples, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            p = [t.strip() for t in s.split(",")]
            try:
                sm.append(float(p[0]))
                mx.append(float(p[1]))
                for n, v in zip(names, p[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# --------------------------------------------------------------------------------------------
# fixture: dataset, index file, ground truth -- cached in a temp dir for back-to-back runs
# --------------------------------------------------------------------------------------------
def cache_dir(wl):
    key = hashlib.sha1(json.dumps(wl, sort_keys=True, default=str).encode()).hexdigest()[:12]
    base = "/dev/shm" if os.path.isdir("/dev/shm") else tempfile.gettempdir()
    d = os.path.join(base, f"cuvs_b200_bench_{key}")
    os.makedirs(d, exist_ok=True)
    return d


def prepare_fixture(wl, device, need_dataset=False):
    """Returns dict(index_path, queries (device), truth (device), build_s).  Builds what is missing."""
    import torch

    from cuvs_b200 import ivf_pq
    d = cache_dir(wl)
    ipath, qpath, tpath = (os.path.join(d, n) for n in ("index.ivfpq", "queries.npy", "truth.npy"))
    done = os.path.join(d, "done")
    out = {"index_path": ipath, "build_s": None, "dir": d}
    if not os.path.exists(done):
        t0 = time.time()
        x, q = gen_dataset(wl, device)
        torch.cuda.synchronize()
        log(f"[bench] generated {tuple(x.shape)} in {time.time() - t0:.1f}s")
        t0 = time.time()
        params = ivf_pq.IndexParams(n_lists=wl["n_lists"], pq_dim=wl["pq_dim"], pq_bits=wl["pq_bits"],
                                    kmeans_n_iters=wl["kmeans_n_iters"],
                                    kmeans_trainset_fraction=wl["kmeans_trainset_fraction"])
        index = ivf_pq.build(params, x)
        torch.cuda.synchronize()
        out["build_s"] = time.time() - t0
        log(f"[bench] built index in {out['build_s']:.1f}s")
        t0 = time.time()
        truth = ground_truth(x, q, wl["k"])
        torch.cuda.synchronize()
        log(f"[bench] exact ground truth in {time.time() - t0:.1f}s")
        ivf_pq.save(ipath, index)
        np.save(qpath, q.cpu().numpy())
        np.save(tpath, truth.cpu().numpy())
        del x, index
        torch.cuda.empty_cache()
        open(done, "w").write("ok")
    out["queries"] = torch.from_numpy(np.load(qpath)).to(device)
    out["truth"] = torch.from_numpy(np.load(tpath)).to(device)
    if need_dataset:      # regenerated from the seeds (refinement reads the original vectors)
        out["dataset"] = gen_dataset(wl, device)[0]
    return out


# --------------------------------------------------------------------------------------------
# CPU baseline (oracle port), bounded sample
# --------------------------------------------------------------------------------------------
def cpu_baseline(index_path, queries_np, wl, n_probes, budget_s=12.0, steps=1, warmup=0,
                 dataset_np=None):
    """The CPU port on all host threads: IVF-PQ search for k0 candidates and, when the workload
    refines, exact re-ranking of those candidates with numpy."""
    from oracle import oracle as O
    t0 = time.time()
    ix = O.OracleIndex.load(index_path)
    ix.flat()
    log(f"[bench] oracle loaded the index in {time.time() - t0:.1f}s")
    cores = O.lib().orc_num_threads()
    lut = {"float32": O.CUDA_R_32F, "float16": O.CUDA_R_16F, "uint8": O.CUDA_R_8U}[wl["lut"]]
    internal = {"float32": O.CUDA_R_32F, "float16": O.CUDA_R_16F}[wl["internal"]]
    k = wl["k"]
    k0 = int(wl["refine_ratio"] * k) if (wl["refine_ratio"] > 1 and dataset_np is not None) else k

    def run(q):
        d, i = O.search(ix, q, k0, n_probes=n_probes, lut_dtype=lut, internal_dtype=internal)
        if k0 > k:
            safe = np.where(i == O.OUT_OF_BOUNDS, 0, i)
            v = dataset_np[safe]                                   # [n, k0, dim]
            dd = ((v - q[:, None, :]) ** 2).sum(2)
            dd = np.where(i == O.OUT_OF_BOUNDS, np.inf, dd)
            o = np.argsort(dd, axis=1)[:, :k]
            i = np.take_along_axis(i, o, 1)
        return i

    # size the sample from a probe run
    n0 = min(len(queries_np), max(cores, 32))
    t0 = time.time()
    run(queries_np[:n0])
    per_q = (time.time() - t0) / n0
    n = int(min(len(queries_np), max(n0, budget_s / max(per_q, 1e-9))))
    times = []
    for it in range(warmup + steps):
        t0 = time.time()
        run(queries_np[:n])
        if it >= warmup:
            times.append(time.time() - t0)
    dt = float(np.mean(times))
    what = f"first {n} of {len(queries_np)} queries, n_probes={n_probes}, k={k}"
    if k0 > k:
        what += f", {k0} candidates re-ranked exactly"
    return {"value": n / dt, "unit": "queries/s", "cores": int(cores), "kind": "port",
            "sample": what + "; same index file; C port of the reference arithmetic, OpenMP over queries"}, dt, n


# --------------------------------------------------------------------------------------------
def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


# DRAM bytes (read + write) per DISTINCT 32-row group scanned in a launch, from the ncu capture of the
# scan kernel on a 4 M-row case of this workload (246.8 MB over 135,125 distinct groups of
# 3 x 512 B; summary under profiles/).  Traffic grows with the distinct groups of a launch, so the
# full-size figure is this constant times the launch's distinct groups.
DRAM_BYTES_PER_UNIQUE_GROUP = 1826.0


def workload_from_args(args):
    wl = dict(SIFT_WORKLOAD if args.workload == "sift" else WORKLOAD)
    if args.rows:
        per_list = wl["n_rows"] // wl["n_lists"]
        wl.update(n_rows=args.rows, n_lists=max(64, args.rows // per_list),
                  n_queries=min(wl["n_queries"], max(100, args.rows // 100)))
    if args.refine_ratio is not None:
        wl["refine_ratio"] = args.refine_ratio
    return wl


def run_ours(args):
    import ctypes as C

    import torch
    import torch.distributed as dist

    from cuvs_b200 import _lib as L
    from cuvs_b200 import ivf_pq, mg, refine
    from cuvs_b200.common import default_resources

    wl = workload_from_args(args)
    probes = tuple(int(p) for p in args.probes.split(",")) if args.probes else wl["probes"]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        # keep stdout to the one JSON line (NCCL prints its version banner there at VERSION level)
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=device)
    res = default_resources()
    lib = L.load()
    k = wl["k"]
    k0 = int(wl["refine_ratio"] * k) if wl["refine_ratio"] > 1 else k
    refining = k0 > k

    # ---- fixture: rank 0 builds (or finds) it, everyone loads its shard ----
    if rank == 0:
        fx = prepare_fixture(wl, device, need_dataset=refining)
    if world > 1:
        dist.barrier()
    if rank != 0:
        fx = prepare_fixture(wl, device, need_dataset=refining)
    index = mg.load_shard(fx["index_path"], rank, world, res) if world > 1 else ivf_pq.load(fx["index_path"])
    queries, truth = fx["queries"], fx["truth"]
    dataset = fx.get("dataset")
    nq = queries.shape[0]
    lut_dt = {"float32": np.float32, "float16": np.float16, "uint8": np.uint8}[wl["lut"]]
    int_dt = {"float32": np.float32, "float16": np.float16}[wl["internal"]]

    def make_sp(p):
        return ivf_pq.SearchParams(n_probes=p, lut_dtype=lut_dt, internal_distance_dtype=int_dt,
                                   max_internal_batch_size=max(nq, 1))

    cand_i = torch.empty((nq, k0), dtype=torch.int64, device=device)
    cand_d = torch.empty((nq, k0), dtype=torch.float32, device=device)
    out_i0 = torch.empty((nq, k), dtype=torch.int64, device=device)
    out_d0 = torch.empty((nq, k), dtype=torch.float32, device=device)

    def one_search(sp, q=None, outs=None):
        """The whole step: IVF-PQ search for k0 candidates (+ merge across ranks) and, with a
        refine ratio above 1, exact re-ranking down to k."""
        q = queries if q is None else q
        out_i, out_d = outs if outs is not None else (out_i0, out_d0)
        if world > 1:
            d, i = mg.search(sp, index, q, k0, True, None, res, sync=False)
        else:
            d, i = ivf_pq.search(sp, index, q, k0, cand_i, cand_d, res, sync=False)
        if refining:
            d, i = refine(dataset, q, i, k=k, metric="sqeuclidean", indices=out_i, distances=out_d,
                          resources=res, sync=False)
        elif outs is not None:
            out_i.copy_(i)
            out_d.copy_(d)
            d, i = out_d, out_i
        return d, i

    def timed(fn, steps, warmup, tail=None):
        for _ in range(warmup):
            fn()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t_host = time.perf_counter()
        for _ in range(steps):
            fn()
        t_host = time.perf_counter() - t_host
        if tail is not None:
            tail()          # e.g. make the timing stream wait for copies still in flight
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if rank == 0:
            log(f"[bench] timed {steps} steps: device {ms / steps:.3f} ms/step, "
                f"host issue {t_host / steps * 1e3:.3f} ms/step")
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = t.item()
        return ms / steps

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()

    # ---- recall / QPS sweep over n_probes ----
    sweep = []
    for p in probes:
        sp = make_sp(p)
        d, i = one_search(sp)
        torch.cuda.synchronize()
        rec = recall_at_k(i, truth)
        ms = timed(lambda: one_search(sp), max(2, min(args.steps, 5)), 2)
        sweep.append({"n_probes": p, "recall_at_10": round(rec, 4), "qps": round(nq / ms * 1e3, 1),
                      "ms_per_batch": round(ms, 3)})
        log(f"[bench] n_probes={p}: recall@10={rec:.4f}  {nq / ms * 1e3:,.0f} q/s")
    ok = [s for s in sweep if s["recall_at_10"] >= 0.95]
    if ok:
        chosen, target_met = ok[0], True
    else:
        best = max(s["recall_at_10"] for s in sweep)
        chosen = [s for s in sweep if s["recall_at_10"] >= best - 0.005][0]
        target_met = False
    p_star = chosen["n_probes"]
    sp = make_sp(p_star)

    # ---- the timed region: K steps, device-resident queries ----
    L.check(lib.cuvsB200StatsEnable(res.handle, True))
    stats = L.SearchStats()
    one_search(sp)
    L.check(lib.cuvsB200StatsGet(res.handle, C.byref(stats), True))
    launches_before = stats.launches
    ms_step = timed(lambda: one_search(sp), args.steps, args.warmup)
    ms_single = ms_step
    # Throughput mode: two batches in flight per GPU, each on its own stream and resources handle
    # (the serving pattern of the reference's benchmark in throughput mode: several host threads, one
    # stream each), so that the small kernels (and, with several GPUs, the NCCL exchanges) of one batch
    # fill the tails of the other's large kernels.
    # The per-kernel figures above (stage times, roofline, launches) come from the single-stream pass.
    n_streams = 1
    if True:
        from cuvs_b200.common import Resources
        n_streams = 2
        lanes = []
        for _ in range(n_streams):
            lanes.append(dict(stream=torch.cuda.Stream(device), res=Resources(),
                              ci=torch.empty_like(cand_i), cd=torch.empty_like(cand_d),
                              oi=torch.empty_like(out_i0), od=torch.empty_like(out_d0)))
        lane_state = {"i": 0}

        def lane_search(q, outs=None, stream_wait=None):
            """One step on the next lane; returns the lane (its stream carries the step)."""
            lane = lanes[lane_state["i"] % n_streams]
            lane_state["i"] += 1
            with torch.cuda.stream(lane["stream"]):
                if stream_wait is not None:
                    for ev in stream_wait:
                        lane["stream"].wait_event(ev)
                lane["res"].use_current_stream()
                if world > 1:
                    d, i = mg.search(sp, index, q, k0, True, None, lane["res"], sync=False)
                else:
                    d, i = ivf_pq.search(sp, index, q, k0, lane["ci"], lane["cd"], lane["res"], sync=False)
                oi, od = outs if outs is not None else (lane["oi"], lane["od"])
                if refining:
                    refine(dataset, q, i, k=k, metric="sqeuclidean", indices=oi, distances=od,
                           resources=lane["res"], sync=False)
                elif outs is not None:
                    oi.copy_(i)
                    od.copy_(d)
            return lane

        def lanes_join():
            main = torch.cuda.current_stream()
            for lane in lanes:
                main.wait_stream(lane["stream"])

        for lane in lanes:
            lane["stream"].wait_stream(torch.cuda.current_stream())
        ms_step = timed(lambda: lane_search(queries), args.steps, args.warmup + n_streams, tail=lanes_join)
        log(f"[bench] {n_streams} batches in flight: {ms_step:.4f} ms/step (one at a time: {ms_single:.4f})")
    L.check(lib.cuvsB200StatsGet(res.handle, C.byref(stats), True))
    n_calls = args.steps + args.warmup
    gpu_launches = int(round((stats.launches - launches_before) * args.steps / n_calls))
    scan_ms = stats.scan_ms / max(1, stats.batches)
    n_pieces = -(-wl["pq_dim"] // (128 // wl["pq_bits"]))
    bytes_scan = stats.scan_groups / max(1, stats.batches) * n_pieces * 512
    bytes_unique = stats.unique_groups / max(1, stats.batches) * n_pieces * 512
    stage = {k2: round(getattr(stats, k2) / max(1, stats.batches), 4)
             for k2 in ("prep_ms", "coarse_ms", "sort_ms", "scan_ms", "merge_ms")}
    L.check(lib.cuvsB200StatsEnable(res.handle, False))
    if refining:
        stage["refine_ms"] = round(timed(lambda: refine(dataset, queries, cand_i, k=k, indices=out_i0,
                                                        distances=out_d0, resources=res, sync=False),
                                         args.steps, 1), 4)

    # ---- the configuration's small batches (1 and 100 queries): latency per call, synchronised ----
    small = []
    if not args.no_e2e:
        for b in (1, 100):
            if b >= nq:
                continue
            qb = queries[:b].contiguous()
            cb_i = torch.empty((b, k0), dtype=torch.int64, device=device)
            cb_d = torch.empty((b, k0), dtype=torch.float32, device=device)
            ob_i = torch.empty((b, k), dtype=torch.int64, device=device)
            ob_d = torch.empty((b, k), dtype=torch.float32, device=device)

            def small_step():
                if world > 1:
                    d, i = mg.search(sp, index, qb, k0, True, None, res, sync=False)
                else:
                    d, i = ivf_pq.search(sp, index, qb, k0, cb_i, cb_d, res, sync=False)
                if refining:
                    refine(dataset, qb, i, k=k, metric="sqeuclidean", indices=ob_i, distances=ob_d,
                           resources=res, sync=False)
                torch.cuda.synchronize()      # latency mode: the caller waits for every batch

            for _ in range(5):
                small_step()
            t0 = time.perf_counter()
            n_rep = 50
            for _ in range(n_rep):
                small_step()
            dt = (time.perf_counter() - t0) / n_rep
            small.append({"batch": b, "latency_ms": round(dt * 1e3, 4), "qps": round(b / dt, 1)})
            log(f"[bench] batch {b}: {dt * 1e3:.3f} ms per call, {b / dt:,.0f} q/s")

    # ---- end to end: pinned host buffers, copies inside the timed region ----
    # Every step copies its queries host -> device and its results device -> host.  The copies run on
    # their own streams with two sets of buffers, so that step s+1's input copy and step s-1's
    # result copy overlap step s's search (a serving loop's usual double buffering); the timed
    # region ends only when the last result has reached the host.
    q_host = queries.cpu().pin_memory()
    q_dev = [torch.empty_like(queries) for _ in range(2)]
    o_dev = [(torch.empty((nq, k), dtype=torch.int64, device=device),
              torch.empty((nq, k), dtype=torch.float32, device=device)) for _ in range(2)]
    i_host = [torch.empty((nq, k), dtype=torch.int64).pin_memory() for _ in range(2)]
    d_host = [torch.empty((nq, k), dtype=torch.float32).pin_memory() for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    e2e_state = {"step": 0}

    def e2e_step():
        s = e2e_state["step"]
        slot = s & 1
        main = torch.cuda.current_stream()
        with torch.cuda.stream(s_in):
            if s >= 2:
                s_in.wait_event(ev_done[slot])       # the search two steps back has read this buffer
            q_dev[slot].copy_(q_host, non_blocking=True)
            ev_in[slot].record(s_in)
        if n_streams > 1:
            # the search runs on its lane's stream, behind this step's input copy and the result
            # copy that last used the output buffer
            lane = lane_search(q_dev[slot], o_dev[slot], [ev_in[slot]] + ([ev_out[slot]] if s >= 2 else []))
            ev_done[slot].record(lane["stream"])
        else:
            main.wait_event(ev_in[slot])
            if s >= 2:
                main.wait_event(ev_out[slot])        # its results have left this output buffer
            one_search(sp, q_dev[slot], o_dev[slot])
            ev_done[slot].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[slot])
            i_host[slot].copy_(o_dev[slot][0], non_blocking=True)
            d_host[slot].copy_(o_dev[slot][1], non_blocking=True)
            ev_out[slot].record(s_out)
        e2e_state["step"] = s + 1

    def e2e_tail():
        main = torch.cuda.current_stream()
        for ev in ev_out:
            main.wait_event(ev)
        if n_streams > 1:
            lanes_join()

    if args.no_e2e:
        ms_e2e, e2e_rec = float("nan"), float("nan")
    else:
        ms_e2e = timed(e2e_step, args.steps, args.warmup, tail=e2e_tail)
        last = (e2e_state["step"] - 1) & 1
        e2e_rec = recall_at_k(i_host[last].to(device), truth)
    clocks = sampler.stop() if rank == 0 else None

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = hbm_peak()
    achieved = bytes_scan / (scan_ms * 1e-3) / 1e9 if scan_ms > 0 else None
    traffic = int(DRAM_BYTES_PER_UNIQUE_GROUP * stats.unique_groups / max(1, stats.batches))
    line = {
        "metric": METRIC, "value": round(nq / ms_step * 1e3, 1), "unit": "queries/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None,
        "dtype": "f32" if wl["lut"] != "uint8" else "f32 (8-bit float look-up table)",
        "data": "synthetic",
        "config": {"workload": wl["name"], "n_rows": wl["n_rows"], "dim": wl["dim"],
                   "n_lists": wl["n_lists"], "pq_dim": wl["pq_dim"], "pq_bits": wl["pq_bits"],
                   "k": k, "recall_k": k, "batch": nq, "n_probes": p_star, "lut_dtype": wl["lut"],
                   "internal_distance_dtype": wl["internal"], "refine_ratio": wl["refine_ratio"],
                   "recall_at_10": chosen["recall_at_10"],
                   "recall_target_met": target_met, "sweep": sweep, "small_batches": small,
                   "parallelism": f"list-sharded x{world}" if world > 1 else "single GPU",
                   "batches_in_flight": n_streams, "ms_per_step_one_batch_in_flight": round(ms_single, 4),
                   "l2": f"inputs larger than L2: {wl['n_rows'] * n_pieces * 16 // 1_000_000} MB of codes per pass",
                   "stage_ms": stage, "build_s": fx.get("build_s")},
        "e2e": {"value": round(nq / ms_e2e * 1e3, 1), "unit": "queries/s",
                "h2d_bytes_per_step": int(q_host.numel() * q_host.element_size()),
                "d2h_bytes_per_step": int(nq * k * 12), "ms_per_step": round(ms_e2e, 4),
                "copies": "every step, double-buffered on side streams (overlap the neighbouring steps)",
                "recall_at_10": round(e2e_rec, 4)},
        "gpu_launches": gpu_launches,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "scan_kernel (LUT build + code scan + top-k)",
                     "achieved": round(achieved, 1) if achieved else None, "peak": peak,
                     "peak_kind": f"of {peak_kind}", "unit": "GB/s",
                     "frac": round(achieved / peak, 4) if achieved else None,
                     "traffic": traffic, "algorithmic_bytes_per_launch": int(bytes_scan),
                     "unique_bytes_per_launch": int(bytes_unique),
                     "kernel_ms": round(scan_ms, 4)},
    }
    if world == 1 and not args.no_cpu:
        cb, _, _ = cpu_baseline(fx["index_path"], queries.cpu().numpy(), wl, p_star,
                                dataset_np=dataset.cpu().numpy() if refining else None)
        cb["value"] = round(cb["value"], 1)
        line["cpu_baseline"] = cb
    emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference arm: the CPU port of the reference search on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = workload_from_args(args)
    import torch
    if not torch.cuda.is_available():
        emit({"impl": "reference",
              "unavailable": "the 10M-vector index fixture is built on the GPU; no GPU here"})
        return
    torch.cuda.set_device(0)
    k = wl["k"]
    k0 = int(wl["refine_ratio"] * k) if wl["refine_ratio"] > 1 else k
    fx = prepare_fixture(wl, torch.device("cuda", 0), need_dataset=k0 > k)
    # operating point: the same rule as the GPU arm, evaluated with the GPU search (fixture work)
    from cuvs_b200 import ivf_pq, refine
    index = ivf_pq.load(fx["index_path"])
    lut_dt = {"float32": np.float32, "float16": np.float16, "uint8": np.uint8}[wl["lut"]]
    recs = []
    for p in wl["probes"]:
        d, i = ivf_pq.search(ivf_pq.SearchParams(n_probes=p, lut_dtype=lut_dt,
                                                 max_internal_batch_size=fx["queries"].shape[0]),
                             index, fx["queries"], k0)
        if k0 > k:
            d, i = refine(fx["dataset"], fx["queries"], i, k=k)
        recs.append((p, recall_at_k(i, fx["truth"])))
    ok = [p for p, r in recs if r >= 0.95]
    best = max(r for _, r in recs)
    p_star = ok[0] if ok else [p for p, r in recs if r >= best - 0.005][0]
    del index
    dataset_np = fx["dataset"].cpu().numpy() if k0 > k else None
    fx.pop("dataset", None)
    torch.cuda.empty_cache()
    cb, dt, n = cpu_baseline(fx["index_path"], fx["queries"].cpu().numpy(), wl, p_star,
                             budget_s=8.0, steps=args.steps, warmup=args.warmup, dataset_np=dataset_np)
    line = {"impl": "reference", "metric": METRIC, "value": round(cb["value"], 1), "unit": "queries/s",
            "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["name"], "n_rows": wl["n_rows"], "dim": wl["dim"],
                       "n_lists": wl["n_lists"], "pq_dim": wl["pq_dim"], "pq_bits": wl["pq_bits"],
                       "k": wl["k"], "batch": n, "n_probes": p_star, "lut_dtype": wl["lut"],
                       "internal_distance_dtype": wl["internal"], "refine_ratio": wl["refine_ratio"]},
            "cpu_baseline": dict(cb, value=round(cb["value"], 1)),
            "e2e": {"value": round(cb["value"], 1), "unit": "queries/s", "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    emit(line)


def emit(line: dict):
    """Write the one JSON line to the process's original stdout."""
    data = (json.dumps(line) + "\n").encode()
    os.write(_REAL_STDOUT, data)


_REAL_STDOUT = 1


def main():
    # Libraries (NCCL's version banner, for one) print to stdout; the contract is ONE JSON line
    # there.  Keep the original stdout for that line and point fd 1 at stderr for everything else.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=0, help="shrink the dataset (testing only)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload", default="deep", choices=["deep", "sift"],
                    help="deep = the headline configuration; sift = long-list integer data (scan roofline)")
    ap.add_argument("--probes", default="", help="comma-separated n_probes to sweep (default: the workload's)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--refine-ratio", type=float, default=None,
                    help="candidates fetched per result before exact re-ranking (1 = no refinement)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

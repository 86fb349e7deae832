#!/usr/bin/env python
"""Benchmark of the RSFK K-NN-graph build on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

A step is one complete K-NN-graph build of the workload (all trees, every leaf
bucket, the exploration sweeps).  Rank 0 prints ONE JSON line.

* ``value``  : points/s with the points already resident in HBM (CUDA events,
               max over ranks).
* ``e2e``    : the same build through the host-buffer entry point the reference
               wrapper binds (``pymodule_rsfk_knn`` via ``gpu_rsfk.RSFK``), host
               to device and device to host copies inside the timed region.
* ``roofline``: the dominant kernel's algorithmic bytes per launch over its
               average CUDA-event duration, against the measured HBM copy peak.
* ``cpu_baseline``: exact brute-force KNN (the CPU oracle's OpenMP routine) on a
               bounded sample of query rows, all host cores.

``--impl reference`` times the reference project's own CUDA library (built from
its unmodified sources into oracle/_ref by ``make -C oracle ref``) through the
same C ABI, in a child process, on the same workload.

Data are seeded synthetic stand-ins with the shapes and distributions of the
configurations (no dataset is downloaded).
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "gpu-rsfk_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

# name: N, D, K, trees, min, max, sweeps, generator
WORKLOADS = {
    "c1": dict(N=20_000, D=32, K=16, trees=4, min=32, max=128, sweeps=1, gen="uniform", seed=0),
    "c2": dict(N=1_000_000, D=100, K=32, trees=50, min=33, max=66, sweeps=1, gen="uniform", seed=0),
    "c3": dict(N=4_000_000, D=2, K=32, trees=32, min=256, max=1024, sweeps=1, gen="gauss2d", seed=1),
    "c4": dict(N=1_000_000, D=960, K=32, trees=20, min=33, max=2048, sweeps=2, gen="gauss960", seed=2),
    "c5": dict(N=20_000_000, D=128, K=64, trees=64, min=65, max=130, sweeps=2, gen="bytes128", seed=3),
    # query (base/query) search in the shape of the reference's own experiment (test_ann.py:40-160:
    # 3 M word vectors reduced to 32 dimensions, half of them as base set, the query set equal to the
    # base set, K=32, buckets of 32..256 points, 5..30 trees); one GPU
    "ann": dict(N=1_500_000, D=32, K=32, trees=20, min=32, max=256, sweeps=0, gen="mix32", seed=4),
}

# DRAM bytes (read+write) per launch of the dominant kernel from the committed
# ncu capture, per unit processed; None until a capture exists.  Filled from
# the summaries under profiles/.
# (ncu --set full captures of a 400 000-point case of c2, summaries under profiles/; traffic grows
# in proportion to the points a launch processes)
NCU_TRAFFIC_PER_POINT = {"explore": 58.81e9 / 400_000, "bucket_knn": 359.7e6 / 400_000,
                         "tree_project": 174.1e6 / 400_000, "tree_subtrees": 702.5e6 / 400_000}


# (DRAM read + write bytes) / algorithmic bytes of the sweep kernel in the committed captures
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {("c4", "explore"): ((492.004e9 + 0.011e9) / 615.675e9, "300 000-point"),
                                    ("c5", "explore"): ((975.550e9 + 12.547e9) / 1082.055e9, "2 000 000-point")}


def dominant_phase(phases):
    """The phase whose kernel took the most time in total.  Phases within 2 % of the largest count
    as tied (on the 1 M x 100 build the projection's 753 launches and the sweep's single launch are
    0.3 % apart and swap places from run to run); among tied phases the one with the fewest
    launches, i.e. the largest single kernel, is named."""
    names = [n for n in phases if n != "tree_level_rest"]
    top = max(phases[n]["total_ms"] for n in names)
    tied = [n for n in names if phases[n]["total_ms"] >= 0.98 * top]
    return min(tied, key=lambda n: (phases[n]["launches"], -phases[n]["total_ms"]))


def make_points(w, n_override=None):
    N = n_override or w["N"]
    D = w["D"]
    if w["gen"] == "uniform":
        np.random.seed(w["seed"])
        return np.random.uniform(0, 1, (N, D)).astype(np.float32)
    rng = np.random.default_rng(w["seed"])
    if w["gen"] == "gauss2d":
        c = rng.uniform(0, 100, (64, 2))
        return (c[rng.integers(0, 64, N)] + rng.normal(0, 1.0, (N, 2))).astype(np.float32)
    if w["gen"] == "gauss960":
        c = rng.normal(0, 1, (100, D))
        out = np.empty((N, D), np.float32)
        for s in range(0, N, 100_000):
            e = min(N, s + 100_000)
            out[s:e] = c[rng.integers(0, 100, e - s)] + rng.normal(0, 0.3, (e - s, D))
        return out
    if w["gen"] == "mix32":
        # stand-in for PCA-reduced embeddings: 200 clusters, variance falling with the dimension
        spectrum = 1.0 / np.sqrt(1.0 + np.arange(D))
        c = rng.normal(0, 1, (200, D)) * spectrum
        out = np.empty((N, D), np.float32)
        for s in range(0, N, 250_000):
            e = min(N, s + 250_000)
            out[s:e] = c[rng.integers(0, 200, e - s)] + rng.normal(0, 0.5, (e - s, D)) * spectrum
        return out
    if w["gen"] == "bytes128":
        c = rng.integers(0, 256, (1000, D)).astype(np.float32)
        out = np.empty((N, D), np.float32)
        for chunk, s in enumerate(range(0, N, 1_000_000)):
            e = min(N, s + 1_000_000)
            r = np.random.default_rng([w["seed"], chunk])
            out[s:e] = np.clip(np.rint(c[r.integers(0, 1000, e - s)] + r.normal(0, 12, (e - s, D))), 0, 255)
        return out
    raise ValueError(w["gen"])


# --------------------------------------------------------------------------- clocks
class ClockSampler(object):
    """Samples SM clock and throttle reasons through NVML (read-only) while the
    timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread:
            self._thread.join()

    def summary(self):
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# --------------------------------------------------------------------------- ours
class TimedEngine(object):
    """DeviceForest proxy that brackets each phase with CUDA events on the
    launching stream."""

    def __init__(self, engine):
        import torch
        self._e, self._torch = engine, torch
        self.records = {"forest": [], "merge": [], "explore": []}
        self.stats = []
        self.enabled = False

    def init_lists(self, *a, **k):
        return self._e.init_lists(*a, **k)

    def _timed(self, key, fn, *a, **k):
        if not self.enabled:
            return fn(*a, **k)
        t = self._torch
        e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        e0.record()
        out = fn(*a, **k)
        e1.record()
        self.records[key].append((e0, e1))
        return out

    def forest(self, *a, **k):
        before = self._e.stats()
        out = self._timed("forest", self._e.forest, *a, **k)
        if self.enabled:
            after = self._e.stats()
            self.stats.append({n: after[n] - before[n] for n in after})
        return out

    def merge_lists(self, *a, **k):
        return self._timed("merge", self._e.merge_lists, *a, **k)

    def explore(self, *a, **k):
        before = self._e.stats()
        out = self._timed("explore", self._e.explore, *a, **k)
        if self.enabled:
            self._e.synchronize()
            after = self._e.stats()
            self.stats.append({n: after[n] - before[n] for n in after})
        return out

    def total_ms(self, key):
        return sum(a.elapsed_time(b) for a, b in self.records[key])


def exact_knn_torch(points_dev, queries, K):
    """Exact KNN of the query rows on the GPU (evaluation only, torch)."""
    import torch
    q = torch.as_tensor(queries, device=points_dev.device, dtype=torch.long)
    out = []
    step = max(1, int(2.5e8 // points_dev.shape[0]))
    for s in range(0, len(q), step):
        d = torch.cdist(points_dev[q[s:s + step]], points_dev, compute_mode="donot_use_mm_for_euclid_dist")
        out.append(torch.topk(d, K, dim=1, largest=False).indices.to(torch.int32))
    return torch.cat(out)


def recall_of(truth, approx):
    hit = 0
    for t, a in zip(truth, approx):
        hit += len(set(t.tolist()) & set(a.tolist()))
    return hit / float(truth.shape[0] * truth.shape[1])


def run_ours(args, w):
    import torch
    import torch.distributed as dist
    from gpu_rsfk import RSFK
    from gpu_rsfk.device import DeviceForest
    from gpu_rsfk import distributed as rdist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")   # NCCL prints to stderr; stdout stays the one JSON line
        dist.init_process_group("nccl", device_id=dev)

    N, D, K = args.points or w["N"], w["D"], w["K"]
    X = make_points(w, args.points)
    # pinned copy only where the end-to-end leg needs it (N > 1: every step uploads the points)
    X_host = torch.from_numpy(X).pin_memory() if (world > 1 and not args.no_e2e) else torch.from_numpy(X)
    X_dev = X_host.to(dev, non_blocking=True)
    torch.cuda.synchronize()

    engine = TimedEngine(DeviceForest(dev))

    def step():
        return rdist.build_knn_graph(engine, X_dev, K, w["trees"], w["min"], w["max"], 5000, w["seed"],
                                     w["sweeps"], True)

    def fence():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    fence()
    launches0 = engine._e.kernel_launches()
    sampler = ClockSampler(local)
    with sampler:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fence()
        e0.record()
        for _ in range(args.steps):
            own_idx, own_dst, rb, re_ = step()
        e1.record()
        fence()
    launches = engine._e.kernel_launches() - launches0
    ms = e0.elapsed_time(e1)
    # Per-kernel times come from one more build with a single tree sequence: in the timed
    # region the forest runs as several sequences on streams of their own, whose kernels
    # overlap, so CUDA events there cannot say how long one kernel took.
    engine._e.set_lanes(1)
    step()                      # untimed: the single sequence's own scratch memory is allocated here
    fence()
    engine.enabled = True
    step()
    fence()
    engine.enabled = False
    engine._e.set_lanes(0)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = N / (ms_per_step * 1e-3)

    # ---- phases and roofline (rank 0's kernels) ---------------------------
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
    tot = {}
    for s in engine.stats:
        for n, v in s.items():
            tot[n] = tot.get(n, 0) + v
    n_forest = max(1, len(engine.records["forest"]))
    n_explore = max(1, len(engine.records["explore"]))
    trees_run = max(1, tot.get("trees", 0))
    rows_own = re_ - rb
    phases = {}
    knn_ms = tot.get("bucket_knn_us", 0) / 1e3
    sub_ms = tot.get("subtree_us", 0) / 1e3
    forest_ms = engine.total_ms("forest")
    sub_pts, sub_nodes = tot.get("sub_active_points", 0), tot.get("sub_nodes", 0)
    lvl_pts = tot.get("tree_active_points", 0) - sub_pts
    lvl_nodes = tot.get("tree_nodes", 0) - sub_nodes
    phases["bucket_knn"] = dict(
        launches=trees_run, ms_per_launch=knn_ms / trees_run,
        bytes_per_launch=4.0 * N * D + 4.0 * N + 2 * 8.0 * N * K)
    tc_launches = tot.get("tc_launches", 0)
    if tc_launches > 0 and knn_ms > 0:
        # tensor-core bucket kernel: useful flops = 2*D*sum(leaf size^2), the contraction counted once,
        # against half of the measured dense bf16 rate (the TF32 ceiling)
        flops = tot.get("tc_gram_flops", 0.0) / tc_launches
        phases["bucket_knn"].update(
            tensor_flops_per_launch=flops, tensor_tflops=flops / (knn_ms / trees_run * 1e-3) / 1e12,
            filter_pass_share=tot.get("tc_pairs_passed", 0) / max(1.0, tot.get("tc_pairs_seen", 0)))
    # tree levels: the projection kernel (one launch per level) and the rest of the level work
    # (decide + scatter kernels, counter read-back by the host)
    proj_ms = tot.get("project_us", 0) / 1e3
    proj_n = max(1, tot.get("project_launches", 0))
    phases["tree_project"] = dict(
        launches=proj_n, ms_per_launch=proj_ms / proj_n,
        bytes_per_launch=(4.0 * (D + 1) * lvl_pts + 4.0 * (D + 1) * lvl_nodes) / proj_n)
    phases["tree_level_rest"] = dict(
        launches=proj_n, ms_per_launch=(forest_ms - knn_ms - sub_ms - proj_ms) / proj_n,
        bytes_per_launch=4.0 * 3 * lvl_pts / proj_n)
    if sub_ms > 0:
        phases["tree_subtrees"] = dict(
            launches=trees_run, ms_per_launch=sub_ms / trees_run,
            bytes_per_launch=(4.0 * (D + 2) * sub_pts + 4.0 * (D + 1) * sub_nodes) / trees_run)
    if engine.records["explore"]:
        C = tot.get("explore_candidates", 0) / n_explore
        phases["explore"] = dict(
            launches=n_explore, ms_per_launch=engine.total_ms("explore") / n_explore,
            bytes_per_launch=4.0 * rows_own * K * (K + 1) + 4.0 * D * (rows_own + C) + 2 * 8.0 * rows_own * K,
            candidates_per_point=C / max(1, rows_own))
    if engine.records["merge"]:
        phases["merge_lists"] = dict(launches=len(engine.records["merge"]),
                                     ms_per_launch=engine.total_ms("merge") / len(engine.records["merge"]),
                                     bytes_per_launch=8.0 * rows_own * K * (world + 1))
    for p in phases.values():
        p["gbs"] = p["bytes_per_launch"] / (p["ms_per_launch"] * 1e-3) / 1e9 if p["ms_per_launch"] > 0 else None
        p["total_ms"] = p["ms_per_launch"] * p["launches"]
    dom = dominant_phase(phases)
    kernel_of = {"bucket_knn": "k_bucket_knn (SIMT)" if tc_launches == 0 else "k_bucket_knn_tc (tcgen05)",
                 "tree_project": "k_project_wide", "tree_level_rest": "k_decide + k_scatter + host read-back",
                 "tree_subtrees": "k_subtree", "merge_lists": "k_merge_lists",
                 # the library stages rows in shared memory for long lists of medium rows (rsfk_knn.cu)
                 "explore": "k_explore_staged" if (32 < K <= 64 and 64 <= D <= 128 and D % 4 == 0) else
                            ("k_explore_wide" if (K <= 32 and 512 <= D <= 1950 and D % 4 == 0) else "k_explore")}
    traffic_unit = NCU_TRAFFIC_PER_POINT.get(dom)
    roofline = dict(bound="hbm", kernel=kernel_of[dom], achieved=phases[dom]["gbs"], peak=peak_gbs,
                    unit="GB/s", frac=(phases[dom]["gbs"] or 0) / peak_gbs, peak_kind=peak_kind,
                    traffic=(traffic_unit * {"explore": rows_own, "tree_project": lvl_pts / proj_n}.get(dom, N))
                    if traffic_unit and args.workload == "c2" else None,
                    traffic_from="ncu capture of a 400 000-point case scaled by the points a launch processes "
                                 "(an under-estimate where the L2 hit rate falls with N)"
                    if traffic_unit and args.workload == "c2" else None,
                    algorithmic_bytes_per_launch=phases[dom]["bytes_per_launch"],
                    ms_per_launch=phases[dom]["ms_per_launch"])
    # the sweeps of the wide-row and long-list configurations: DRAM bytes of an ncu capture of a smaller
    # case (summaries under profiles/) per algorithmic byte, scaled by this launch's algorithmic bytes
    ratio = NCU_TRAFFIC_PER_ALGORITHMIC_BYTE.get((args.workload, dom))
    if ratio is not None and roofline["traffic"] is None:
        roofline["traffic"] = ratio[0] * phases[dom]["bytes_per_launch"]
        roofline["traffic_from"] = ("ncu capture of a %s case (DRAM bytes per algorithmic byte %.3f) scaled by the "
                                    "algorithmic bytes of this launch (an under-estimate where the L2 hit rate "
                                    "falls with N)" % (ratio[1], ratio[0]))
    tensor_roofline = None
    if "tensor_tflops" in phases["bucket_knn"]:
        tf32_peak = 0.5 * float(peaks.get("bf16_tflops", 1590.0))
        b = phases["bucket_knn"]
        tensor_roofline = dict(bound="tensor", kernel="k_bucket_knn_tc (tcgen05 kind::tf32)",
                               achieved=b["tensor_tflops"], peak=tf32_peak, unit="TFLOP/s",
                               frac=b["tensor_tflops"] / tf32_peak,
                               peak_kind=("half of the measured bf16 rate" if "bf16_tflops" in peaks
                                          else "half of the fallback bf16 rate"),
                               flops_per_launch=b["tensor_flops_per_launch"], ms_per_launch=b["ms_per_launch"],
                               hbm_achieved=b["gbs"], hbm_frac=(b["gbs"] or 0) / peak_gbs, traffic=None)
        if dom == "bucket_knn":
            roofline = tensor_roofline

    # ---- recall of the last build -----------------------------------------
    recall = None
    parity = None
    if not args.no_recall or world > 1:
        full_idx, full_dst = rdist.gather_graph(own_idx, own_dst, N)
        if rank == 0 and not args.no_recall:
            nq = min(N, args.recall_queries)
            queries = np.sort(np.random.default_rng(w["seed"] + 1000).choice(N, nq, replace=False))
            truth = exact_knn_torch(X_dev, queries, K).cpu().numpy()
            recall = recall_of(truth, full_idx[torch.as_tensor(queries, device=dev)].cpu().numpy())
        if world > 1:
            # self-check, outside the timed region: the graph the ranks built together against
            # the graph rank 0 builds alone (same seeds): they must be the same bits
            if rank == 0:
                si, sd, _, _ = rdist.build_knn_graph(engine, X_dev, K, w["trees"], w["min"], w["max"], 5000,
                                                     w["seed"], w["sweeps"], True, single=True)
                torch.cuda.synchronize()
                same_i = int((si == full_idx).all(dim=1).sum().item())
                same_d = int((sd.view(torch.int32) == full_dst.view(torch.int32)).all(dim=1).sum().item())
                parity = {"rows": N, "rows_with_identical_indices": same_i, "rows_with_identical_distance_bits": same_d,
                          "against": "the same build on rank 0 alone"}
                del si, sd
            dist.barrier()
        del full_idx, full_dst
    del own_idx, own_dst
    torch.cuda.empty_cache()

    # ---- end to end through host buffers -----------------------------------
    e2e = None
    if args.no_e2e:
        pass
    elif world == 1:
        import gpu_rsfk
        r = RSFK(random_state=w["seed"])
        times = []
        lib_gpus = min(args.library_gpus, torch.cuda.device_count())
        if lib_gpus > 1:   # one process, the library itself spreads the call over the GPUs
            gpu_rsfk.set_devices(list(range(lib_gpus)))
        for i in range(args.e2e_steps + 2):
            res = r.find_nearest_neighbors(X, K, n_trees=w["trees"], min_tree_children=w["min"],
                                           max_tree_children=w["max"], nn_exploring_factor=w["sweeps"])
            if i > 1:          # two untimed calls: context creation, scratch growth
                times.append(r._last_search_time)
        t_e2e = float(np.mean(times))
        e2e = dict(value=N / t_e2e, unit="points/s", h2d_bytes_per_step=4 * N * D + 8 * N * K,
                   d2h_bytes_per_step=8 * N * K, ms_per_step=t_e2e * 1e3,
                   ms_each=[round(t * 1e3, 2) for t in times],
                   api="gpu_rsfk.RSFK.find_nearest_neighbors -> pymodule_rsfk_knn (host buffers)")
        if lib_gpus > 1:
            gpu_rsfk.set_devices(None)
            one = r.find_nearest_neighbors(X, K, n_trees=w["trees"], min_tree_children=w["min"],
                                           max_tree_children=w["max"], nn_exploring_factor=w["sweeps"])
            e2e["library_gpus"] = lib_gpus
            e2e["rows_identical_to_one_gpu"] = int(((one[0] == res[0]).all(axis=1) &
                                                    (one[1].view(np.int32) == res[1].view(np.int32)).all(axis=1)).sum())
            del one
        del res
    else:
        out_i = torch.empty((rdist.row_block(N, world), K), dtype=torch.int32).pin_memory()
        out_d = torch.empty((rdist.row_block(N, world), K), dtype=torch.float32).pin_memory()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        xb, xe = rdist.owned_rows(N, rank, world)
        for i in range(args.e2e_steps + 1):
            if i == 1:
                fence()
                e0.record()
            # every rank uploads its own block of rows; an all-gather over NVLink completes the replica
            xd = rdist.replicate_points(X_host[xb:xe].to(dev, non_blocking=True), N)
            oi, od, rb, re_ = rdist.build_knn_graph(engine, xd, K, w["trees"], w["min"], w["max"], 5000,
                                                    w["seed"], w["sweeps"], True)
            out_i[:re_ - rb].copy_(oi, non_blocking=True)
            out_d[:re_ - rb].copy_(od, non_blocking=True)
            del xd, oi, od
        e1.record()
        fence()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_e2e = float(t.item()) * 1e-3 / args.e2e_steps
        e2e = dict(value=N / t_e2e, unit="points/s", h2d_bytes_per_step=4 * N * D,
                   d2h_bytes_per_step=8 * N * K, ms_per_step=t_e2e * 1e3,
                   api="gpu_rsfk.distributed.replicate_points + build_knn_graph: every rank uploads its block of "
                       "rows from pinned host memory, an NVLink all-gather completes the replica, every rank "
                       "reads back its own rows")

    # ---- CPU baseline: exact brute force on a bounded sample ---------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_bruteforce(X, K, w["seed"], args.cpu_seconds)

    if rank == 0:
        line = {
            "metric": "K-NNG build points/s at fixed recall@K", "value": value, "unit": "points/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "%s: N=%d D=%d K=%d n_trees=%d min/max_tree_children=%d/%d sweeps=%d %s seed %d"
                                   % (args.workload, N, D, K, w["trees"], w["min"], w["max"], w["sweeps"],
                                      w["gen"], w["seed"]),
                       "parallelism": "trees sharded %d-way, all-to-all merge, all-gather per sweep" % world
                       if world > 1 else "single GPU",
                       "l2": "inputs (%.0f MB points + %.0f MB lists) exceed the 126 MB L2; no flush"
                             % (4e-6 * N * D, 8e-6 * N * K)},
            "recall_at_k": recall, "multi_gpu_parity": parity,
            "e2e": e2e, "gpu_launches": int(launches), "clocks": sampler.summary(),
            "roofline": roofline, "bucket_knn_tensor_roofline": tensor_roofline,
            "phases": {n: {k: (round(v, 4) if isinstance(v, float) else v) for k, v in p.items()}
                       for n, p in phases.items()},
            "phases_from": "one further build with a single tree sequence (RSFK lanes = 1), kernels back to "
                           "back on one stream; the timed region overlaps the kernels of several sequences",
            "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def cpu_bruteforce(X, K, seed, seconds):
    """Exact KNN of a bounded sample of rows against all N points with the
    oracle's OpenMP routine; rows/s is directly comparable to points/s."""
    from oracle import rsfk_oracle as orc
    N = X.shape[0]
    rng = np.random.default_rng(seed + 2000)
    probe = np.sort(rng.choice(N, min(N, 64), replace=False)).astype(np.int32)
    t0 = time.time()
    _, _, threads = orc.bruteforce_knn(X, K, probe)
    per_row = (time.time() - t0) / len(probe)
    nq = int(max(64, min(N, seconds / max(per_row, 1e-9))))
    q = np.sort(rng.choice(N, nq, replace=False)).astype(np.int32)
    t0 = time.time()
    orc.bruteforce_knn(X, K, q)
    dt = time.time() - t0
    return {"value": nq / dt, "unit": "points/s", "cores": threads, "kind": "port",
            "sample": "exact brute-force KNN (OpenMP, fmaf) of %d seeded query rows against all %d points, %.1f s"
                      % (nq, N, dt)}


# --------------------------------------------------------------------------- query (ANN) workload
ANN_METRIC = "query search queries/s at fixed recall@K"


def ann_points(args, w):
    """(base points, query points).  The query set is the base set itself (as the
    reference's experiment has it) or, with --distinct-queries, as many further draws
    of the same mixture."""
    N = args.points or w["N"]
    if not args.distinct_queries:
        X = make_points(w, N)
        return X, X
    both = make_points(w, 2 * N)
    return np.ascontiguousarray(both[:N]), np.ascontiguousarray(both[N:])


def ann_config(args, w, N, NQ):
    return {"workload": "%s: base N=%d, queries NQ=%d (%s), D=%d K=%d n_trees=%d min/max_tree_children=%d/%d %s seed %d"
                        % (args.workload, N, NQ, "fresh draws" if args.distinct_queries else "the base set itself",
                           w["D"], w["K"], w["trees"], w["min"], w["max"], w["gen"], w["seed"]),
            "parallelism": "single GPU",
            "l2": "inputs (%.0f MB points + %.0f MB queries + %.0f MB lists) exceed the 126 MB L2; no flush"
                  % (4e-6 * N * w["D"], 4e-6 * NQ * w["D"], 8e-6 * NQ * w["K"])}


def run_ann(args, w):
    import torch
    from gpu_rsfk import RSFK
    from gpu_rsfk.device import DeviceForest
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise RuntimeError("the query workload is a single-GPU bench line")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: there is no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    D, K, T = w["D"], w["K"], w["trees"]
    X, Q = ann_points(args, w)
    N, NQ = X.shape[0], Q.shape[0]
    X_dev = torch.from_numpy(X).to(dev)
    Q_dev = X_dev if Q is X else torch.from_numpy(Q).to(dev)
    f = DeviceForest(dev)

    def step():
        idx, dist = f.init_lists(NQ, K, dev, self_in_row=False)
        f.forest_ann(X_dev, Q_dev, idx, dist, T, w["min"], w["max"], seed=w["seed"])
        return idx, dist

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    launches0 = f.kernel_launches()
    sampler = ClockSampler(0)
    with sampler:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            idx, dist = step()
        e1.record()
        torch.cuda.synchronize()
    launches = f.kernel_launches() - launches0
    ms_per_step = e0.elapsed_time(e1) / args.steps
    # per-kernel device times from one more search with a single tree sequence (see run_ours)
    f.set_lanes(1)
    before = f.stats()
    idx, dist = step()
    torch.cuda.synchronize()
    after = f.stats()
    f.set_lanes(0)
    tot = {n: after[n] - before[n] for n in after}
    value = NQ / (ms_per_step * 1e-3)

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak_gbs = float(peaks.get("hbm_gbs", 6650.0))
    trees_run = max(1, tot["trees"])
    sub_pts, sub_nodes = tot["sub_active_points"], tot["sub_nodes"]
    lvl_pts, lvl_nodes = tot["tree_active_points"] - sub_pts, tot["tree_nodes"] - sub_nodes
    proj_n = max(1, tot["project_launches"])
    phases = {
        "tree_build_host_observed": dict(launches=trees_run, ms_per_launch=tot["tree_build_us"] / 1e3 / trees_run,
                                         bytes_per_launch=(4.0 * (D + 2) * tot["tree_active_points"]
                                                           + 4.0 * (D + 1) * tot["tree_nodes"]) / trees_run),
        "tree_project": dict(launches=proj_n, ms_per_launch=tot["project_us"] / 1e3 / proj_n,
                             bytes_per_launch=(4.0 * (D + 1) * lvl_pts + 4.0 * (D + 1) * lvl_nodes) / proj_n),
        "tree_subtrees": dict(launches=trees_run, ms_per_launch=tot["subtree_us"] / 1e3 / trees_run,
                              bytes_per_launch=(4.0 * (D + 2) * sub_pts + 4.0 * (D + 1) * sub_nodes) / trees_run),
        # hyperplanes + descent + grouping: every query row once, every hyperplane once, leaf ids out
        "query_route": dict(launches=trees_run, ms_per_launch=tot["route_us"] / 1e3 / trees_run,
                            bytes_per_launch=4.0 * NQ * D + 4.0 * (D + 1) * tot["tree_nodes"] / trees_run + 12.0 * NQ),
        # bucket update: every query row and every base row once, lists read and written
        "query_update": dict(launches=trees_run, ms_per_launch=tot["query_update_us"] / 1e3 / trees_run,
                             bytes_per_launch=4.0 * NQ * D + 4.0 * N * D + 4.0 * N + 2 * 8.0 * NQ * K),
    }
    for p in phases.values():
        p["gbs"] = p["bytes_per_launch"] / (p["ms_per_launch"] * 1e-3) / 1e9 if p["ms_per_launch"] > 0 else None
        p["total_ms"] = p["ms_per_launch"] * p["launches"]
    dom = max((n for n in phases if n != "tree_build_host_observed"), key=lambda n: phases[n]["total_ms"])
    kernel_of = {"tree_project": "k_project_wide", "tree_subtrees": "k_subtree",
                 "query_route": "k_planes + k_route + k_leaf_offsets + k_place_queries",
                 "query_update": "k_ann_leaf (k_ann_bucket where the largest leaf does not fit shared memory)"}
    roofline = dict(bound="hbm", kernel=kernel_of[dom], achieved=phases[dom]["gbs"], peak=peak_gbs, unit="GB/s",
                    frac=(phases[dom]["gbs"] or 0) / peak_gbs,
                    peak_kind="measured" if "hbm_gbs" in peaks else "fallback", traffic=None,
                    algorithmic_bytes_per_launch=phases[dom]["bytes_per_launch"],
                    ms_per_launch=phases[dom]["ms_per_launch"])

    recall = None
    if not args.no_recall:
        nq = min(NQ, args.recall_queries)
        rows = np.sort(np.random.default_rng(w["seed"] + 1000).choice(NQ, nq, replace=False))
        rows_t = torch.as_tensor(rows, device=dev)
        truth = []
        chunk = max(1, int(2.5e8 // N))
        x2 = (X_dev * X_dev).sum(1)
        for s in range(0, nq, chunk):
            qv = Q_dev[rows_t[s:s + chunk]]
            d2 = x2[None, :] - 2.0 * (qv @ X_dev.T)
            truth.append(d2.topk(K, dim=1, largest=False).indices)
        truth = torch.cat(truth).cpu().numpy()
        recall = recall_of(truth, idx[rows_t].cpu().numpy())
    del idx, dist
    torch.cuda.empty_cache()

    e2e = None
    if not args.no_e2e:
        r = RSFK(random_state=w["seed"])
        times = []
        for i in range(args.e2e_steps + 2):
            r.find_nearest_neighbors_ann(X, Q, K, n_trees=T, min_tree_children=w["min"],
                                         max_tree_children=w["max"], ensure_valid_indices=False)
            if i > 1:
                times.append(r._last_search_time)
        t = float(np.mean(times))
        e2e = dict(value=NQ / t, unit="queries/s", h2d_bytes_per_step=4 * (N + NQ) * D + 8 * NQ * K,
                   d2h_bytes_per_step=8 * NQ * K, ms_per_step=t * 1e3, ms_each=[round(v * 1e3, 2) for v in times],
                   api="gpu_rsfk.RSFK.find_nearest_neighbors_ann -> pymodule_rsfk_knn_ann (host buffers)")

    cpu = None
    if not args.no_cpu:
        from oracle import rsfk_oracle as orc
        probe = Q[:32]
        t0 = time.time()
        orc.bruteforce_ann(X, probe, K)
        per_row = (time.time() - t0) / len(probe)
        nq = int(max(32, min(NQ, args.cpu_seconds / max(per_row, 1e-9))))
        t0 = time.time()
        orc.bruteforce_ann(X, Q[:nq], K)
        dt = time.time() - t0
        cpu = {"value": nq / dt, "unit": "queries/s", "cores": os.cpu_count(), "kind": "port",
               "sample": "exact brute-force search (OpenMP, fmaf) of the first %d query rows against all %d base "
                         "points, %.1f s" % (nq, N, dt)}

    print(json.dumps({
        "metric": ANN_METRIC, "value": value, "unit": "queries/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": ann_config(args, w, N, NQ),
        "recall_at_k": recall, "e2e": e2e, "gpu_launches": int(launches), "clocks": sampler.summary(),
        "roofline": roofline,
        "phases": {n: {k: (round(v, 4) if isinstance(v, float) else v) for k, v in p.items()}
                   for n, p in phases.items()},
        "cpu_baseline": cpu}))


def ann_reference_worker(args, w):
    """Child process: the reference's pymodule_rsfk_knn_ann (src/python/pymodule_ext.cu:149-181) with the
    query set equal to the base set -- the shape of its own experiment and the only one its driver
    handles within bounds (src/rsfk.cu:396-403)."""
    L = ctypes.CDLL(REF_SO)
    L.pymodule_rsfk_knn_ann.restype = None
    L.pymodule_rsfk_knn_ann.argtypes = [ctypes.c_int] * 11 + [ctypes.c_void_p] * 5
    X = make_points(w, args.points)
    N, D, K, T = X.shape[0], w["D"], w["K"], w["trees"]
    Q = X.copy()
    times = []
    for s in range(args.warmup + args.steps):
        idx = np.full((N, K), -1, np.int32)
        dst = np.full((N, K), np.inf, np.float32)
        log = np.zeros(16 * T + 2, np.float32)
        t0 = time.time()
        L.pymodule_rsfk_knn_ann(T, K, N, N, D, w["min"], w["max"], 5000, 0, w["seed"], 0, X.ctypes.data,
                                Q.ctypes.data, idx.ctypes.data, dst.ctypes.data, log.ctypes.data)
        if s >= args.warmup:
            times.append(time.time() - t0)
    recall = None
    if not args.no_recall:
        import torch
        dev = torch.device("cuda", 0)
        Xd = torch.from_numpy(X).to(dev)
        nq = min(N, args.recall_queries)
        rows = np.sort(np.random.default_rng(w["seed"] + 1000).choice(N, nq, replace=False))
        truth = exact_knn_torch(Xd, rows, K).cpu().numpy()
        recall = recall_of(truth, idx[rows])
    print("REFRESULT " + json.dumps({"times": times, "recall": recall, "trees": T, "forest_s": 0.0,
                                     "explore_s": 0.0}))


def run_ann_reference(args, w):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    base = {"impl": "reference"}
    if args.distinct_queries:
        print(json.dumps(dict(base, unavailable="the reference's query driver reads and scatters out of bounds "
                                                "unless the query set is the base set (src/rsfk.cu:396-403); "
                                                "not run")))
        return
    if not os.path.exists(REF_SO):
        print(json.dumps(dict(base, unavailable="oracle/_ref/librsfk_ref.so was not built (make -C oracle ref)")))
        return
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-worker", "--workload", args.workload,
           "--steps", str(args.steps), "--warmup", str(args.warmup), "--recall-queries", str(args.recall_queries)]
    if args.points:
        cmd += ["--points", str(args.points)]
    if args.no_recall:
        cmd += ["--no-recall"]
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    try:
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.ref_timeout)
    except subprocess.TimeoutExpired:
        print(json.dumps(dict(base, unavailable="reference library did not finish within %d s" % args.ref_timeout)))
        return
    res = [l for l in out.stdout.splitlines() if l.startswith("REFRESULT ")]
    if out.returncode != 0 or not res:
        tail = (out.stderr or out.stdout).strip().splitlines()[-1:] or ["no output"]
        print(json.dumps(dict(base, unavailable="reference library failed (exit %d): %s" % (out.returncode, tail[0][:200]))))
        return
    r = json.loads(res[0][len("REFRESULT "):])
    t = float(np.mean(r["times"]))
    N = args.points or w["N"]
    value = N / t
    print(json.dumps({
        "impl": "reference", "metric": ANN_METRIC, "value": value, "unit": "queries/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": ann_config(args, w, N, N), "recall_at_k": r["recall"],
        "cpu_baseline": {"value": value, "unit": "queries/s", "cores": 0, "kind": "reference",
                         "sample": "the reference's own CUDA library (it has no CPU path), unmodified sources "
                                   "compiled for sm_100, one GPU, host buffers, whole workload"},
        "e2e": {"value": value, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# --------------------------------------------------------------------------- reference arm
REF_SO = os.path.join(ROOT, "oracle", "_ref", "librsfk_ref.so")
# the reference built with its tile variant of the bucket kernel (oracle/Makefile: ref_tiles)
REF_TILES_SO = os.path.join(ROOT, "oracle", "_ref", "librsfk_ref_tiles.so")


def reference_worker(args, w):
    """Child process: the reference's own library through its C ABI
    (reference: src/python/pymodule_ext.cu:124-147), host buffers, as its wrapper calls it."""
    L = ctypes.CDLL(REF_TILES_SO if args.ref_variant == "tiles" else REF_SO)
    i = ctypes.c_int
    L.pymodule_rsfk_knn.restype = None
    L.pymodule_rsfk_knn.argtypes = [i] * 10 + [ctypes.c_void_p] * 4
    N, D, K = args.points or w["N"], w["D"], w["K"]
    X = make_points(w, args.points)
    trees = args.ref_trees or w["trees"]
    times, recalls = [], []
    truth = queries = None
    if not args.no_recall:
        import torch
        nq = min(N, args.recall_queries)
        queries = np.sort(np.random.default_rng(w["seed"] + 1000).choice(N, nq, replace=False))
        X_dev = torch.from_numpy(X).cuda()
        truth = exact_knn_torch(X_dev, queries, K).cpu().numpy()
        del X_dev
        torch.cuda.empty_cache()
    for s in range(args.warmup + args.steps):
        idx = np.full((N, K), -1, np.int32)
        dst = np.full((N, K), np.inf, np.float32)
        idx[:, 0] = np.arange(N)
        dst[:, 0] = 0
        log = np.zeros(16 * trees + 2, np.float32)
        t0 = time.time()
        L.pymodule_rsfk_knn(trees, K, N, D, w["min"], min(w["max"], 1024), 5000, 0, w["seed"], w["sweeps"],
                            X.ctypes.data, idx.ctypes.data, dst.ctypes.data, log.ctypes.data)
        if s >= args.warmup:
            times.append(time.time() - t0)
            if truth is not None:       # the reference is not deterministic: every run's recall
                recalls.append(recall_of(truth, idx[queries]))
    recall = recalls[-1] if recalls else None
    print("REFRESULT " + json.dumps({"times": times, "recall": recall, "recalls": recalls, "trees": trees,
                                     "forest_s": float(log[16 * trees]), "explore_s": float(log[16 * trees + 1])}))


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    N, D, K = args.points or w["N"], w["D"], w["K"]
    base = {"impl": "reference"}
    if not os.path.exists(REF_TILES_SO if args.ref_variant == "tiles" else REF_SO):
        print(json.dumps(dict(base, unavailable="oracle/_ref/librsfk_ref*.so was not built (make -C oracle ref ref_tiles)")))
        return
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference-worker", "--workload", args.workload,
           "--steps", str(args.steps), "--warmup", str(args.warmup), "--recall-queries", str(args.recall_queries)]
    if args.points:
        cmd += ["--points", str(args.points)]
    if args.ref_trees:
        cmd += ["--ref-trees", str(args.ref_trees)]
    if args.no_recall:
        cmd += ["--no-recall"]
    if args.max_children:
        cmd += ["--max-children", str(args.max_children)]
    cmd += ["--ref-variant", args.ref_variant]
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT"):
        env.pop(k, None)
    env["CUDA_VISIBLE_DEVICES"] = os.environ.get("LOCAL_RANK", "0") if "CUDA_VISIBLE_DEVICES" not in os.environ else os.environ["CUDA_VISIBLE_DEVICES"].split(",")[0]
    try:
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=args.ref_timeout)
    except subprocess.TimeoutExpired:
        print(json.dumps(dict(base, unavailable="reference library did not finish within %d s" % args.ref_timeout)))
        return
    res = [l for l in out.stdout.splitlines() if l.startswith("REFRESULT ")]
    if out.returncode != 0 or not res:
        tail = (out.stderr or out.stdout).strip().splitlines()[-1:] or ["no output"]
        print(json.dumps(dict(base, unavailable="reference library failed (exit %d): %s" % (out.returncode, tail[0][:200]))))
        return
    r = json.loads(res[0][len("REFRESULT "):])
    t = float(np.mean(r["times"]))
    scale = w["trees"] / float(r["trees"])
    note = ""
    if r["trees"] != w["trees"]:
        # bounded sample: fewer trees; the forest part scales with the tree count
        t = r["forest_s"] * scale + (t - r["forest_s"])
        note = " (forest time of %d trees scaled to %d)" % (r["trees"], w["trees"])
    value = N / t
    line = {
        "impl": "reference", "metric": "K-NNG build points/s at fixed recall@K", "value": value,
        "unit": "points/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "%s: N=%d D=%d K=%d n_trees=%d min/max_tree_children=%d/%d sweeps=%d %s seed %d"
                               % (args.workload, N, D, K, w["trees"], w["min"], min(w["max"], 1024), w["sweeps"],
                                  w["gen"], w["seed"])},
        "recall_at_k": r["recall"],
        "cpu_baseline": {"value": value, "unit": "points/s", "cores": 0, "kind": "reference",
                         "sample": "the reference's own CUDA library (it has no CPU path), unmodified sources "
                                   "compiled for sm_100, one GPU, host buffers, whole workload" + note
                                   + (" (bucket kernel: its tile variant, one launch line edited)"
                                      if args.ref_variant == "tiles" else "")},
        "e2e": {"value": value, "unit": "points/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "reference_forest_s": r["forest_s"], "reference_explore_s": r["explore_s"],
        "recall_each_run": r.get("recalls"), "s_each_run": r["times"],
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-worker"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--points", type=int, default=0, help="override N (debugging)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--recall-queries", type=int, default=10_000)
    ap.add_argument("--no-recall", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--ref-trees", type=int, default=0, help="reference arm: time this many trees and scale")
    ap.add_argument("--ref-timeout", type=int, default=900)
    ap.add_argument("--ref-variant", default="default", choices=["default", "tiles"],
                    help="reference arm: its default bucket kernel or its tile variant")
    ap.add_argument("--distinct-queries", action="store_true",
                    help="query workload: fresh draws instead of the base set itself")
    ap.add_argument("--library-gpus", type=int, default=1,
                    help="host-buffer leg of a single-process run: GPUs the library spreads one call over")
    ap.add_argument("--max-children", type=int, default=0,
                    help="override max_tree_children of the workload (both arms), e.g. 1024 to meet the reference's limit")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.max_children:
        w["max"] = args.max_children
    if args.workload == "ann":
        {"reference": run_ann_reference, "reference-worker": ann_reference_worker}.get(args.impl, run_ann)(args, w)
    elif args.impl == "reference":
        run_reference(args, w)
    elif args.impl == "reference-worker":
        reference_worker(args, w)
    else:
        run_ours(args, w)


if __name__ == "__main__":
    main()

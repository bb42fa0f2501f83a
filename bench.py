"""Benchmark of the per-batch temporal-embedding path: scored temporal edges per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5] [--impl ours|reference]

A step is one batch of the workload's stream (bs positive edges + bs negatives scored) run through
TGN.compute_edge_probabilities in eval mode with budgeted reuse and the batch's cache plan.
The timed batches are consecutive batches from the middle of the stream (neighbour lists are full
there); the state tables start cold, which changes values, not the amount of work.

Prints ONE JSON line (rank 0).  `value` = edges/s with the inputs of all timed batches already in
HBM; `e2e` = the same through the public Python API with host (NumPy) inputs, one pinned H2D copy
and the D2H read of the scores per step; `roofline` = the fused gather-attention kernel, timed with
CUDA events around each of its launches; `cpu_baseline` = the CPU oracle on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "temporal edges scored/sec (2-layer, K=10)"
ROW_BYTES = 688


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c5")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-batches", type=int, default=None, help="batches of the CPU baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="direct", choices=["direct", "nccl"],
                    help="N > 1: how the layer-1 rows travel between the GPUs (peer stores or an NCCL all-gather)")
    ap.add_argument("--split", default="layers", choices=["layers", "rows"],
                    help="N > 1: layers = the first N // 2 GPUs compute layer 1 and the memory update, the others "
                         "the top layer and the scores (default); rows = every GPU its share of both layers' rows")
    ap.add_argument("--layer1-ranks", type=int, default=None,
                    help="--split layers: how many GPUs compute layer 1 and the memory update (default N // 2)")
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: strong = the workload's batch split over the GPUs (default); weak = a batch of "
                         "bs edges PER GPU, i.e. the same stream cut into batches of bs * N edges")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="the timed window of --steps steps is repeated until this much time has been timed; the "
                         "median window is reported (0: one window, e.g. under a profiler)")
    ap.add_argument("--plan-batches", type=int, default=None,
                    help="plan only this many leading batches of the stream (quick runs)")
    return ap.parse_args()


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML every few milliseconds; result()
    keeps the samples that fall inside the timed windows (host time stamps taken right after the
    synchronisation before a window and right after the one behind it)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.max_mhz, self.windows = index, [], False, None, []
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                t = time.perf_counter()
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.samples.append((t, mhz, r))
            except Exception:
                break
            time.sleep(0.002)

    def window(self, t0, t1):
        self.windows.append((t0, t1))

    def result(self):
        self.stop_flag = True
        nv = self.nv
        if nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["unavailable"], "samples": 0}
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        inside = [(m, r) for t, m, r in self.samples if any(a <= t <= b for a, b in self.windows)]
        where = "inside the timed windows"
        if not inside:      # windows shorter than the sampling period: the whole measurement phase then
            inside = [(m, r) for _, m, r in self.samples]
            where = "over the measurement phase (no sample fell inside a timed window)"
        reasons = sorted(k for k, bit in names.items() if any(r & bit for _, r in inside))
        return {"sm_mhz": float(np.median([m for m, _ in inside])), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside), "sampled": where}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def workload_config(g, spec, start, extra=None):
    cfg = {"workload": f"{spec.name}: {g.n_nodes - 1} nodes, {g.n_edges} edges, bs={spec.bs}, "
                       f"L={spec.n_layers}, K={spec.n_degree}, budget={spec.budget} {spec.strategy}",
           "first_timed_batch": int(start),
           "l2": "inputs larger than L2: edge-feature and state tables total "
                 f"{(g.n_edges + 1 + 7 * g.n_nodes) * ROW_BYTES / 1e9:.1f} GB and every step gathers different rows"}
    if extra:
        cfg.update(extra)
    return cfg


def build_setup(a, device, quiet=True):
    """Graph, negatives, neighbour finder, plan and model for the workload (every rank)."""
    import contextlib

    import torch

    from orca_b200 import params, synthetic
    from orca_b200.cache import get_cache_plan
    from orca_b200.neighbor_finder import get_neighbor_finder
    from orca_b200.tgn import TGN
    t0 = time.time()
    g = synthetic.make_graph(a.workload)
    if a.scaling == "weak" and a.gpus > 1:
        # same graph and stream, batches of bs edges per GPU (the batch size only cuts the stream)
        import dataclasses
        g.spec = dataclasses.replace(g.spec, bs=g.spec.bs * a.gpus)
    spec = g.spec
    neg = synthetic.negative_destinations(g, seed=0)
    nf = get_neighbor_finder(g, device=device)
    ns = argparse.Namespace(bs=spec.bs, n_degree=spec.n_degree, budget=spec.budget, reuse=True, gradient=False,
                            n_nodes=g.n_nodes, n_edges=g.n_edges + 1)
    t1 = time.time()
    with contextlib.redirect_stdout(sys.stderr):
        if a.plan_batches:
            import dataclasses
            import types
            m = min(g.n_edges, a.plan_batches * spec.bs)
            sub = types.SimpleNamespace(sources=g.sources[:m], destinations=g.destinations[:m],
                                        timestamps=g.timestamps[:m])
            plan = get_cache_plan(ns, sub, nf, g.n_nodes, spec.strategy, broadcast_from=0)
        else:
            plan = get_cache_plan(ns, g, nf, g.n_nodes, spec.strategy, broadcast_from=0)
    t2 = time.time()
    tgn = TGN(neighbor_finder=nf, node_features=None, edge_features=g.edge_features, device=device,
              n_layers=spec.n_layers, n_heads=2, dropout=0.1, use_memory=True, node_dimension=172,
              time_dimension=172, memory_dimension=172, embedding_module_type="graph_attention",
              message_function="identity", aggregator_type="last", memory_updater_type="gru",
              n_neighbors=spec.n_degree, args=ns)
    sd = {k: torch.from_numpy(v) for k, v in params.random_state_dict(spec.n_layers, seed=0).items()}
    sd["embedding_module.time_encoder.w.weight"] = sd["time_encoder.w.weight"]
    sd["embedding_module.time_encoder.w.bias"] = sd["time_encoder.w.bias"]
    tgn.load_state_dict(sd)
    tgn.eval()
    if not quiet:
        print(f"[bench] graph+finder {t1 - t0:.1f}s, plan {t2 - t1:.1f}s, model {time.time() - t2:.1f}s",
              file=sys.stderr)
    return g, neg, plan, tgn


def pick_window(n_batches, steps, warmup):
    """First batch index of the warm-up so that the timed batches sit mid-stream."""
    total = steps + warmup
    if total > n_batches:
        raise SystemExit(f"--steps + --warmup = {total} exceeds the {n_batches} batches of the stream")
    first = max(0, min(n_batches // 2 - warmup, n_batches - total))
    return first


def batch_arrays(g, neg, b):
    bs = g.spec.bs
    s, e = b * bs, min(g.n_edges, (b + 1) * bs)
    return g.sources[s:e], g.destinations[s:e], neg[s:e], g.timestamps[s:e], g.edge_idxs[s:e]


def reset_state(tgn, plan, first):
    tgn.memory.__init_memory__()
    if tgn.n_layers > 1:
        tgn.embedding_module.reset_history()
        h = tgn.embedding_module.histories[0]
        h.cache_flag_dev.zero_()
        h.n_prev[0] = -1
        if first > 0:
            h.update_flag(plan[first - 1], None)
    tgn.test_mode = True


def algorithmic_bytes(b, k, n1, n2, p):
    """Bytes one batch must move, every gathered row counted once, weights excluded:
    sampling Q*(28K+80), attention rows (N1+N2)*(R*(2K+2)+12K), scoring 3B*R+8B, message + GRU per
    unique positive P*(13R+8)."""
    q = n1 + n2
    R = ROW_BYTES
    return q * (28 * k + 80) + (n1 + n2) * (R * (2 * k + 2) + 12 * k) + 3 * b * R + 8 * b + p * (13 * R + 8)


def run_ours(a):
    import torch
    import torch.distributed as dist

    from orca_b200 import _lib
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    L = _lib.lib()
    g, neg, plan, tgn = build_setup(a, device, quiet=rank != 0)
    if world > 1:
        tgn.set_distributed(rank, world, exchange=a.exchange, split=a.split, layer1_ranks=a.layer1_ranks)
    spec = g.spec
    K, W = a.steps, a.warmup
    nb_avail = len(plan)
    first = pick_window(nb_avail, K, W)
    k = spec.n_degree
    stream = _lib.stream_ptr(device)
    idle = torch.cuda.Stream(device)     # never given work: "inputs ready" for batches preloaded in HBM

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()

    def timed(run_window, min_seconds=a.min_seconds, max_repeats=400):
        """run_window(i0, n, is_timed) runs steps i0 .. i0+n-1.  W untimed + K timed steps from the same reset
        state, repeated until `min_seconds` of timed region have accumulated; returns (median ms of a K-step
        window, repeats, host ms per window)."""
        ms_all, host_all, total = [], [], 0.0
        while (total < min_seconds * 1e3 or not ms_all) and len(ms_all) < max_repeats:
            reset_state(tgn, plan, first)
            run_window(0, W, False)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            e0.record()
            run_window(W, K, True)
            host_all.append((time.perf_counter() - t0) * 1e3)   # time the CPU needed to enqueue the steps
            e1.record()
            barrier()
            sampler.window(t0, time.perf_counter())
            ms = torch.tensor([e0.elapsed_time(e1)], device=device)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)     # every rank sees the same number: same repeat count
            ms_all.append(float(ms.item()))
            total += ms_all[-1]
        return float(np.median(ms_all)), len(ms_all), float(np.median(host_all))

    # ---------------- end to end: the public API with host (NumPy) inputs.  TGN.eval_epoch scores a run of
    # batches in one call; per batch the library copies the batch from pinned host memory to the device, runs
    # it and copies its scores back to the host.  (Multi-GPU: every rank reads back the scores of its edges
    # per batch; the ranks' parts are exchanged once per call.)
    bs = spec.bs
    counted = {}
    per_batch_api = world > 1 and tgn._exchange is None

    def api_window(i0, n, is_timed):
        lo, hi = (first + i0) * bs, min(g.n_edges, (first + i0 + n) * bs)
        pl = plan[first + i0: first + i0 + n]
        if per_batch_api:
            # (the NCCL exchange sits between two library calls per batch: no whole-epoch call there)
            out = []
            for j in range(n):
                a = batch_arrays(g, neg, first + i0 + j)
                p, q = tgn.compute_edge_probabilities(*a, k, True, False, pl[j])
                out.append((p, q))
            pos = np.concatenate([p.cpu().numpy().ravel() for p, _ in out])
            ngs = np.concatenate([q.cpu().numpy().ravel() for _, q in out])
        else:
            pos, ngs = tgn.eval_epoch(g.sources[lo:hi], g.destinations[lo:hi], neg[lo:hi], g.timestamps[lo:hi],
                                      g.edge_idxs[lo:hi], k, bs, pl)
        if is_timed:
            counted["h2d"] = 24 * (hi - lo) + 4 * sum(len(x) for x in pl)
            counted["d2h"] = 8 * (hi - lo) // world
            counted["scores"] = (pos, ngs)

    ms_e2e, rep_e2e, host_e2e = timed(api_window)
    tgn.check_status()
    edges = sum(len(batch_arrays(g, neg, first + W + i)[0]) for i in range(K))
    e2e = {"value": edges / (ms_e2e / 1e3), "unit": "edges/s",
           "h2d_bytes_per_step": counted["h2d"] // K, "d2h_bytes_per_step": counted["d2h"] // K,
           "ms_per_step": ms_e2e / K, "repeats": rep_e2e,
           "api": ("TGN.compute_edge_probabilities per batch" if per_batch_api else
                   "TGN.eval_epoch (one call per timed window; per-batch H2D and D2H inside the library)")}

    # ---------------- device-resident inputs: packed batches preloaded, the C ABI called directly
    packed = []
    for i in range(W + K):
        src, dst, ng, ts, eidx = batch_arrays(g, neg, first + i)
        pl = plan[first + i]
        ints = torch.from_numpy(np.concatenate([src, dst, ng, eidx, pl]).astype(np.int32)).to(device)
        packed.append((ints, torch.from_numpy(np.ascontiguousarray(ts)).to(device), len(src), len(pl)))
    probs = torch.empty((W + K, 2 * bs), device=device)
    torch.cuda.synchronize()
    tgn._input_stream = idle.cuda_stream
    ws, u_cap = tgn._workspace(bs, k)

    def abi_step(i):
        ints, ts, n, n_plan = packed[i]
        desc = tgn._descriptor(k)        # cached; only the state-table pointers are refreshed (reset_state)
        if world > 1:
            # sharded attention layers and scores; the scores stay sharded (every rank keeps those of its edges)
            from orca_b200 import shard
            if tgn._exchange is not None:     # rows exchanged by peer stores inside the library: one call
                _lib.check(L.orca_tgn_eval_batch_sharded(desc, 0, ints.data_ptr(), ts.data_ptr(), n,
                                                         ints.data_ptr() + 16 * n, n_plan, u_cap, ws.data_ptr(),
                                                         ws.numel(), None, None, probs[i].data_ptr(), None,
                                                         tgn._status.data_ptr(), stream))
                return
            rpr = shard.rows_per_rank(3 * n + u_cap, world)
            emb1_local = torch.empty(rpr, 172, device=device)
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 1, ints.data_ptr(), ts.data_ptr(), n,
                                                     ints.data_ptr() + 16 * n, n_plan, u_cap, ws.data_ptr(),
                                                     ws.numel(), emb1_local.data_ptr(), None, None, None,
                                                     tgn._status.data_ptr(), stream))
            emb1_all = shard.all_gather_rows(emb1_local)
            _lib.check(L.orca_tgn_eval_batch_sharded(desc, 2, ints.data_ptr(), ts.data_ptr(), n,
                                                     ints.data_ptr() + 16 * n, n_plan, u_cap, ws.data_ptr(),
                                                     ws.numel(), None, emb1_all.data_ptr(), probs[i].data_ptr(),
                                                     None, tgn._status.data_ptr(), stream))
            return
        _lib.check(L.orca_tgn_eval_batch(desc, ints.data_ptr(), ts.data_ptr(), n, ints.data_ptr() + 16 * n, n_plan,
                                         u_cap, ws.data_ptr(), ws.numel(), probs[i].data_ptr(), None,
                                         tgn._status.data_ptr(), stream))

    def abi_window(i0, n, is_timed):
        for i in range(i0, i0 + n):
            abi_step(i)

    ms_dev, rep_dev, host_dev = timed(abi_window)
    counts = tgn.check_status()
    launches_per_batch = counts[2]
    clocks = sampler.result()

    # ---------------- roofline pass: same batches, CUDA events around every gather-attention launch
    reset_state(tgn, plan, first)
    counters = torch.zeros(2, dtype=torch.int64, device=device)
    for i in range(W):
        abi_step(i)
    torch.cuda.synchronize()
    _lib.check(L.orca_attn_gather_profile(tgn._ctx, 1, counters.data_ptr()))
    tgn.set_option(_lib.OPT_TRACE, 1)
    step_bytes = 0
    for i in range(K):
        abi_step(W + i)
        n1, p, _ = tgn.check_status()
        n = packed[W + i][2]
        step_bytes += algorithmic_bytes(n, k, n1 if spec.n_layers == 2 else 3 * n,
                                        3 * n if spec.n_layers == 2 else 0, p)
    gms = np.zeros(1, dtype=np.float64)
    gl = np.zeros(1, dtype=np.int64)
    _lib.check(L.orca_attn_gather_profile_read(tgn._ctx, gms.ctypes.data, gl.ctypes.data))
    _lib.check(L.orca_attn_gather_profile(tgn._ctx, 0, None))
    n_ph = L.orca_trace_phases()
    ph_ms = np.zeros(n_ph, dtype=np.float64)
    _lib.check(L.orca_trace_read(tgn._ctx, ph_ms.ctypes.data))
    tgn.set_option(_lib.OPT_TRACE, 0)
    phases = {L.orca_trace_phase_name(i).decode(): round(float(ph_ms[i]) * 1e3 / K, 2) for i in range(n_ph)}
    rows_g, slots_g = (int(x) for x in counters.cpu().numpy())
    peak, peak_kind = load_peaks()
    gather_bytes = rows_g * (2 * ROW_BYTES + 12 * k) + slots_g * 2 * ROW_BYTES
    achieved = gather_bytes / (gms[0] / 1e3) / 1e9 if gms[0] > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": "attn_gather_kernel", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind + " copy bandwidth",
                "traffic": GATHER_TRAFFIC_RATIO * gather_bytes / max(int(gl[0]), 1), "launches": int(gl[0]),
                "avg_launch_us": gms[0] * 1e3 / max(int(gl[0]), 1),
                "algorithmic_bytes_per_launch": gather_bytes / max(int(gl[0]), 1)}
    step_frac = step_bytes / (ms_dev / 1e3) / 1e9 / peak

    parity = parity_vs_single(a, g, neg, plan, tgn, first, device, rank, world) if world > 1 else None

    value = edges / (ms_dev / 1e3)
    line = {"metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_dev / K, "higher_is_better": True, "scaling": a.scaling if world > 1 else "strong",
            "vs_baseline": None, "repeats": rep_dev,
            "dtype": "f32", "data": "synthetic",
            "config": workload_config(g, spec, first + W, {
                "whole_step_hbm_frac": step_frac / world, "algorithmic_bytes_per_edge": step_bytes / edges,
                "timing": f"median of {rep_dev} windows of {K} steps, each after a state reset and {W} warm-up steps",
                **({"weak_scaling": f"batches of {spec.bs // world} edges per GPU: the stream is cut into batches "
                                    f"of {spec.bs} edges"} if (world > 1 and a.scaling == "weak") else {}),
                "sharding": ("replicated tables; "
                             + (f"layer 1 and the memory update on {tgn._layer1_ranks} GPU(s) (rows by row % "
                                f"{tgn._layer1_ranks}), top layer and scores on the other {world - tgn._layer1_ranks} "
                                f"(edges by edge % {world - tgn._layer1_ranks}); " if tgn._layer1_ranks
                                else "attention rows and scores split by row/edge % n_gpus; ")
                             + "layer-1 rows and updated memory rows "
                             + ("written to every GPU by peer stores over NVLink" if tgn._exchange is not None
                                else "all-gathered with NCCL") + " once per batch") if world > 1 else "single GPU"}),
            "roofline": roofline, "e2e": e2e, "gpu_launches": int(launches_per_batch * K), "clocks": clocks,
            "host_enqueue_ms_per_step": {"e2e": host_e2e / K, "value": host_dev / K},
            "phases_us_per_step": phases}
    if parity is not None:
        line["parity_vs_single"] = parity
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(a, g, neg, plan, first + W)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def parity_vs_single(a, g, neg, plan, tgn, first, device, rank, world, n_batches=6):
    """The sharded model against an unsharded replica on rank 0: the same batches from the same reset
    state; largest score difference and whether the state tables ended bit-identical."""
    import torch
    import torch.distributed as dist

    spec = g.spec
    k = spec.n_degree
    reset_state(tgn, plan, first)
    got = []
    for i in range(n_batches):
        src, dst, ng, ts, eidx = batch_arrays(g, neg, first + i)
        p, q = tgn.compute_edge_probabilities(src, dst, ng, ts, eidx, k, True, False, plan[first + i])
        got.append(torch.cat([p, q]).clone())
    tgn.check_status()
    out = None
    if rank == 0:
        import copy

        from orca_b200.tgn import TGN
        ns = copy.copy(tgn.args)           # a second model on this GPU: same graph and weights, state of its own
        single = TGN(neighbor_finder=tgn.embedding_module.neighbor_finder, node_features=None,
                     edge_features=g.edge_features, device=device, n_layers=spec.n_layers, n_heads=2, dropout=0.1,
                     use_memory=True, node_dimension=172, time_dimension=172, memory_dimension=172,
                     embedding_module_type="graph_attention", message_function="identity", aggregator_type="last",
                     memory_updater_type="gru", n_neighbors=k, args=ns)
        single.load_state_dict(tgn.state_dict())
        single.eval()
        reset_state(single, plan, first)
        worst = 0.0
        for i in range(n_batches):
            src, dst, ng, ts, eidx = batch_arrays(g, neg, first + i)
            p, q = single.compute_edge_probabilities(src, dst, ng, ts, eidx, k, True, False, plan[first + i])
            worst = max(worst, float((torch.cat([p, q]) - got[i]).abs().max()))
        single.check_status()
        out = {"batches": n_batches, "max_abs_score_diff": worst,
               "memory_equal": bool(torch.equal(single.memory.memory, tgn.memory.memory)),
               "history_equal": bool(torch.equal(single.embedding_module.histories[0].emb,
                                                 tgn.embedding_module.histories[0].emb))}
        del single
    dist.barrier()
    return out


# DRAM traffic of attn_gather_kernel: (dram__bytes_read.sum + dram__bytes_write.sum) of two consecutive
# launches captured with ncu on workload c4 (17.01 + 16.65 MB read, 0 written) over the algorithmic bytes of
# those launches (2 x 30.68 MB), applied to the algorithmic bytes of this run's launches; the counter cannot
# be read while timing
GATHER_TRAFFIC_RATIO = (15.276032 + 14.909696) / (2 * 30.683416)


def oracle_sample(g, neg, plan, first, n_batches, sub_bs, threads, min_seconds=0.0):
    """Times the CPU oracle (the restatement of the reference's PyTorch + numba path) on
    `n_batches` consecutive batches starting at `first`, each cut to its first `sub_bs` edges; with
    `min_seconds` it goes on past `n_batches` (while the plan lasts) until that much time is spent.
    Returns (edges, seconds, batches)."""
    import torch

    from oracle import tgn_oracle
    from orca_b200 import params
    torch.set_num_threads(threads)
    spec = g.spec
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    orc = tgn_oracle.OracleTGN(adj, g.edge_features, params.random_state_dict(spec.n_layers, seed=0), g.n_nodes,
                               n_layers=spec.n_layers, budget=spec.budget)
    if spec.n_layers > 1 and first > 0:
        orc.cache_flag[0][np.asarray(plan[first - 1], dtype=np.int64)] = 1
    # one untimed batch warms the thread pools and the page cache of the big tables
    src, dst, ng, ts, eidx = (x[:sub_bs] for x in batch_arrays(g, neg, max(first - 1, 0)))
    orc.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, plan[max(first - 1, 0)])
    edges, i = 0, 0
    t0 = time.perf_counter()
    while first + i < len(plan) and (i < n_batches or time.perf_counter() - t0 < min_seconds):
        src, dst, ng, ts, eidx = (x[:sub_bs] for x in batch_arrays(g, neg, first + i))
        orc.compute_edge_probabilities(src, dst, ng, ts, eidx, spec.n_degree, plan[first + i])
        edges += len(src)
        i += 1
    return edges, time.perf_counter() - t0, i


def cpu_baseline(a, g, neg, plan, first):
    threads = os.cpu_count() or 1
    nb = min(a.cpu_batches or 8, len(plan) - first)
    edges, sec, nb = oracle_sample(g, neg, plan, first, nb, g.spec.bs, threads,
                                   min_seconds=0.0 if a.cpu_batches else 12.0)
    return {"value": edges / sec, "unit": "edges/s", "cores": threads, "kind": "port",
            "sample": f"{nb} consecutive whole batches from batch {first} ({edges} edges), "
                      f"CPU oracle (numpy + fp32 torch), {sec:.1f}s"}


def run_reference(a):
    """The reference arm: the CPU restatement of the reference's own path on the host cores (the
    reference is Python + numba and is not installed on the GPU box; the oracle is its port)."""
    rank = int(os.environ.get("RANK", 0))
    if rank != 0:
        return
    import contextlib

    from orca_b200 import synthetic
    from oracle import planner, tgn_oracle
    g = synthetic.make_graph(a.workload)
    spec = g.spec
    neg = synthetic.negative_destinations(g, seed=0)
    K, W = a.steps, a.warmup
    threads = os.cpu_count() or 1
    # the plan only steers which neighbours count as cached; it is computed by the CPU planner on a
    # prefix of the stream that covers the timed window
    first = pick_window(g.n_batches, K, W)
    # every step is one whole stream batch (about 0.15 s of CPU work at 2000 edges)
    sub_bs = spec.bs
    adj = tgn_oracle.Adjacency(g.sources, g.destinations, g.edge_idxs, g.timestamps, g.n_nodes)
    m = min(g.n_edges, (first + W + K) * spec.bs)
    t0 = time.time()
    plan = planner.get_cache_plan(g.sources[:m], g.destinations[:m], g.timestamps[:m], spec.bs, spec.n_degree,
                                  spec.budget, adj, g.n_nodes, spec.strategy)
    print(f"[bench] reference arm: CPU plan over {len(plan)} batches {time.time() - t0:.1f}s", file=sys.stderr)
    del adj
    edges, sec, _ = oracle_sample(g, neg, plan, first + W, K, sub_bs, threads)
    value = edges / sec
    sample = f"{K} consecutive whole batches from batch {first + W} ({edges} edges), {sec:.1f}s"
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": a.gpus, "steps": K,
            "warmup": W, "ms_per_step": sec * 1e3 / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(g, spec, first + W),
            "cpu_baseline": {"value": value, "unit": "edges/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


if __name__ == "__main__":
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)

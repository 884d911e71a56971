#!/usr/bin/env python
"""Benchmark of the minibatch hot path: k-hop neighbor sampling + feature gather.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one `sample_batches`-sized round of BATCHES_PER_STEP seed batches
(batch size, fanout, graph and feature shape from the workload), each batch
sampled, deduplicated, relabelled and its feature rows gathered.  Prints ONE
JSON line (rank 0).  Inputs are seeded synthetic stand-ins generated in place
(R-MAT graph, ~N(0,1) features); no dataset is read.

  value   sampled edges/s with the graph, features and seed batches resident in
          HBM, driven through the C ABI (ag_loader_*), whole job over all GPUs.
  e2e     the same metric through the public Python API (NeighborLoader.submit /
          next_batch) with host seed arrays copied to the device and the batch
          counts read back every batch; the sampled batch itself stays in GPU
          memory, where the training step consumes it.
  --impl reference   the CPU restatement of the reference's sampler + gather
          (oracle/, C + OpenMP) on the host cores, same workload.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BATCHES_PER_STEP = 16
METRIC = "sampled edges/s (k-hop sampling + dedup/relabel + feature gather)"

WORKLOADS = {
    # 100M-vertex R-MAT, 2B edges, 256-dim bf16 features, batch 1024, fanout [25, 10]
    "c2": dict(nodes=100_000_000, edges=2_000_000_000, dim=256, dtype="bf16", batch=1024, fanout=[25, 10],
               weighted=False, label="C2: R-MAT 100M vertices / 2B edges, 256-dim bf16, batch 1024, fanout [25,10]"),
    # 1M-vertex R-MAT, 16M edges, 128-dim f32, batch 128, fanout [15, 10]
    "c1": dict(nodes=1 << 20, edges=16 << 20, dim=128, dtype="f32", batch=128, fanout=[15, 10], weighted=False,
               label="C1: R-MAT 1M vertices / 16M edges, 128-dim f32, batch 128, fanout [15,10]"),
    # 10M-vertex weighted R-MAT, 200M edges, 128-dim f16, batch 512, fanout [15, 10, 5]
    "c3": dict(nodes=10_000_000, edges=200_000_000, dim=128, dtype="f16", batch=512, fanout=[15, 10, 5],
               weighted=True, label="C3: weighted R-MAT 10M vertices / 200M edges, 128-dim f16, batch 512, fanout [15,10,5]"),
    # C2's batch shape and feature rows on a graph small enough to profile (features 2 GB, CSR 0.3 GB)
    "c2s": dict(nodes=4_000_000, edges=64_000_000, dim=256, dtype="bf16", batch=1024, fanout=[25, 10],
                weighted=False, label="C2-small: R-MAT 4M vertices / 64M edges, 256-dim bf16, batch 1024, fanout [25,10]"),
    "tiny": dict(nodes=1 << 16, edges=1 << 20, dim=64, dtype="bf16", batch=256, fanout=[10, 5], weighted=False,
                 label="tiny: R-MAT 64K vertices / 1M edges, 64-dim bf16, batch 256, fanout [10,5]"),
}
GRAPH_SEED, FEATURE_SEED, SEEDS_SEED, SAMPLER_SEED = 1, 2, 3, 42

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per gathered row of
# k_gather_vec, from the ncu capture summarised in
# profiles/k_gather_vec_c2small_ncu_full.md: 647.6 MB for a launch over 495,171 rows
# of 256 bf16 -> f32 (1536 algorithmic bytes per row).
NCU_DRAM_BYTES_PER_ROW = {"bf16256": 1308}


def sector(x: int) -> int:
    return (x + 31) // 32 * 32


def gather_bytes_per_row(w) -> int:
    esize = 4 if w["dtype"] == "f32" else 2
    return sector(w["dim"] * esize) + w["dim"] * 4


def sampling_bytes(edges: int, nodes: int, frontier: int) -> int:
    """Algorithmic bytes of the sampling kernels: per frontier vertex one offsets
    sector; per emitted edge one destination sector (upper bound: picks of a
    sampled row are scattered), 24 B of edge outputs and a dedup probe sector read
    and written; per new vertex 4 B (nodes) + 32 B (frontier entry)."""
    return frontier * 32 + edges * (32 + 24 + 64) + nodes * 36


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return 6650.0, "fallback (earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        for l in rows:
            f = [x.strip() for x in l.split(",")]
            try:
                sm.append(float(f[0])); smax = float(f[1])
            except Exception:
                continue
            for name, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- #
#  reference arm: the CPU restatement on the host cores                        #
# --------------------------------------------------------------------------- #
def cpu_threads() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def host_description() -> str:
    """`nproc` and the CPU model name of the box the CPU legs ran on."""
    model = "unknown CPU"
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                model = line.split(":", 1)[1].strip()
                break
    except OSError:
        pass
    return f"{cpu_threads()} logical CPUs, {model}"


def host_seed_batches(w, first_batch: int, count: int) -> np.ndarray:
    from aethergraph_b200 import synth

    return np.concatenate([synth.seed_batch(w["nodes"], w["batch"], SEEDS_SEED, first_batch + i)
                           for i in range(count)]) if count else np.empty(0, dtype=np.uint32)


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # one CPU, one measurement: the other ranks exit without work
    from oracle import ago

    ago.build()
    threads = cpu_threads()
    t_setup = time.time()
    offsets, dst = ago.synth_rmat_csr(w["nodes"], w["nodes"], w["edges"], GRAPH_SEED, threads=threads)
    payload = ago.synth_features(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED, threads=threads)
    if w["weighted"]:
        raise SystemExit(json.dumps({"impl": "reference", "unavailable":
                                     "weighted workloads take their weights from the GPU generator"}))
    t_setup = time.time() - t_setup
    s = ago.Sampler(offsets, dst, w["fanout"], seed=SAMPLER_SEED)
    per_step = BATCHES_PER_STEP
    total = (args.warmup + args.steps) * per_step
    seeds = host_seed_batches(w, 0, total)
    bs = w["batch"]
    if args.warmup:
        s.bench(payload, w["dim"], w["dtype"], seeds[:args.warmup * per_step * bs], bs, 0, threads)
    t0 = time.time()
    r = s.bench(payload, w["dim"], w["dtype"], seeds[args.warmup * per_step * bs:], bs,
                args.warmup * per_step, threads)
    wall = time.time() - t0
    secs = r["seconds"]
    value = r["edges"] / secs
    gbs = r["nodes"] * gather_bytes_per_row(w) / secs / 1e9
    sample = f"{args.steps} steps x {per_step} batches of {bs} seeds (the full step, all {threads} host threads)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": secs * 1e3 / max(args.steps, 1),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u32 ids / " + w["dtype"] + "->f32",
        "data": "synthetic (seeded R-MAT graph + ~N(0,1) features generated on the host by the generator's CPU twin)",
        "config": {"workload": w["label"], "batches_per_step": per_step, "rng_mode": "wyrand_exact",
                   "inputs_larger_than_l2": True, "implementation":
                   "C restatement of the reference's Rust CPU sampler + gather (no Rust toolchain on this image)"},
        "gather_gbs": gbs, "edges": r["edges"], "nodes": r["nodes"], "checksum": f"{r['checksum']:016x}",
        "setup_s": round(t_setup, 1), "wall_s": round(wall, 3),
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": threads, "kind": "port", "sample": sample,
                         "host": host_description()},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- #
#  device arm                                                                  #
# --------------------------------------------------------------------------- #
def run_device(args, w):
    import torch
    import torch.distributed as dist

    import aethergraph_b200 as ag
    from aethergraph_b200 import _lib, synth
    from aethergraph_b200.loader import NeighborLoader
    from aethergraph_b200.sampler import _Buffers

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: aethergraph_b200 has no CPU path "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L = _lib.lib()

    # ---- inputs, resident in HBM (CSR and features replicated per GPU) ------
    t_setup = time.time()
    g = synth.rmat_graph(w["nodes"], w["edges"], GRAPH_SEED, weight_sigma=1.0 if w["weighted"] else 0.0)
    if args.features != "replicated" and world > 1:
        # every rank holds 1/world of the rows; remote rows cross NVLink inside the gather kernel.
        # "sharded": rows dealt round-robin (balanced); "sharded-range": contiguous vertex ranges.
        from aethergraph_b200 import dist as agd

        layout = "range" if args.features == "sharded-range" else "cyclic"
        local_shard = synth.features_shard(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED, rank, world, layout)
        feats = agd.open_sharded_features(local_shard)
    else:
        feats = synth.features(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED)
    torch.cuda.synchronize()
    t_setup = time.time() - t_setup
    cfg = ag.SamplingConfig(num_neighbors=w["fanout"], seed=SAMPLER_SEED, weighted=w["weighted"])
    per_step, bs = BATCHES_PER_STEP, w["batch"]
    n_batches = (args.warmup + args.steps) * per_step
    # rank r handles global batches r, r + world, ... (weak scaling: every rank does K steps)
    gidx = [rank + world * i for i in range(n_batches)]
    seeds_host = [synth.seed_batch(w["nodes"], bs, SEEDS_SEED, b) for b in gidx]
    seeds_dev = torch.from_numpy(np.concatenate(seeds_host).view(np.int32)).to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    # ---- value: C ABI, inputs resident, recycled output buffers ------------
    threads = args.threads
    # Batches per launch chain: large chains amortise the per-kernel latency of the
    # sampling stages, but every worker should still see several chains in the timed region.
    if args.group:
        group = args.group
    else:
        per_worker = args.steps * per_step // (3 * threads)
        group = 32 if per_worker >= 32 else 16 if per_worker >= 16 else 8
    depth = args.depth if args.depth else max(8, group // 2)
    h = C.c_void_p()
    ccfg = cfg._to_c(SAMPLER_SEED, bs)
    _lib.check(L.ag_loader_create(g._h, feats._h, C.byref(ccfg), 1, depth, threads, group, 1, C.byref(h)))
    mn, me = C.c_uint64(), C.c_uint64()
    _lib.check(L.ag_loader_bounds(h, bs, C.byref(mn), C.byref(me)))
    # One thread both submits and consumes here, so it must never block in submit:
    # keep no more batches outstanding than the loader's work queue (8 x depth) holds.
    window = min(8 * depth, depth + threads * group + group)
    ring = [_Buffers.alloc(dev, mn.value, me.value, bs, True, w["dim"]) for _ in range(window)]
    R = len(ring)
    batch = _lib.Batch()
    stats0 = _lib.LoaderStats()
    stats1 = _lib.LoaderStats()

    # Argument arrays for ag_loader_submit_many / ag_loader_next_many, built once.
    base = seeds_dev.data_ptr()
    idx_all = (C.c_int64 * n_batches)(*gidx)
    ptr_all = (C.c_void_p * n_batches)(*[base + 4 * bs * i for i in range(n_batches)])
    len_all = (C.c_uint64 * n_batches)(*([bs] * n_batches))
    ring_c = (_lib.SubgraphBuffers * (R + group))(*[ring[j % R].c for j in range(R + group)])
    out_batches = (_lib.Batch * 64)()
    n_out = C.c_uint32()
    sz_i64, sz_ptr, sz_u64, sz_buf = C.sizeof(C.c_int64), C.sizeof(C.c_void_p), C.sizeof(C.c_uint64), \
        C.sizeof(_lib.SubgraphBuffers)

    recent: list = []  # (n_id pointer, node count) of the last `group` delivered batches

    def run_resident(first: int, count: int):
        """Submit batches [first, first+count) with device seeds; returns (edges, nodes)."""
        edges = nodes = 0
        submitted = delivered = 0
        while delivered < count:
            while submitted < count and submitted - delivered + min(group, count - submitted) <= R:
                i = first + submitted
                n = min(group, count - submitted)
                _lib.check(L.ag_loader_submit_many(
                    h, n, C.byref(idx_all, i * sz_i64), C.byref(ptr_all, i * sz_ptr), C.byref(len_all, i * sz_u64),
                    _lib.AG_MEM_DEVICE, C.byref(ring_c, (i % R) * sz_buf), None, None))
                submitted += n
            _lib.check(L.ag_loader_next_many(h, -1, 64, out_batches, C.byref(n_out)))
            for j in range(n_out.value):
                edges += out_batches[j].counts.num_edges
                nodes += out_batches[j].counts.num_nodes
                recent.append((out_batches[j].bufs.n_id, out_batches[j].counts.num_nodes))
            del recent[:-group]
            delivered += n_out.value
        return edges, nodes

    # NOTE: seeded loaders number batches by submission; to keep every rank's
    # batch b on ag_batch_seed(seed, b) the loader is fed consecutive positions
    # and the global batch index only picks the seed ids.
    run_resident(0, args.warmup * per_step)
    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    _lib.check(L.ag_loader_stats_get(h, C.byref(stats0)))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    wall0 = time.time()
    e0.record()
    edges, nodes = run_resident(args.warmup * per_step, args.steps * per_step)
    e1.record()
    barrier()
    wall1 = time.time()
    ms = max_over_ranks(e0.elapsed_time(e1))
    _lib.check(L.ag_loader_stats_get(h, C.byref(stats1)))
    clk = clocks.stop(wall0, wall1)
    tot_edges, tot_nodes = sum_over_ranks(edges), sum_over_ranks(nodes)
    value = tot_edges / (ms * 1e-3)
    row_bytes = gather_bytes_per_row(w)
    gather_gbs = tot_nodes * row_bytes / (ms * 1e-3) / 1e9
    g_ms = stats1.gather_ms - stats0.gather_ms
    s_ms = stats1.sample_ms - stats0.sample_ms
    n_timed = args.steps * per_step
    peak, peak_src = peaks()
    achieved = nodes * row_bytes / (g_ms * 1e-3) / 1e9 if g_ms > 0 else None
    # one gather launch per chain (a chain covers up to `group` batches, the batch is blockIdx.y)
    launches = max(int(stats1.chains - stats0.chains), 1)
    per_row = NCU_DRAM_BYTES_PER_ROW.get(w["dtype"] + str(w["dim"]))
    roofline = {
        "kernel": "k_gather_vec (feature-row gather + upcast)", "bound": "hbm",
        "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": (achieved / peak) if achieved else None, "peak_source": peak_src,
        "frac_of_nominal_8tbs": (achieved / 8000.0) if achieved else None,
        "bytes_per_launch": nodes * row_bytes / launches, "ms_per_launch": g_ms / launches,
        "launches": launches, "traffic": (per_row * nodes / launches) if per_row else None,
        "traffic_note": "ncu dram bytes per gathered row on the C2-small capture x rows per launch",
        "note": "per-launch time from CUDA events on the launching stream while the other "
                "streams' sampling kernels run beside it",
        "pipeline": {"algorithmic_gbs": (tot_nodes * row_bytes + sampling_bytes(tot_edges, tot_nodes, tot_nodes))
                     / (ms * 1e-3) / 1e9,
                     "frac_of_peak": ((tot_nodes * row_bytes + sampling_bytes(tot_edges, tot_nodes, tot_nodes))
                                      / (ms * 1e-3) / 1e9) / (peak * world),
                     "sample_ms_per_batch": s_ms / n_timed},
    }
    # The same kernel on its own: the node ids of the last delivered batches, gathered
    # by one standalone launch per repetition with nothing else on the GPU (what the
    # committed ncu capture measures; the in-pipeline figure above shares the SMs and
    # HBM with the other workers' sampling kernels).
    if recent and not args.only_value:
        holder = _Buffers(ring[0].c, ring, dev, w["dim"])  # the ring keeps the memory alive
        ids = torch.cat([holder.view(ptr, (int(n),), "<i8") for ptr, n in recent])
        x_alone = torch.empty((ids.shape[0], w["dim"]), dtype=torch.float32, device=dev)
        for _ in range(3):
            feats.gather(ids, out=x_alone)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize(dev)
        reps = 10
        a0.record()
        for _ in range(reps):
            feats.gather(ids, out=x_alone)
        a1.record()
        torch.cuda.synchronize(dev)
        alone_ms = a0.elapsed_time(a1) / reps
        alone_gbs = ids.shape[0] * row_bytes / (alone_ms * 1e-3) / 1e9
        roofline["alone"] = {"achieved": alone_gbs, "frac": alone_gbs / peak, "ms_per_launch": alone_ms,
                             "rows_per_launch": int(ids.shape[0]), "launches": reps,
                             "note": "same kernel and ids, one launch at a time on an otherwise idle GPU; "
                                     "working set per launch exceeds L2"}
        del ids, x_alone
    L.ag_loader_free(h)
    del ring

    # ---- e2e: public Python API, host seeds in, counts back -----------------
    e2e_value = ms_e2e = host_value = host_ms = None
    d2h_host = 0
    if not args.only_value:
        loader = NeighborLoader(g, cfg, prefetch_depth=depth, sampler_threads=threads, features=feats, group=group)
        pinned = None

        def run_e2e(first: int, count: int, to_host: bool = False):
            """Host seed arrays in through the public API; `to_host` also copies every
            batch (ids, local edge index, feature rows) into pinned host memory."""
            nonlocal d2h_host
            edges = submitted = delivered = 0
            while delivered < count:
                while submitted < count and submitted - delivered < window:
                    b = (first + submitted) % n_batches
                    loader.submit(gidx[b], seeds_host[b])
                    submitted += 1
                _, sg, x = loader.next_batch()
                if to_host:
                    nn, ne = sg.num_nodes, sg.num_edges
                    pinned["n_id"][:nn].copy_(sg.nodes_t, non_blocking=True)
                    pinned["ei"][:, :ne].copy_(sg.edge_index_local_t, non_blocking=True)
                    pinned["x"][:nn].copy_(x, non_blocking=True)
                    torch.cuda.current_stream().synchronize()
                    d2h_host += nn * 8 + ne * 16 + nn * w["dim"] * 4
                edges += sg.num_edges
                delivered += 1
            return edges

        # warm-up long enough for the loader's buffer pool to reach its working size
        run_e2e(0, max(args.warmup * per_step, 2 * window))
        barrier()
        e0.record()
        edges_e2e = run_e2e(args.warmup * per_step, args.steps * per_step)
        e1.record()
        barrier()
        ms_e2e = max_over_ranks(e0.elapsed_time(e1))
        e2e_value = sum_over_ranks(edges_e2e) / (ms_e2e * 1e-3)
        # the same with every batch also copied to pinned host memory (what a host-side consumer sees)
        pinned = {"n_id": torch.empty(mn.value, dtype=torch.int64).pin_memory(),
                  "ei": torch.empty((2, me.value), dtype=torch.int64).pin_memory(),
                  "x": torch.empty((mn.value, w["dim"]), dtype=torch.float32).pin_memory()}
        run_e2e(0, per_step, True)
        d2h_host = 0
        barrier()
        e0.record()
        edges_host = run_e2e(args.warmup * per_step, args.steps * per_step, True)
        e1.record()
        barrier()
        host_ms = max_over_ranks(e0.elapsed_time(e1))
        host_value = sum_over_ranks(edges_host) / (host_ms * 1e-3)
        loader.shutdown()
        del loader

    # ---- CPU baseline beside it (rank 0, one GPU only) ----------------------
    cpu = None
    parity = None
    if rank == 0 and world == 1 and not args.no_cpu and not args.only_value:
        cpu, parity = cpu_baseline(g, feats, w, cfg)

    if rank == 0:
        hops = len(w["fanout"])
        line = {
            "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / max(args.steps, 1), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u32 ids / " + w["dtype"] + "->f32",
            "data": "synthetic (seeded R-MAT graph + ~N(0,1) features generated in HBM)",
            "config": {"workload": w["label"], "batches_per_step": per_step, "rng_mode": "wyrand_exact",
                       "sampler_threads": threads, "group": group, "prefetch_depth": depth, "parallelism": f"dp{world}",
                       "features": ("%s, remote rows over NVLink (%d/%d of the rows)"
                                    % ("sharded by contiguous vertex range" if args.features == "sharded-range"
                                       else "sharded round-robin by vertex id", world - 1, world))
                       if (args.features != "replicated" and world > 1) else "replicated",
                       "inputs_larger_than_l2": True},
            "gather_gbs": gather_gbs, "edges_per_step": tot_edges / max(args.steps, 1),
            "rows_per_step": tot_nodes / max(args.steps, 1), "setup_s": round(t_setup, 1),
            "clocks": clk, "roofline": roofline, "cpu_baseline": cpu, "parity_full_scale": parity,
            "e2e": None if e2e_value is None else {
                "value": e2e_value, "unit": "edges/s", "h2d_bytes_per_step": world * per_step * bs * 4,
                "d2h_bytes_per_step": world * per_step * C.sizeof(_lib.SampleCounts),
                "ms_per_step": ms_e2e / max(args.steps, 1),
                "note": "public Python API: host seed arrays in, per-batch counts out; the sampled batch and "
                        "its feature rows stay in GPU memory, where the training step reads them",
                "host_results": {"value": host_value, "unit": "edges/s", "ms_per_step": host_ms / max(args.steps, 1),
                                 "d2h_bytes_per_step": d2h_host / max(args.steps, 1),
                                 "note": "same calls, every batch (int64 ids, local edge index, f32 feature rows) "
                                         "also copied to pinned host memory: PCIe-bound"}},
            # one launch chain per group of batches (the batch is blockIdx.y): seed insert,
            # hops + 1 assign, hops pick, finalize, gather
            "gpu_launches": world * -(-n_timed // group) * (2 * hops + 4),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        barrier()  # no rank frees its feature shard while a peer may still be reading it
        del feats
        barrier()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
#  heterogeneous workload (C4): secondary, `--workload c4` / `c4s`               #
# --------------------------------------------------------------------------- #
HETERO = {
    # user / post / comment / subreddit; three stored relations plus their reverses (user seeds
    # need incoming edge types); fanouts votes [15,10], writes [10,5], belongs_to [3,2]
    "c4": dict(scale=1, label="C4: user 50M / post 20M / comment 100M / subreddit 100K, 6 edge types, batch 1024"),
    "c4s": dict(scale=10, label="C4 at 1/10 scale: user 5M / post 2M / comment 10M / subreddit 10K, 6 edge types, batch 1024"),
}


def hetero_cpu_leg(g, nn, ets, fan, host_rel, seeds, stores):
    """The CPU restatement of the hetero sampler on the same relations (one thread,
    sampling only) and a bit-for-bit check of one batch and its gathered rows."""
    import torch

    import aethergraph_b200 as ag
    from oracle import ago

    # reverse relation = transpose of the stored one
    names = list(nn)
    rels = []
    for (s, r, d) in ets[:3]:
        off, dd = host_rel[r]
        rels.append((names.index(s), names.index(d), off, dd))
    for (s, r, d) in ets[3:]:
        off, dd = host_rel[r[4:]]
        t_off, t_src = ago.transpose(off, dd, nn[d], nn[s])
        rels.append((names.index(s), names.index(d), t_off, t_src))
    o = ago.HeteroSampler([nn[k] for k in names], rels, fan, seed=SAMPLER_SEED)
    ok, cpu_edges, t_cpu = True, 0, time.time()
    nb_cpu = 0
    while time.time() - t_cpu < 6.0 and nb_cpu < len(seeds):
        o.reseed(ago.batch_seed(SAMPLER_SEED, nb_cpu))
        want = o.sample(0, seeds[nb_cpu])
        cpu_edges += sum(len(x) for x in want["edge_src_local"])
        nb_cpu += 1
    t_cpu = time.time() - t_cpu
    # parity of batch 0 at this scale, bit for bit
    s1 = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig(dict(zip(ets, fan)), seed=ago.batch_seed(SAMPLER_SEED, 0)))
    got = s1.sample("user", seeds[0]).raw_u32()
    o.reseed(ago.batch_seed(SAMPLER_SEED, 0))
    want = o.sample(0, seeds[0])
    for k in ("nodes", "edge_src_local", "edge_dst_local"):
        ok = ok and all(np.array_equal(a, b) for a, b in zip(got[k], want[k]))
    # ... and the rows gathered for it: x of a type == the type's stored rows at its node ids
    s2 = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig(dict(zip(ets, fan)), seed=7), features=stores)
    sg2 = s2.sample("user", seeds[1])
    for nt in nn:
        ids = sg2.nodes_t(nt)
        if ids.shape[0]:
            ok = ok and bool(torch.equal(sg2.x_t(nt), stores[nt].gather(ids)))
    cpu = {"value": cpu_edges / t_cpu, "unit": "edges/s", "cores": 1, "kind": "port",
           "sample": f"{nb_cpu} batches, one thread, sampling only, {t_cpu:.1f} s", "host": host_description()}
    return cpu, bool(ok)


def run_hetero(args, hw):
    """Sampled edges/s of the heterogeneous sampler + per-type feature gather on one
    GPU, with the CPU restatement timed beside it on the same relations."""
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from oracle import ago

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    sc = hw["scale"]
    nn = {"user": 50_000_000 // sc, "post": 20_000_000 // sc, "comment": 100_000_000 // sc, "subreddit": 100_000 // sc}
    t0 = time.time()
    votes = synth.rmat_relation(nn["user"], nn["post"], 30 * nn["user"], 11)
    writes = synth.rmat_relation(nn["user"], nn["comment"], 8 * nn["user"], 12)
    belongs_dst = torch.from_numpy((synth._mix(np.arange(nn["post"], dtype=np.uint64) + np.uint64(13))
                                    % np.uint64(nn["subreddit"])).astype(np.int32)).cuda()
    belongs = (torch.arange(nn["post"] + 1, dtype=torch.int64, device="cuda"), belongs_dst)
    rel = {"votes": votes, "writes": writes, "belongs_to": belongs}
    src = {k: synth.relation_sources(v[0]) for k, v in rel.items()}
    ets = [("user", "votes", "post"), ("user", "writes", "comment"), ("post", "belongs_to", "subreddit"),
           ("post", "rev_votes", "user"), ("comment", "rev_writes", "user"), ("subreddit", "rev_belongs_to", "post")]
    arrays = [(src["votes"], votes[1]), (src["writes"], writes[1]), (src["belongs_to"], belongs[1]),
              (votes[1], src["votes"]), (writes[1], src["writes"]), (belongs[1], src["belongs_to"])]
    fan = [[15, 10], [10, 5], [3, 2], [15, 10], [10, 5], [3, 2]]
    g = ag.HeteroCsrGraph.from_device_edges(nn, [(*et, *a) for et, a in zip(ets, arrays)])
    host_rel = None
    if not args.no_cpu and sc > 1:  # the CPU leg needs the relations on the host (skipped at full scale)
        host_rel = {k: (v[0].cpu().numpy().astype(np.uint64), v[1].cpu().numpy().view(np.uint32)) for k, v in rel.items()}
    del src, arrays, votes, writes, belongs, rel
    torch.cuda.empty_cache()
    dims = {"user": 128, "post": 128, "comment": 128, "subreddit": 64}
    stores = {nt: synth.features(nn[nt], dims[nt], "bf16", 20 + i) for i, nt in enumerate(nn)}
    torch.cuda.synchronize()
    t_setup = time.time() - t0
    cfg = ag.HeteroSamplingConfig(dict(zip(ets, fan)), seed=SAMPLER_SEED)
    bs, per_step = 1024, BATCHES_PER_STEP
    n_batches = (args.warmup + args.steps) * per_step
    seeds = [synth.seed_batch(nn["user"], bs, SEEDS_SEED, b) for b in range(n_batches)]
    group = args.group if args.group else 16
    loader = ag.HeteroNeighborLoader(g, cfg, "user", prefetch_depth=max(8, group), sampler_threads=args.threads,
                                     features=stores, group=group)
    row_bytes = {nt: dims[nt] * 2 + dims[nt] * 4 for nt in nn}
    window = min(8 * max(8, group) - 1, args.threads * group + group)

    def run(first, count):
        edges = rows_b = sub = got = 0
        while got < count:
            while sub < count and sub - got < window:
                loader.submit(first + sub, seeds[first + sub]); sub += 1
            _, sg = loader.next_batch()
            for t, nt in enumerate(nn):  # the rows of every type were gathered in the batch's launch chain
                rows_b += int(sg._c.nodes[t]) * row_bytes[nt]
            edges += int(sg._c.total_edges)
            got += 1
        return edges, rows_b

    run(0, args.warmup * per_step)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    edges, gbytes = run(args.warmup * per_step, args.steps * per_step)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    loader.shutdown()
    cpu, ok = None, None
    if not args.no_cpu and sc > 1:
        cpu, ok = hetero_cpu_leg(g, nn, ets, fan, host_rel, seeds, stores)
    line = {
        "metric": METRIC, "value": edges / (ms * 1e-3), "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / max(args.steps, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32 ids / bf16->f32", "data": "synthetic (per-relation R-MAT generated in HBM)",
        "config": {"workload": hw["label"], "batches_per_step": per_step, "sampler_threads": args.threads, "group": group,
                   "fanout": {"/".join(et): f for et, f in zip(ets, fan)}},
        "gather_gbs": gbytes / (ms * 1e-3) / 1e9, "edges_per_step": edges / max(args.steps, 1), "setup_s": round(t_setup, 1),
        "cpu_baseline": cpu, "parity_full_scale": ok,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(g, feats, w, cfg):
    """Times the CPU restatement on a bounded sample of the same workload (graph and
    features copied back from the GPU) and checks two full-size batches bit for bit."""
    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from oracle import ago

    ago.build()
    if w["nodes"] * w["dim"] * (4 if w["dtype"] == "f32" else 2) + w["edges"] * 4 > 150e9:
        return None, None
    n = g.num_nodes
    offsets, dst, weights = g.to_host()
    payload = feats.payload_to_host()
    threads = cpu_threads()
    s = ago.Sampler(offsets, dst, w["fanout"], weights=weights, weighted=w["weighted"], seed=SAMPLER_SEED)
    bs = w["batch"]
    # bounded sample: batches 0, 1, ... of the workload's seed stream, grown until
    # the timed run lasts about ten seconds
    seeds_host = [synth.seed_batch(w["nodes"], bs, SEEDS_SEED, b) for b in range(4 * threads)]
    nb, cap = len(seeds_host), 1 << 16
    while True:
        seeds = np.concatenate(seeds_host[:nb])
        r = s.bench(payload, w["dim"], w["dtype"], seeds, bs, 0, threads)
        if r["seconds"] >= 8.0 or nb >= cap:
            break
        nb = min(cap, max(nb + 1, int(nb * min(16.0, 12.0 / max(r["seconds"], 1e-3)))))
        seeds_host += [synth.seed_batch(w["nodes"], bs, SEEDS_SEED, b) for b in range(len(seeds_host), nb)]
    # one thread, one persistent sampler reused across batches (the reference's NeighborSampler reuse)
    n1 = max(4, min(nb, int(4.0 * nb / max(r["seconds"], 1e-3) / threads)))
    r1 = s.bench(payload, w["dim"], w["dtype"], np.concatenate(seeds_host[:n1]), bs, 0, 1)
    cpu = {"value": r["edges"] / r["seconds"], "unit": "edges/s", "cores": threads, "kind": "port",
           "gather_gbs": r["nodes"] * gather_bytes_per_row(w) / r["seconds"] / 1e9,
           "single_thread": {"value": r1["edges"] / r1["seconds"], "unit": "edges/s",
                             "sample": f"{n1} batches, 1 thread, {r1['seconds']:.2f} s"},
           "host": host_description(),
           "sample": f"{nb} batches of {bs} seeds of the same workload (graph and features copied back from "
                     f"the GPU), {threads} threads, {r['seconds']:.2f} s"}
    # full-size parity: batch positions 0 and 1, bit for bit
    sampler = ag.ParallelBatchSampler(g, cfg, features=feats, streams=2)
    ok = True
    for pos, sg in enumerate(sampler.sample_batches(seeds_host[:2])):
        s.reseed(ago.batch_seed(SAMPLER_SEED, pos))
        want = s.sample(seeds_host[pos])
        got = sg.raw_u32()
        for k in ("nodes", "edge_src", "edge_dst", "edge_ids", "src_local", "dst_local", "seed_locals"):
            ok = ok and np.array_equal(got[k], want[k])
        xw = ago.gather(payload, n, w["dim"], w["dtype"], want["nodes"])
        ok = ok and np.array_equal(sg.x.cpu().numpy().view(np.uint32), xw.view(np.uint32))
    cpu["reference_gpu_hop1"] = reference_gpu_hop1(g, w, seeds_host)
    return cpu, bool(ok)


def reference_gpu_hop1(g, w, seeds_host):
    """Secondary baseline: hop 1 of the workload (Philox fast mode, fanout = first
    hop) through the reference's OWN CUDA kernel `warp_sample_neighbors` — compiled
    from the reference checkout into oracle/_ref/ — against this library's
    ag_sample_hop_reservoir, same device arrays, outputs compared bit for bit."""
    import torch

    from aethergraph_b200 import _lib
    from aethergraph_b200.sampler import reservoir_hop
    from oracle import ago

    if not os.path.exists(ago.REF_WARP_SAMPLER):
        return None
    fanout = int(w["fanout"][0])
    nodes = np.concatenate(seeds_host[:64]).astype(np.uint64)  # 64 batches' seeds in one launch
    nodes_dev = torch.from_numpy(nodes.view(np.int64)).cuda()
    po, pd, pw = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _lib.check(_lib.lib().ag_graph_device_ptrs(g._h, C.byref(po), C.byref(pd), C.byref(pw)))
    out = torch.empty((len(nodes), fanout), dtype=torch.int32, device="cuda")
    cnt = torch.empty((len(nodes),), dtype=torch.int32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / reps

    ref_us = timed(lambda: ago.ref_warp_sample(po.value, pd.value, g.num_nodes, nodes_dev.data_ptr(), out.data_ptr(),
                                               cnt.data_ptr(), len(nodes), fanout, SAMPLER_SEED, 0, st))
    mine = [None]

    def run_mine():
        mine[0] = reservoir_hop(g, nodes_dev, fanout, SAMPLER_SEED, 0)

    own_us = timed(run_mine)
    same = bool(torch.equal(mine[0][0], out) and torch.equal(mine[0][1], cnt))
    return {"nodes": int(len(nodes)), "fanout": fanout, "reference_kernel_us": ref_us, "this_library_us": own_us,
            "identical_output": same,
            "note": "warp_sample_neighbors compiled unmodified from the reference checkout vs ag_sample_hop_reservoir"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default=os.environ.get("AG_BENCH_WORKLOAD", "c2"),
                    choices=sorted(WORKLOADS) + sorted(HETERO))
    ap.add_argument("--threads", type=int, default=int(os.environ.get("AG_BENCH_THREADS", "0")),
                    help="loader worker threads, each with its own CUDA stream (0: 3, heterogeneous workloads 2)")
    ap.add_argument("--depth", type=int, default=0, help="prefetch depth (0: max(8, group / 2))")
    ap.add_argument("--group", type=int, default=int(os.environ.get("AG_BENCH_GROUP", "0")),
                    help="batches a worker runs as one launch chain (0: chosen from --steps)")
    ap.add_argument("--features", default="replicated", choices=["replicated", "sharded", "sharded-range"],
                    help="with more than one GPU: every GPU holds all feature rows, or 1/N of them "
                         "(dealt round-robin, or as contiguous vertex ranges)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--only-value", action="store_true",
                    help="run the resident (C ABI) leg only: no e2e, no CPU baseline (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    if args.threads <= 0:
        args.threads = 2 if args.workload in HETERO else 3
    if args.workload in HETERO:
        return run_hetero(args, HETERO[args.workload])
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    else:
        run_device(args, w)


if __name__ == "__main__":
    main()

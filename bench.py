#!/usr/bin/env python
"""Benchmark of the minibatch hot path: k-hop neighbor sampling + feature gather.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = the workload's `batches_per_step` seed batches (512 for C2; batch size,
fanout, graph and feature shape from the workload), each batch sampled,
deduplicated, relabelled and its feature rows gathered.  The timed region of K
steps is repeated (`--repeats`, default 5) and the median is reported with the
minimum and maximum.  Prints ONE JSON line (rank 0).  Inputs are seeded synthetic
stand-ins generated in place (R-MAT graph, ~N(0,1) features); no dataset is read.

  value   sampled edges/s with the graph, features and seed batches resident in
          HBM, driven through the C ABI (ag_loader_*), whole job over all GPUs.
  e2e     the same metric through the public Python API (NeighborLoader.submit /
          next_batch) with host seed arrays copied to the device and the batch
          counts read back every batch; the sampled batch itself stays in GPU
          memory, where the training step consumes it.
  sharded (2 or more GPUs) the same resident leg once more with the feature rows
          split over the GPUs (1/N each, dealt round-robin) and remote rows
          fetched over NVLink in address order; a batch is compared bit for bit
          with the rows of the replicated table.
  secondary (1 GPU)  C1, C3 and the heterogeneous C4 at 1/10 size, each with its
          own CPU baseline and full-size parity check.
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

BATCHES_PER_STEP = 512   # default; a workload may carry its own `per_step`
METRIC = "sampled edges/s (k-hop sampling + dedup/relabel + feature gather)"

WORKLOADS = {
    # 100M-vertex R-MAT, 2B edges, 256-dim bf16 features, batch 1024, fanout [25, 10]
    "c2": dict(nodes=100_000_000, edges=2_000_000_000, dim=256, dtype="bf16", batch=1024, fanout=[25, 10],
               weighted=False, label="C2: R-MAT 100M vertices / 2B edges, 256-dim bf16, batch 1024, fanout [25,10]"),
    # 1M-vertex R-MAT, 16M edges, 128-dim f32, batch 128, fanout [15, 10]
    # small batches are bound by launch latency and host work per chain: long chains, two workers
    # (measured: 3 x 32 -> 0.78, 3 x 128 -> 1.46, 2 x 128 -> 2.16, 4 x 128 -> 0.93 G edges/s)
    "c1": dict(nodes=1 << 20, edges=16 << 20, dim=128, dtype="f32", batch=128, fanout=[15, 10], weighted=False,
               group=128, threads=2, depth=64,
               label="C1: R-MAT 1M vertices / 16M edges, 128-dim f32, batch 128, fanout [15,10]"),
    # 10M-vertex weighted R-MAT, 200M edges, 128-dim f16, batch 512, fanout [15, 10, 5]
    "c3": dict(nodes=10_000_000, edges=200_000_000, dim=128, dtype="f16", batch=512, fanout=[15, 10, 5],
               weighted=True, label="C3: weighted R-MAT 10M vertices / 200M edges, 128-dim f16, batch 512, fanout [15,10,5]"),
    # C2's batch shape and feature rows on a graph small enough to profile (features 2 GB, CSR 0.3 GB)
    "c2s": dict(nodes=4_000_000, edges=64_000_000, dim=256, dtype="bf16", batch=1024, fanout=[25, 10],
                weighted=False, label="C2-small: R-MAT 4M vertices / 64M edges, 256-dim bf16, batch 1024, fanout [25,10]"),
    "tiny": dict(nodes=1 << 16, edges=1 << 20, dim=64, dtype="bf16", batch=256, fanout=[10, 5], weighted=False,
                 per_step=32, label="tiny: R-MAT 64K vertices / 1M edges, 64-dim bf16, batch 256, fanout [10,5]"),
    # 500M-vertex R-MAT, 12B edges (52 GB CSR replicated per GPU), 128-dim bf16 features sharded over the GPUs
    # (128 GB in all), 4096 seeds per GPU and batch, fanout [15, 10, 5]; 2 or more GPUs
    "c5": dict(nodes=500_000_000, edges=12_000_000_000, dim=128, dtype="bf16", batch=4096, fanout=[15, 10, 5],
               weighted=False, per_step=32, group=4, threads=2, depth=4, sharded_only=True,
               label="C5: R-MAT 500M vertices / 12B edges, 128-dim bf16 sharded over the GPUs, batch 4096, fanout [15,10,5]"),
    # C5's batch shape and sharded features on a graph that fits next to anything (tests of the sharded leg)
    "c5s": dict(nodes=20_000_000, edges=480_000_000, dim=128, dtype="bf16", batch=4096, fanout=[15, 10, 5],
                weighted=False, per_step=32, group=4, threads=2, depth=4, sharded_only=True,
                label="C5-small: R-MAT 20M vertices / 480M edges, 128-dim bf16 sharded over the GPUs, batch 4096, fanout [15,10,5]"),
}
GRAPH_SEED, FEATURE_SEED, SEEDS_SEED, SAMPLER_SEED = 1, 2, 3, 42

# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per gathered row of
# k_gather_vec from one ncu capture of the C2-small workload: 647.6 MB for a launch
# over 495,171 rows of 256 bf16 -> f32 (1536 algorithmic bytes per row).
NCU_DRAM_BYTES_PER_ROW = {"bf16256": 1308}
NVLINK_PEER_COPY_GBS = 770.0  # measured peer copy bandwidth per direction per GPU on this pool


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


def per_step_of(w) -> int:
    return int(w.get("per_step", BATCHES_PER_STEP))


def common_config(w, world: int, features: str) -> dict:
    """The `config` keys both arms print (what is measured, not how)."""
    return {"workload": w["label"], "batches_per_step": per_step_of(w), "rng_mode": "wyrand_exact",
            "parallelism": f"dp{world}", "features": features, "inputs_larger_than_l2": True}


def run_reference(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # one CPU, one measurement: the other ranks exit without work
    from oracle import ago

    ago.build()
    threads = cpu_threads()
    if w["weighted"]:
        raise SystemExit(json.dumps({"impl": "reference", "unavailable":
                                     "weighted workloads take their weights from the GPU generator"}))
    if w["nodes"] * w["dim"] * (4 if w["dtype"] == "f32" else 2) + w["edges"] * 4 > 0.8 * host_memory_bytes():
        raise SystemExit(json.dumps({"impl": "reference", "unavailable":
                                     "the workload's graph and features do not fit this host's memory"}))
    t_setup = time.time()
    offsets, dst = ago.synth_rmat_csr(w["nodes"], w["nodes"], w["edges"], GRAPH_SEED, threads=threads)
    payload = ago.synth_features(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED, threads=threads)
    t_setup = time.time() - t_setup
    s = ago.Sampler(offsets, dst, w["fanout"], seed=SAMPLER_SEED)
    per_step = per_step_of(w)
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
        "data": "synthetic (seeded R-MAT graph + ~N(0,1) features; the reference arm generates them on the host "
                "with the generator's CPU twin, bit-identical to the device arm's inputs)",
        "config": common_config(w, args.gpus, "replicated"),
        "impl_config": {"implementation": "C restatement of the reference's Rust CPU sampler + gather "
                                          "(no Rust toolchain on this image)", "threads": threads},
        "gather_gbs": gbs, "edges": r["edges"], "nodes": r["nodes"], "checksum": f"{r['checksum']:016x}",
        "setup_s": round(t_setup, 1), "wall_s": round(wall, 3),
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": threads, "kind": "port", "sample": sample,
                         "host": host_description()},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def host_memory_bytes() -> int:
    try:
        return os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    except (ValueError, OSError):
        return 1 << 62


# --------------------------------------------------------------------------- #
#  device arm                                                                  #
# --------------------------------------------------------------------------- #
class ResidentLeg:
    """The C-ABI loader fed with device-resident seed batches and recycled output
    buffers: what `value` (and the sharded record) time."""

    def __init__(self, L, _lib, g, feats, ccfg, dev, w, threads, group, depth, seeds_dev, gidx, rank, world):
        from aethergraph_b200.sampler import _Buffers

        self.L, self._lib, self.group, self.w = L, _lib, group, w
        bs = w["batch"]
        self.h = C.c_void_p()
        _lib.check(L.ag_loader_create(g._h, feats._h, C.byref(ccfg), 1, depth, threads, group, 1, C.byref(self.h)))
        # global batch b = rank + world * i draws from batch_seed(seed, b) at any world size
        _lib.check(L.ag_loader_set_seed_sequence(self.h, rank, world))
        mn, me = C.c_uint64(), C.c_uint64()
        _lib.check(L.ag_loader_bounds(self.h, bs, C.byref(mn), C.byref(me)))
        self.mn, self.me = mn.value, me.value
        # One thread both submits and consumes, so it must never block in submit:
        # keep no more batches outstanding than the loader's work queue (8 x depth) holds.
        self.window = min(8 * depth, depth + threads * group + group)
        # The caller owns the output buffers and sizes them: the worst-case bound of a batch
        # (every pick a new vertex) is many times what this workload's batches produce, so a
        # first chain in full-size buffers measures them and the ring gets twice that.  A batch
        # that outgrew its buffers would come back as an error, not silently cut.
        cap_n, cap_e = self.mn, self.me
        probe_n = min(group, len(gidx))
        if probe_n and not w.get("full_size_buffers"):
            probe = [_Buffers.alloc(dev, self.mn, self.me, bs, True, w["dim"]) for _ in range(probe_n)]
            base0 = seeds_dev.data_ptr()
            idx = (C.c_int64 * probe_n)(*gidx[:probe_n])
            ptr = (C.c_void_p * probe_n)(*[base0 + 4 * bs * i for i in range(probe_n)])
            ln = (C.c_uint64 * probe_n)(*([bs] * probe_n))
            bufs = (_lib.SubgraphBuffers * probe_n)(*[b.c for b in probe])
            _lib.check(L.ag_loader_submit_many(self.h, probe_n, idx, ptr, ln, _lib.AG_MEM_DEVICE, bufs, None, None))
            got, seen_n, seen_e = 0, 0, 0
            out = (_lib.Batch * 64)()
            n_out = C.c_uint32()
            while got < probe_n:
                _lib.check(L.ag_loader_next_many(self.h, -1, 64, out, C.byref(n_out)))
                for j in range(n_out.value):
                    seen_n = max(seen_n, out[j].counts.num_nodes)
                    seen_e = max(seen_e, out[j].counts.num_edges)
                got += n_out.value
            cap_n = min(self.mn, 2 * seen_n + 4096)
            cap_e = min(self.me, 2 * seen_e + 4096)
            del probe
        self.cap_n, self.cap_e = cap_n, cap_e
        self.ring = [_Buffers.alloc(dev, cap_n, cap_e, bs, True, w["dim"]) for _ in range(self.window)]
        R = self.R = len(self.ring)
        n_batches = len(gidx)
        base = seeds_dev.data_ptr()
        self.idx_all = (C.c_int64 * n_batches)(*gidx)
        self.ptr_all = (C.c_void_p * n_batches)(*[base + 4 * bs * i for i in range(n_batches)])
        self.len_all = (C.c_uint64 * n_batches)(*([bs] * n_batches))
        self.ring_c = (_lib.SubgraphBuffers * (R + group))(*[self.ring[j % R].c for j in range(R + group)])
        self.out_batches = (_lib.Batch * 64)()
        self.n_out = C.c_uint32()
        self.recent: list = []  # (n_id pointer, x pointer, node count) of the last `group` delivered batches
        self.intervals: set = set()  # (begin, end) of every chain's gather on the device clock, in ms

    def run(self, first: int, count: int):
        """Submit batches [first, first + count) with device seeds; returns (edges, nodes)."""
        L, _lib, group, R = self.L, self._lib, self.group, self.R
        sz_i64, sz_ptr, sz_u64 = C.sizeof(C.c_int64), C.sizeof(C.c_void_p), C.sizeof(C.c_uint64)
        sz_buf = C.sizeof(_lib.SubgraphBuffers)
        edges = nodes = 0
        submitted = delivered = 0
        while delivered < count:
            while submitted < count and submitted - delivered + min(group, count - submitted) <= R:
                i = first + submitted
                n = min(group, count - submitted)
                _lib.check(L.ag_loader_submit_many(
                    self.h, n, C.byref(self.idx_all, i * sz_i64), C.byref(self.ptr_all, i * sz_ptr),
                    C.byref(self.len_all, i * sz_u64), _lib.AG_MEM_DEVICE, C.byref(self.ring_c, (i % R) * sz_buf),
                    None, None))
                submitted += n
            _lib.check(L.ag_loader_next_many(self.h, -1, 64, self.out_batches, C.byref(self.n_out)))
            for j in range(self.n_out.value):
                ob = self.out_batches[j]
                edges += ob.counts.num_edges
                nodes += ob.counts.num_nodes
                self.recent.append((ob.bufs.n_id, ob.bufs.x, ob.counts.num_nodes))
                if ob.counts.gather_end_ms > ob.counts.gather_begin_ms:
                    self.intervals.add((ob.counts.gather_begin_ms, ob.counts.gather_end_ms))
            del self.recent[:-group]
            delivered += self.n_out.value
        return edges, nodes

    def stats(self):
        s = self._lib.LoaderStats()
        self._lib.check(self.L.ag_loader_stats_get(self.h, C.byref(s)))
        return s

    def close(self):
        if self.h:
            self.L.ag_loader_free(self.h)
            self.h = None
        self.ring = None
        self.recent = []
        import torch

        torch.cuda.empty_cache()  # the ring came from torch's allocator; the library's own allocations need the room


def union_ms(intervals) -> float:
    """Total length of the union of (begin, end) intervals."""
    total, cur_b, cur_e = 0.0, None, None
    for b, e in sorted(intervals):
        if cur_e is None or b > cur_e:
            if cur_e is not None:
                total += cur_e - cur_b
            cur_b, cur_e = b, e
        else:
            cur_e = max(cur_e, e)
    if cur_e is not None:
        total += cur_e - cur_b
    return total


def timed_repeats(run, first, count, repeats, barrier, max_over_ranks, sum_over_ranks):
    """`repeats` timed regions of `count` batches each, CUDA events around each,
    barrier + synchronize on both sides, max over ranks.  Returns per-repeat
    (ms, edges, nodes) with edges / nodes summed over the ranks."""
    import torch

    out = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        got = run(first, count)
        e1.record()
        barrier()
        ms = max_over_ranks(e0.elapsed_time(e1))
        edges, nodes = got if isinstance(got, tuple) else (got, 0)
        out.append((ms, sum_over_ranks(edges), sum_over_ranks(nodes)))
    return out


def median_run(runs):
    """The repeat with the median throughput, and the spread."""
    vals = sorted((e / (ms * 1e-3), ms, e, n) for (ms, e, n) in runs)
    mid = vals[len(vals) // 2]
    return {"value": mid[0], "ms": mid[1], "edges": mid[2], "nodes": mid[3],
            "min": vals[0][0], "max": vals[-1][0], "n": len(vals)}


def run_peer_probe(args, w):
    """The gather kernel alone over a sharded store, rows fetched from the peers only:
    GB/s of stored bytes arriving per GPU, all ranks gathering at once, for several
    request sizes and both request orders.  `AG_FEATURE_ALLOC=cudamalloc` in the
    environment makes the shards plain device allocations mapped through legacy CUDA IPC
    handles, the default shareable blocks mapped with 2 MB pages."""
    import torch
    import torch.distributed as dist

    from aethergraph_b200 import dist as agd
    from aethergraph_b200 import synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world < 2:
        raise SystemExit("--peer-probe needs 2 or more GPUs (one process per GPU)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    n, dim, dtype = w["nodes"], w["dim"], w["dtype"]
    stored_row = dim * (4 if dtype == "f32" else 2)
    shard = synth.features_shard(n, dim, dtype, FEATURE_SEED, rank, world, "cyclic")
    view = agd.open_sharded_features(shard)
    gen = torch.Generator(device=dev)
    gen.manual_seed(1000 + rank)
    rows_out = []
    for order in ("direct", "ordered"):
        view.set_gather_order(order)
        for rows in (100_000, 400_000, 1_600_000, 3_200_000):
            base = torch.randint(0, n // world - 1, (rows,), device=dev, generator=gen, dtype=torch.int64)
            off = torch.randint(1, world, (rows,), device=dev, generator=gen)
            ids = base * world + (rank + off) % world      # rows of the peers only, uniform over them
            out = torch.empty((rows, dim), dtype=torch.float32, device=dev)
            for _ in range(2):
                view.gather(ids, out=out)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 5
            e0.record()
            for _ in range(reps):
                view.gather(ids, out=out)
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / reps], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            rows_out.append({"order": order, "rows": rows, "ms": ms, "peer_gbs_per_gpu": rows * stored_row / ms / 1e6})
            del ids, out, base, off
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 0:
        print(json.dumps({"probe": "rows gathered from the peers' shards only, all ranks at once (max over ranks)",
                          "n_gpus": world, "peer_memory_gb": n * stored_row * (world - 1) / world / 1e9,
                          "row_bytes": stored_row, "mapping": os.environ.get("AG_FEATURE_ALLOC", "shareable blocks, 2 MB pages"),
                          "results": rows_out}), flush=True)
    del view
    dist.barrier()
    del shard
    dist.destroy_process_group()


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
    sharded_only = bool(w.get("sharded_only"))
    if sharded_only and world < 2:
        raise SystemExit(f"workload {args.workload} shards its feature rows over the GPUs: run it with --gpus 2, 4 or 8")
    main_layout = args.features
    if sharded_only and main_layout == "replicated":
        main_layout = "sharded"

    def memlog(where: str):
        """AG_BENCH_MEMLOG=1: free device memory at the stages of the run, on stderr."""
        if os.environ.get("AG_BENCH_MEMLOG") == "1":
            free, total = torch.cuda.mem_get_info(dev)
            print(f"[rank {rank}] {where}: {free / 1e9:.1f} GB free of {total / 1e9:.1f}, torch holds "
                  f"{torch.cuda.memory_reserved(dev) / 1e9:.1f} GB", file=sys.stderr, flush=True)

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

    def open_shards(layout_flag: str):
        """1 / world of the rows on every rank; remote rows cross NVLink inside the gather."""
        from aethergraph_b200 import dist as agd

        layout = "range" if layout_flag == "sharded-range" else "cyclic"
        if world == 1:
            # one GPU: eight shards that all live here — the sharded code path (keys, sort,
            # address-ordered fetch) without a link, for profiling the kernels under ncu
            parts = [synth.features_shard(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED, r, 8, layout) for r in range(8)]
            return ag.FeatureStore.view_sharded(parts, 0)
        shard = synth.features_shard(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED, rank, world, layout)
        return agd.open_sharded_features(shard)

    def sharded_leg(view, layout_flag: str, replicated, cache_gb: float, repeats: int, order: str = "auto"):
        """One resident leg over the sharded view, with `cache_gb` GiB of hot rows copied to
        every GPU first (0: none) and the given gather order.  Returns the record."""
        cached_rows = view.cache_hot_rows(g, int(cache_gb * (1 << 30))) if cache_gb > 0 else view.cache_hot_rows(g, 0)
        view.set_gather_order(order)
        barrier()
        lg = ResidentLeg(L, _lib, g, view, ccfg, dev, w, threads_sh, group_sh, depth_sh, seeds_dev, gidx, rank, world)
        lg.run(0, first_timed)
        barrier()
        st0 = view.gather_stats()
        runs_s = timed_repeats(lg.run, first_timed, n_timed, repeats, barrier, max_over_ranks, sum_over_ranks)
        st1 = view.gather_stats()
        rec = sharded_summary(w, world, median_run(runs_s), stored_row, lg, view, replicated, dev, sum_over_ranks,
                              layout_flag, args.steps, [a - b for a, b in zip(st1, st0)], sum(r[0] for r in runs_s))
        rec["gather_order"] = order if order != "auto" else "direct (auto: every peer is mapped with large pages)"
        rec["hot_rows_copied_per_gpu"] = int(cached_rows)
        rec["hot_rows_gib_per_gpu"] = cached_rows * stored_row / float(1 << 30)
        rec["impl_config"] = {"sampler_threads": threads_sh, "group": group_sh, "prefetch_depth": depth_sh}
        lg.close()
        view.set_gather_order(args.gather_order)
        barrier()
        return rec

    def sharded_record(view, layout_flag: str, replicated):
        """The sharded leg as configured, and beside it the same leg without the hot-row copy
        and with the address-ordered gather (one timed region each)."""
        keys = ("value", "ms_per_step", "remote_gbs_per_gpu", "frac_of_peer_copy_peak", "rows_loaded_per_row_requested",
                "rows_from_hot_copy_per_row_loaded", "parity")
        rec = sharded_leg(view, layout_flag, replicated, args.hot_cache_gb, max(1, min(args.repeats, 3)), args.gather_order)
        if args.hot_cache_gb > 0:
            nc = sharded_leg(view, layout_flag, replicated, 0.0, 1, args.gather_order)
            rec["without_hot_rows"] = {k: nc[k] for k in keys}
        other = "ordered" if args.gather_order != "ordered" else "direct"
        oc = sharded_leg(view, layout_flag, replicated, args.hot_cache_gb, 1, other)
        rec["address_ordered" if other == "ordered" else "direct"] = {k: oc[k] for k in keys}
        if args.hot_cache_gb > 0:
            view.cache_hot_rows(g, int(args.hot_cache_gb * (1 << 30)))
        return rec

    def features_label(layout_flag: str) -> str:
        if layout_flag == "replicated" or world == 1:
            return "replicated"
        how = "contiguous vertex ranges" if layout_flag == "sharded-range" else "rows dealt round-robin by vertex id"
        return f"sharded over the GPUs ({how}), {world - 1}/{world} of the rows fetched over NVLink"

    # ---- inputs, resident in HBM (CSR replicated per GPU) -------------------
    t_setup = time.time()
    g = synth.rmat_graph(w["nodes"], w["edges"], GRAPH_SEED, weight_sigma=1.0 if w["weighted"] else 0.0)
    feats = open_shards(main_layout) if main_layout != "replicated" else \
        synth.features(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED)
    if main_layout != "replicated":
        feats.set_gather_order(args.gather_order)
        if args.hot_cache_gb > 0:
            feats.cache_hot_rows(g, int(args.hot_cache_gb * (1 << 30)))
    torch.cuda.synchronize()
    memlog("after set-up")
    t_setup = time.time() - t_setup
    cfg = ag.SamplingConfig(num_neighbors=w["fanout"], seed=SAMPLER_SEED, weighted=w["weighted"])
    per_step, bs = per_step_of(w), w["batch"]
    n_batches = (args.warmup + args.steps) * per_step
    # rank r handles global batches r, r + world, ... (weak scaling: every rank does K steps)
    gidx = [rank + world * i for i in range(n_batches)]
    seeds_host = [synth.seed_batch(w["nodes"], bs, SEEDS_SEED, b) for b in gidx]
    seeds_dev = torch.from_numpy(np.concatenate(seeds_host).view(np.int32)).to(dev)

    # two workers x chains of 64: the same resident value as three x 32 and a better e2e, because
    # one more host thread per rank is left to the consumer (measured at one and at eight GPUs)
    threads = args.threads or int(w.get("threads", 2))
    group = args.group or int(w.get("group", 64))
    depth = args.depth or int(w.get("depth", max(8, group // 2)))
    # sharded legs: remote rows have a longer way, so more chains are kept in flight
    threads_sh = args.threads or int(w.get("threads_sharded", w.get("threads", 4)))
    group_sh = args.group or int(w.get("group_sharded", w.get("group", 64)))
    depth_sh = args.depth or int(w.get("depth", max(8, group_sh // 2)))
    ccfg = cfg._to_c(SAMPLER_SEED, bs)
    row_bytes = gather_bytes_per_row(w)
    stored_row = sector(w["dim"] * (4 if w["dtype"] == "f32" else 2))
    peak, peak_src = peaks()
    first_timed, n_timed = args.warmup * per_step, args.steps * per_step
    hops = len(w["fanout"])

    # ---- value: C ABI, inputs resident, recycled output buffers ------------
    leg = ResidentLeg(L, _lib, g, feats, ccfg, dev, w, threads, group, depth, seeds_dev, gidx, rank, world)
    leg.run(0, first_timed)
    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    stats0 = leg.stats()
    leg.intervals = set()
    wall0 = time.time()
    runs = timed_repeats(leg.run, first_timed, n_timed, args.repeats, barrier, max_over_ranks, sum_over_ranks)
    wall1 = time.time()
    stats1 = leg.stats()
    clk = clocks.stop(wall0, wall1)
    med = median_run(runs)
    value, ms = med["value"], med["ms"]
    gather_gbs = med["nodes"] * row_bytes / (ms * 1e-3) / 1e9
    g_ms = stats1.gather_ms - stats0.gather_ms
    s_ms = stats1.sample_ms - stats0.sample_ms
    own_nodes = int(stats1.nodes - stats0.nodes)   # this rank, all repeats
    # Every sampler thread's chain has its own gather stream, so gather launches of
    # different chains overlap one another: the time the kernel was running is the union
    # of the launches' device intervals, not the sum of their durations.
    busy_ms = union_ms(leg.intervals)
    raw = own_nodes * row_bytes / (g_ms * 1e-3) / 1e9 if g_ms > 0 else None
    achieved = own_nodes * row_bytes / (busy_ms * 1e-3) / 1e9 if busy_ms > 0 else raw
    # one gather launch per chain (a chain covers up to `group` batches, the batch is blockIdx.y)
    launches = max(int(stats1.chains - stats0.chains), 1)
    per_row = NCU_DRAM_BYTES_PER_ROW.get(w["dtype"] + str(w["dim"]))
    pipeline_bytes = med["nodes"] * row_bytes + sampling_bytes(med["edges"], med["nodes"], med["nodes"])
    total_ms = sum(r[0] for r in runs)
    roofline = {
        "kernel": "k_gather_vec (feature-row gather + upcast)" if main_layout == "replicated" else
                  "k_gather_peer (feature-row gather over the shards + upcast)", "bound": "hbm",
        "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": (achieved / peak) if achieved else None, "peak_source": peak_src,
        "frac_of_nominal_8tbs": (achieved / 8000.0) if achieved else None,
        "bytes_per_launch": own_nodes * row_bytes / launches,
        "ms_per_launch": (busy_ms if busy_ms > 0 else g_ms) / launches,
        "launches": launches, "traffic": (per_row * own_nodes / launches) if per_row else None,
        "traffic_note": "extrapolated: ncu dram bytes per gathered row on the C2-small capture x rows per launch",
        "note": "CUDA events around every gather launch on its launching stream, over the timed regions, while "
                "the sampling kernels of the other chains run beside it.  Launches of different chains overlap "
                "one another, so the duration is the union of their device intervals / launches; "
                "`events_per_launch` is the plain mean of the launch durations, `alone` the same kernel by itself",
        "gather_running_share_of_timed_region": (busy_ms / total_ms) if total_ms else None,
        "events_per_launch": {"achieved": raw, "frac": (raw / peak) if raw else None, "ms_per_launch": g_ms / launches},
        "step": {"gather_gbs": gather_gbs, "frac_of_peak": gather_gbs / (peak * world),
                 "note": "gather bytes of a step / step time: the whole pipeline as seen from the gather's roofline"},
        "pipeline": {"algorithmic_gbs": pipeline_bytes / (ms * 1e-3) / 1e9,
                     "frac_of_peak": pipeline_bytes / (ms * 1e-3) / 1e9 / (peak * world),
                     "sample_ms_per_batch": s_ms / max(n_timed * args.repeats, 1)},
    }
    # The same kernel on its own: the node ids of the last delivered batches, gathered
    # by one standalone launch per repetition with nothing else on the GPU (the
    # in-pipeline figure above shares the SMs and HBM with the other workers'
    # sampling kernels).
    if leg.recent and not (args.only_value or args.brief):
        holder = _Buffers(leg.ring[0].c, leg.ring, dev, w["dim"])  # the ring keeps the memory alive
        ids = torch.cat([holder.view(ptr, (int(n),), "<i8") for ptr, _, n in leg.recent])
        x_alone = torch.empty((ids.shape[0], w["dim"]), dtype=torch.float32, device=dev)
        for _ in range(3):
            feats.gather(ids, out=x_alone)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
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
        del ids, x_alone, holder
        barrier()
    leg.close()
    del leg
    memlog("after the resident leg")
    sharded_main = None
    if main_layout != "replicated" and world > 1:
        sharded_main = sharded_record(feats, main_layout, None)
        barrier()
        memlog("after the sharded legs")

    # ---- e2e: public Python API, host seeds in, counts back -----------------
    e2e_med = host_med = None
    d2h_host = host_batches = 0
    host_sample = ""
    window = min(8 * depth, depth + threads * group + group)
    if not (args.only_value or args.brief):
        loader = NeighborLoader(g, cfg, prefetch_depth=depth, sampler_threads=threads, features=feats, group=group,
                                seed_sequence=(rank, world))
        pinned = None
        mn, me = C.c_uint64(), C.c_uint64()
        _lib.check(L.ag_loader_bounds(loader._h, bs, C.byref(mn), C.byref(me)))

        def run_e2e(first: int, count: int, to_host: bool = False):
            """Host seed arrays in through the public API (submitted a chain at a time);
            `to_host` also copies every batch (ids, local edge index, feature rows) into
            pinned host memory."""
            nonlocal d2h_host
            edges = nodes = submitted = delivered = 0
            while delivered < count:
                while submitted < count and submitted - delivered + min(group, count - submitted) <= window:
                    n = min(group, count - submitted)
                    b0 = (first + submitted) % n_batches
                    lo = [(b0 + j) % n_batches for j in range(n)]
                    loader.submit_epoch([seeds_host[b] for b in lo], [gidx[b] for b in lo])
                    submitted += n
                _, sg, x = loader.next_batch()
                if to_host:
                    nn, ne = sg.num_nodes, sg.num_edges
                    pinned["n_id"][:nn].copy_(sg.nodes_t, non_blocking=True)
                    pinned["ei"][:, :ne].copy_(sg.edge_index_local_t, non_blocking=True)
                    pinned["x"][:nn].copy_(x, non_blocking=True)
                    torch.cuda.current_stream().synchronize()
                    d2h_host += nn * 8 + ne * 16 + nn * w["dim"] * 4
                edges += sg.num_edges
                nodes += sg.num_nodes
                delivered += 1
            return edges, nodes

        # warm-up long enough for the loader's buffer pool to reach its working size
        run_e2e(0, max(first_timed, 2 * window))
        run_e2e(first_timed, n_timed)   # one untimed pass over the timed batches: their buffers reach their sizes
        e2e_runs = timed_repeats(run_e2e, first_timed, n_timed, args.repeats, barrier, max_over_ranks, sum_over_ranks)
        e2e_med = median_run(e2e_runs)
        # the same with every batch also copied to pinned host memory (what a host-side
        # consumer sees): PCIe-bound, so a bounded sample of the step is enough
        host_batches = min(n_timed, 2 * per_step, 1024)
        pinned = {"n_id": torch.empty(mn.value, dtype=torch.int64).pin_memory(),
                  "ei": torch.empty((2, me.value), dtype=torch.int64).pin_memory(),
                  "x": torch.empty((mn.value, w["dim"]), dtype=torch.float32).pin_memory()}
        run_e2e(0, min(64, host_batches), True)
        d2h_host = 0
        host_runs = timed_repeats(lambda f, c: run_e2e(f, c, True), first_timed, host_batches, 1, barrier,
                                  max_over_ranks, sum_over_ranks)
        host_med = median_run(host_runs)
        host_sample = f"{host_batches} batches"
        loader.shutdown()
        del loader, pinned

    # ---- CPU baseline beside it (rank 0, one GPU only) ----------------------
    cpu = None
    parity = None
    if rank == 0 and world == 1 and not args.no_cpu and not args.only_value:
        cpu, parity = cpu_baseline(g, feats, w, cfg, seconds=args.cpu_seconds, ref_kernel=not args.brief)

    # ---- sharded features (2 or more GPUs): 1/N of the rows per GPU ----------
    sharded = sharded_main
    if world > 1 and main_layout == "replicated" and not args.only_value and not args.no_sharded:
        view = open_shards("sharded")
        sharded = sharded_record(view, "sharded", feats)
        sharded["vs_replicated"] = sharded["value"] / value if value else None
        barrier()  # no rank frees its shard while a peer may still be reading it
        del view
        barrier()

    # ---- the same leg over the block-scaled int8 payload (1 GPU) -------------------
    int8_leg = None
    if world == 1 and not args.only_value and not args.brief and not args.no_secondary and w["dim"] % 16 == 0 \
            and main_layout == "replicated":
        f8 = synth.features(w["nodes"], w["dim"], "i8", FEATURE_SEED)
        leg8 = ResidentLeg(L, _lib, g, f8, ccfg, dev, w, threads, group, depth, seeds_dev, gidx, rank, world)
        leg8.run(0, first_timed)
        med8 = median_run(timed_repeats(leg8.run, first_timed, n_timed, max(1, min(args.repeats, 3)), barrier,
                                        max_over_ranks, sum_over_ranks))
        rb8 = sector(w["dim"] + 4 * ((w["dim"] + 31) // 32)) + w["dim"] * 4
        # rows of the last batch against the codec's own decode of the same stored bytes
        ok8 = None
        if leg8.recent:
            holder = _Buffers(leg8.ring[0].c, leg8.ring, dev, w["dim"])
            n_id_ptr, x_ptr, nn = leg8.recent[-1]
            ids8 = holder.view(n_id_ptr, (int(nn),), "<i8")[:4096]
            x8 = holder.view(x_ptr, (int(nn), w["dim"]), "<f4")[:4096]
            ok8 = bool(torch.equal(x8.view(torch.int32), f8.gather(ids8).view(torch.int32)))
            del holder
        int8_leg = {"value": med8["value"], "unit": "edges/s", "ms_per_step": med8["ms"] / max(args.steps, 1),
                    "gather_gbs": med8["nodes"] * rb8 / (med8["ms"] * 1e-3) / 1e9, "bytes_per_row": rb8,
                    "rows_match_standalone_gather": ok8,
                    "note": "features stored as block-scaled int8 (one byte per element + one f32 scale per 32 "
                            "elements of a row, the reference's BlockScaledI8): lossy, the gathered rows are what its "
                            "decode gives; 288 B read + 1024 B written per row instead of 512 + 1024"}
        leg8.close()
        del leg8, f8

    secondary = None
    if rank == 0 and world == 1 and not args.only_value and not args.brief and not args.no_secondary \
            and args.workload == "c2":
        del g, feats
        torch.cuda.empty_cache()
        g = feats = None
        secondary = secondary_legs(args)

    if rank == 0:
        chains = -(-n_timed // group)
        line = {
            "metric": METRIC, "value": value, "unit": "edges/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / max(args.steps, 1), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u32 ids / " + w["dtype"] + "->f32",
            "data": "synthetic (seeded R-MAT graph + ~N(0,1) features generated in HBM)",
            "config": common_config(w, world, features_label(main_layout)),
            "impl_config": {"sampler_threads": threads, "group": group, "prefetch_depth": depth,
                            "implementation": "libaethergpu.so (CUDA, sm_100a) through the C ABI"},
            "repeats": {"n": med["n"], "min": med["min"], "max": med["max"],
                        "note": f"value = median of {med['n']} timed regions of {args.steps} steps each"},
            "gather_gbs": gather_gbs, "edges_per_step": med["edges"] / max(args.steps, 1),
            "rows_per_step": med["nodes"] / max(args.steps, 1), "setup_s": round(t_setup, 1),
            "timed_region_s": round(ms * 1e-3, 4),
            "clocks": clk, "roofline": roofline, "cpu_baseline": cpu, "parity_full_scale": parity,
            "e2e": None if e2e_med is None else {
                "value": e2e_med["value"], "unit": "edges/s", "h2d_bytes_per_step": world * per_step * bs * 4,
                "d2h_bytes_per_step": world * per_step * C.sizeof(_lib.SampleCounts),
                "ms_per_step": e2e_med["ms"] / max(args.steps, 1), "min": e2e_med["min"], "max": e2e_med["max"],
                "repeats": e2e_med["n"],
                "note": "public Python API: host seed arrays in (submit_epoch, a chain at a time), per-batch "
                        "counts out; the sampled batch and its feature rows stay in GPU memory, where the "
                        "training step reads them",
                "host_results": {"value": host_med["value"], "unit": "edges/s", "sample": host_sample,
                                 "d2h_bytes_per_batch": d2h_host / max(1, host_batches),
                                 "note": "same calls, every batch (int64 ids, local edge index, f32 feature rows) "
                                         "also copied to pinned host memory: PCIe-bound"}},
            "sharded": sharded, "int8_payload": int8_leg, "secondary": secondary,
            # one launch chain per group of batches (the batch is blockIdx.y): seed insert,
            # hops + 1 assign, hops pick, gather (sharded: + key, sorted gather, overflow)
            "gpu_launches": world * chains * (2 * hops + 3 + (3 if sharded_main else 0)),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        barrier()  # no rank frees its feature shard while a peer may still be reading it
        del feats
        barrier()
        dist.destroy_process_group()


def sharded_summary(w, world, med, stored_row, leg, view, replicated, dev, sum_over_ranks, layout_flag, steps,
                    stats_delta, total_ms):
    """The record of a leg over sharded features: throughput, the remote share of the
    stored rows as GB/s per GPU against the measured peer-copy bandwidth, and a bit
    for bit check of the last delivered batch's rows (most of them remote) against the
    replicated table (or, without one, rows regenerated from the counter-based generator)."""
    import torch

    from aethergraph_b200 import synth
    from aethergraph_b200.sampler import _Buffers

    ms = med["ms"]
    remote_share = (world - 1) / world
    asked, loaded, from_copy = stats_delta   # this rank, all timed repeats
    # rows that really crossed NVLink: loaded once per chain, not served by the local copy of the
    # hot rows, and (round-robin or range shards alike) owned by a peer with probability (W - 1) / W
    remote_gbs = (loaded - from_copy) * remote_share * stored_row / (total_ms * 1e-3) / 1e9 if total_ms else 0.0
    ok, checked = True, 0
    if leg.recent:
        holder = _Buffers(leg.ring[0].c, leg.ring, dev, w["dim"])
        n_id_ptr, x_ptr, n = leg.recent[-1]
        n = int(n)
        ids = holder.view(n_id_ptr, (n,), "<i8")
        x = holder.view(x_ptr, (n, w["dim"]), "<f4")
        if replicated is not None:
            want = replicated.gather(ids)
            ok = bool(torch.equal(x.view(torch.int32), want.view(torch.int32)))
            checked = n
        else:
            # regenerate some of the rows from (seed, row, column): contiguous runs of the table
            pick = ids[:: max(1, n // 64)][:64].tolist()
            for v in pick:
                one = synth.features(w["nodes"], w["dim"], w["dtype"], FEATURE_SEED, row_range=(v, v + 1))
                want = one.gather(torch.tensor([v], dtype=torch.int64, device=dev))
                pos = int((ids == v).nonzero()[0])
                ok = ok and bool(torch.equal(x[pos].view(torch.int32), want[0].view(torch.int32)))
                checked += 1
        del holder
    ok_all = sum_over_ranks(1.0 if ok else 0.0) == float(world)
    return {"layout": "contiguous vertex ranges" if layout_flag == "sharded-range" else "round-robin by vertex id",
            "value": med["value"], "unit": "edges/s", "ms_per_step": ms / max(steps, 1),
            "min": med["min"], "max": med["max"],
            "gather_gbs": med["nodes"] * gather_bytes_per_row(w) / (ms * 1e-3) / 1e9,
            "remote_gbs_per_gpu": remote_gbs, "frac_of_peer_copy_peak": remote_gbs / NVLINK_PEER_COPY_GBS,
            "peer_copy_peak_gbs": NVLINK_PEER_COPY_GBS,
            "remote_note": "stored bytes of the rows rank 0 fetched from its peers per second: rows loaded (every "
                           "requested row in direct order, once per launch chain in address order) less the ones "
                           "served by the local copy of the hot rows, times (W - 1) / W",
            "rows_loaded_per_row_requested": (loaded / asked) if asked else None,
            "rows_from_hot_copy_per_row_loaded": (from_copy / loaded) if loaded else None,
            "parity": bool(ok_all), "parity_rows_checked_per_rank": checked}


def secondary_legs(args) -> dict:
    """C1, C3 and C4 at 1/10 size, each in its own process after the main workload
    has left the GPU: value, CPU baseline and full-size parity of each."""
    out = {}
    for name, steps in (("c1", 4), ("c3", 2), ("c4s", 2)):
        cmd = [sys.executable, os.path.abspath(__file__), "--workload", name, "--steps", str(steps), "--warmup", "3",
               "--repeats", "3", "--brief", "--cpu-seconds", "4"]
        try:
            r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
            line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
            out[name] = {k: line.get(k) for k in ("value", "unit", "ms_per_step", "gather_gbs", "cpu_baseline",
                                                  "parity_full_scale", "repeats", "steps")}
            out[name]["workload"] = line["config"]["workload"]
        except Exception as e:  # a failed secondary leg must not lose the main line
            out[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
    return out


# --------------------------------------------------------------------------- #
#  heterogeneous workload (C4): secondary, `--workload c4` / `c4s`               #
# --------------------------------------------------------------------------- #
HETERO = {
    # user / post / comment / subreddit; three stored relations plus their reverses (user seeds
    # need incoming edge types); fanouts votes [15,10], writes [10,5], belongs_to [3,2]
    "c4": dict(scale=1, label="C4: user 50M / post 20M / comment 100M / subreddit 100K, 6 edge types, batch 1024"),
    "c4s": dict(scale=10, label="C4 at 1/10 scale: user 5M / post 2M / comment 10M / subreddit 10K, 6 edge types, batch 1024"),
}


def hetero_cpu_leg(g, nn, ets, fan, host_rel, seeds, stores, seconds=6.0):
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
    while time.time() - t_cpu < seconds and nb_cpu < len(seeds):
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
    bs, per_step = 1024, int(hw.get("per_step", 128))
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
    runs = []
    for _ in range(max(1, args.repeats)):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        edges, gbytes = run(args.warmup * per_step, args.steps * per_step)
        e1.record()
        torch.cuda.synchronize()
        runs.append((e0.elapsed_time(e1), edges, gbytes))
    med = median_run(runs)
    ms, edges, gbytes = med["ms"], med["edges"], med["nodes"]
    loader.shutdown()
    cpu, ok = None, None
    if not args.no_cpu and sc > 1:
        cpu, ok = hetero_cpu_leg(g, nn, ets, fan, host_rel, seeds, stores, min(6.0, args.cpu_seconds))
    line = {
        "metric": METRIC, "value": edges / (ms * 1e-3), "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / max(args.steps, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u32 ids / bf16->f32", "data": "synthetic (per-relation R-MAT generated in HBM)",
        "config": {"workload": hw["label"], "batches_per_step": per_step,
                   "fanout": {"/".join(et): f for et, f in zip(ets, fan)}},
        "impl_config": {"sampler_threads": args.threads, "group": group},
        "repeats": {"n": med["n"], "min": med["min"], "max": med["max"]},
        "gather_gbs": gbytes / (ms * 1e-3) / 1e9, "edges_per_step": edges / max(args.steps, 1), "setup_s": round(t_setup, 1),
        "cpu_baseline": cpu, "parity_full_scale": ok,
    }
    print(json.dumps(line), flush=True)


def cpu_baseline(g, feats, w, cfg, seconds: float = 10.0, ref_kernel: bool = True):
    """Times the CPU restatement on a bounded sample of the same workload (graph and
    features copied back from the GPU; about `seconds` of CPU work) and checks two
    full-size batches bit for bit."""
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
    # (weighted picks draw a key per neighbour of every frontier row: start small)
    seeds_host = [synth.seed_batch(w["nodes"], bs, SEEDS_SEED, b) for b in range(threads if w["weighted"] else 4 * threads)]
    nb, cap = len(seeds_host), 1 << 16
    while True:
        seeds = np.concatenate(seeds_host[:nb])
        r = s.bench(payload, w["dim"], w["dtype"], seeds, bs, 0, threads)
        if r["seconds"] >= 0.8 * seconds or nb >= cap:
            break
        nb = min(cap, max(nb + 1, int(nb * min(16.0, 1.2 * seconds / max(r["seconds"], 1e-3)))))
        seeds_host += [synth.seed_batch(w["nodes"], bs, SEEDS_SEED, b) for b in range(len(seeds_host), nb)]
    # one thread, one persistent sampler reused across batches (the reference's NeighborSampler reuse)
    n1 = max(2, min(nb, int(0.4 * seconds * nb / max(r["seconds"], 1e-3) / threads)))
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
    if ref_kernel:
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
                    help="loader worker threads, each with its own CUDA stream (0: the workload's, normally 3; "
                         "heterogeneous workloads 2)")
    ap.add_argument("--depth", type=int, default=0, help="prefetch depth (0: max(8, group / 2))")
    ap.add_argument("--group", type=int, default=int(os.environ.get("AG_BENCH_GROUP", "0")),
                    help="batches a worker runs as one launch chain (0: the workload's, normally 32)")
    ap.add_argument("--features", default="replicated", choices=["replicated", "sharded", "sharded-range"],
                    help="with more than one GPU: every GPU holds all feature rows, or 1/N of them "
                         "(dealt round-robin, or as contiguous vertex ranges)")
    ap.add_argument("--repeats", type=int, default=5,
                    help="timed regions of --steps steps each; the median is reported, with min and max")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="CPU work of the bounded cpu_baseline sample")
    ap.add_argument("--brief", action="store_true",
                    help="value, cpu_baseline and parity only (what a secondary workload reports)")
    ap.add_argument("--no-sharded", action="store_true", help="2 or more GPUs: skip the sharded-features record")
    ap.add_argument("--hot-cache-gb", type=float, default=1.0,
                    help="sharded features: GiB of the hottest rows (highest in-degree) copied to every GPU (0: none)")
    ap.add_argument("--gather-order", default="auto", choices=["auto", "ordered", "direct"],
                    help="sharded features: how remote rows are requested (auto: direct loads when every peer is "
                         "mapped with large pages)")
    ap.add_argument("--no-secondary", action="store_true", help="1 GPU: skip the secondary workloads (C1, C3, C4 at 1/10)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--peer-probe", action="store_true",
                    help="2 or more GPUs: time the gather kernel alone on rows of the peers' shards")
    ap.add_argument("--only-value", action="store_true",
                    help="run the resident (C ABI) leg only: no e2e, no CPU baseline (profiling runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup
    args.repeats = max(1, args.repeats)
    if args.workload in HETERO:
        if args.threads <= 0:
            args.threads = 2
        return run_hetero(args, HETERO[args.workload])
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w)
    elif args.peer_probe:
        run_peer_probe(args, w)
    else:
        run_device(args, w)


if __name__ == "__main__":
    main()

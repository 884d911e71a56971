"""Prefetching `NeighborLoader` over the native GPU pipeline.

Mirrors `aethergraph._core.NeighborLoader` / `PrefetchStats`
(python/aethergraph/_core.pyi:352-464): `submit(batch_idx, seeds)` queues a
batch, `next_batch()` returns `(batch_idx, subgraph, features)`.  With a config
seed, batches come back in submission order and batch number `seq` is sampled
from `batch_seed(seed, seq)` whatever the number of sampler threads; without a
seed they come back as they finish.  `None` is returned only after `shutdown()`;
a worker failure raises RuntimeError, a 30 s wait TimeoutError.

The batches are born in GPU memory: `subgraph.*_t` and `features` are CUDA
tensors that view one pooled device allocation per batch.  The allocation goes
back to the loader's pool when the last tensor or subgraph object that refers
to it is dropped.  Pass `host_features=True` to get the feature block as a host
numpy array the way the reference returns it.
"""
from __future__ import annotations

import ctypes as C
import os
import secrets
import threading
from typing import Any

import numpy as np

from . import _lib
from .features import FeatureStore
from .graph import CsrGraph
from .sampler import (SampledSubgraph, SamplingConfig, _Buffers, _check_config, apply_subgraph_type,
                      coerce_seeds)

__all__ = ["NeighborLoader", "PrefetchStats"]

_FETCH = 32  # batches taken from the native queue per call


class PrefetchStats:
    """Snapshot of the loader's counters (crates/aethergraph-core/src/loader/prefetch.rs:853-899)."""

    def __init__(self, s: _lib.LoaderStats):
        self.hits, self.misses, self.total = s.hits, s.misses, s.total
        self.sample_time_ns, self.feature_load_time_ns = s.sample_time_ns, s.feature_load_time_ns
        self.submitted, self.edges, self.nodes = s.submitted, s.edges, s.nodes
        self.gather_ms, self.sample_ms = s.gather_ms, s.sample_ms

    @property
    def hit_rate(self) -> float:
        return 1.0 if self.total == 0 else self.hits / self.total

    def to_dict(self) -> dict[str, Any]:
        return {"hits": self.hits, "misses": self.misses, "total": self.total, "hit_rate": self.hit_rate,
                "sample_time_ns": self.sample_time_ns, "feature_load_time_ns": self.feature_load_time_ns}


class _Lease:
    """Holds one pooled batch; gives it back to the loader when nothing refers to it
    any more, or when `release()` is called.  The release records a stream — the one
    given to `record_stream` / `release`, else torch's current stream at that moment —
    so kernels already queued on it finish before the memory is written again."""

    __slots__ = ("loader", "batch", "stream", "released")

    def __init__(self, loader: "NeighborLoader", batch: _lib.Batch):
        self.loader, self.batch, self.stream, self.released = loader, batch, None, False

    def release(self, stream=None) -> None:
        if self.released:
            return
        ld = self.loader
        if ld is None or not ld._h:
            return
        st = stream if stream is not None else self.stream
        raw = _raw_stream(st) if st is not None else _raw_current_stream(ld._dev_index)
        self.released = True
        ld._release(ld._h, C.byref(self.batch), raw)

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


def _raw_stream(stream) -> int:
    """cudaStream_t of a torch.cuda.Stream, or the integer itself."""
    return int(getattr(stream, "cuda_stream", stream))


def _raw_current_stream(device_index: int) -> int:
    """cudaStream_t of torch's current stream on the device (the cheap accessor; the
    Stream object `torch.cuda.current_stream` builds costs several microseconds)."""
    import torch

    try:
        return torch._C._cuda_getCurrentRawStream(device_index)
    except AttributeError:
        return torch.cuda.current_stream(device_index).cuda_stream


class NeighborLoader:
    def __init__(self, graph: CsrGraph, config: SamplingConfig, prefetch_depth: int = 2,
                 sampler_threads: int = 1, *, features: FeatureStore | None = None,
                 host_features: bool = False, profiling: bool = False, group: int = 8,
                 seed_sequence: tuple[int, int] = (0, 1)):
        """`seed_sequence=(base, stride)`: the loader's batch number `seq` is sampled
        from `batch_seed(seed, base + stride * seq)`.  Rank r of a W-rank job that takes
        global batches r, r + W, ... passes `(r, W)`, so every global batch is drawn from
        the same stream whatever W is."""
        import torch

        composed = config.disjoint or config.cumulative
        _check_config(graph, config, pipelined=not composed)
        if prefetch_depth < 1:
            raise ValueError("prefetch_depth must be >= 1")
        if sampler_threads < 1:
            raise ValueError("sampler_threads must be >= 1")
        self.graph, self.config, self.features = graph, config, features
        self._depth, self._host_features = prefetch_depth, host_features
        self._seeded = config.seed is not None
        seed = config.seed if self._seeded else secrets.randbits(64)
        self._composed = None
        if composed:
            # Disjoint and cumulative batches are compositions of the plain sampler's launch
            # chains (one per seed / per hop): they are sampled when they are asked for, in
            # submission order, batch `seq` from batch_seed(seed, base + stride * seq) like
            # every other batch.  Same interface, no prefetch.
            from .sampler import NeighborSampler

            self._composed = NeighborSampler(graph, config, features=features)
            self._composed_seed, self._seed_seq = seed, tuple(int(v) for v in seed_sequence)
            self._h = None
            self._dim = features.feature_dim if features is not None else None
            self._pending: list = []
            self._next_seq = self._served = 0
            self._closed = False
            return
        cfg = config._to_c(seed)
        self._h = C.c_void_p()
        _lib.check(_lib.lib().ag_loader_create(graph._h, features._h if features is not None else None,
                                               C.byref(cfg), int(self._seeded), prefetch_depth, sampler_threads,
                                               max(1, int(group)), int(profiling), C.byref(self._h)))
        if tuple(seed_sequence) != (0, 1):
            _lib.check(_lib.lib().ag_loader_set_seed_sequence(self._h, int(seed_sequence[0]), int(seed_sequence[1])))
        self._dev = torch.device("cuda", graph.device)
        self._dev_index = int(graph.device)
        self._release = _lib.lib().ag_loader_release_batch
        self._dim = features.feature_dim if features is not None else None
        self._lock = threading.Lock()
        self._next_seq = 0
        self._next_deliver = 0            # seeded loaders deliver in seq order
        self._seeds: dict[int, np.ndarray] = {}
        self._fetched: list = []          # batches already taken from the native queue
        self._fetch_buf = (_lib.Batch * _FETCH)()
        self._closed = False

    @staticmethod
    def with_features(graph: CsrGraph, config: SamplingConfig, feature_path, prefetch_depth: int = 2,
                      sampler_threads: int = 1, **kw) -> "NeighborLoader":
        store = FeatureStore.load(os.fspath(feature_path), device=graph.device)
        if store.num_nodes < graph.num_nodes:
            raise ValueError(f"feature file has {store.num_nodes} rows but the graph has {graph.num_nodes} nodes")
        return NeighborLoader(graph, config, prefetch_depth, sampler_threads, features=store, **kw)

    # -- properties --------------------------------------------------------
    @property
    def feature_dim(self) -> int | None:
        return self._dim

    @property
    def has_features(self) -> bool:
        return self.features is not None

    @property
    def num_nodes(self) -> int:
        return self.graph.num_nodes

    @property
    def prefetch_depth(self) -> int:
        return self._depth

    # -- producer side -----------------------------------------------------
    def submit(self, batch_idx: int, seeds) -> None:
        """Queue a batch.  `batch_idx` is echoed back by `next_batch()`; any value is accepted."""
        s = coerce_seeds(seeds, self.graph.num_nodes)
        if self._composed is not None:
            if self._closed:
                raise RuntimeError("loader is shut down")
            self._pending.append((int(batch_idx), self._next_seq, s))
            self._next_seq += 1
            return
        with self._lock:
            # The C call blocks while the work queue is full; the lock keeps the
            # Python-side sequence counter in step with the library's.
            seq = self._next_seq
            self._seeds[seq] = s  # in place before a worker can finish the batch
            rc = _lib.lib().ag_loader_submit(self._h, int(batch_idx), s.ctypes.data if len(s) else None,
                                             len(s), _lib.AG_MEM_HOST, None, None)
            if rc != _lib.AG_OK:
                del self._seeds[seq]
                _lib.check(rc)
            self._next_seq += 1

    def submit_epoch(self, batches, batch_indices=None) -> None:
        """Queue batches 0 .. len(batches) - 1 (or `batch_indices`) in one native call.
        The call blocks while the work queue (8 x prefetch_depth batches) is full, so a
        thread that also consumes the results submits at most that many at a time."""
        seeds = [coerce_seeds(b, self.graph.num_nodes) for b in batches]
        n = len(seeds)
        if n == 0:
            return
        if self._composed is not None:
            for i, s in enumerate(seeds):
                self.submit(i if batch_indices is None else int(batch_indices[i]), s)
            return
        idx = (C.c_int64 * n)(*(range(n) if batch_indices is None else [int(i) for i in batch_indices]))
        ptrs = (C.c_void_p * n)(*[s.ctypes.data if len(s) else None for s in seeds])
        lens = (C.c_uint64 * n)(*[len(s) for s in seeds])
        done = C.c_uint32()
        with self._lock:
            first = self._next_seq
            for i, s in enumerate(seeds):
                self._seeds[first + i] = s
            rc = _lib.lib().ag_loader_submit_many(self._h, n, idx, ptrs, lens, _lib.AG_MEM_HOST, None, None,
                                                  C.byref(done))
            self._next_seq += done.value
            for i in range(done.value, n):
                del self._seeds[first + i]
            _lib.check(rc)

    # -- consumer side -----------------------------------------------------
    def _take(self, blocking: bool):
        if self._composed is not None:
            if self._closed or not self._pending:
                if self._closed or not blocking:
                    return None
                raise TimeoutError("no batch was submitted")
            idx, seq, seeds = self._pending.pop(0)
            base, stride = self._seed_seq
            if self._seeded:
                self._composed.reseed(_lib.lib().ag_batch_seed(self._composed_seed, base + stride * seq))
            self._served += 1
            return idx, self._composed.sample(seeds)
        if not self._fetched:
            if self._closed:
                return None
            got = C.c_uint32()
            if blocking:
                rc = _lib.lib().ag_loader_next_many(self._h, -1, _FETCH, self._fetch_buf, C.byref(got))
            else:
                rc = _lib.lib().ag_loader_try_next(self._h, self._fetch_buf)
                got.value = 1 if rc == _lib.AG_OK else 0
            if rc == _lib.AG_ERR_SHUTDOWN:
                return None
            if rc == _lib.AG_ERR_TIMEOUT and not blocking:
                return None
            if rc in (_lib.AG_ERR_SAMPLING, _lib.AG_ERR_VALUE, _lib.AG_ERR_LOAD) and self._seeded:
                # a batch that failed by itself was consumed by the library: forget its seeds too
                self._seeds.pop(self._next_deliver, None)
                self._next_deliver += 1
            _lib.check(rc)
            for i in range(got.value - 1, -1, -1):  # reversed: pop() hands them out in order
                b = _lib.Batch.from_buffer_copy(self._fetch_buf[i])
                self._fetched.append(b)
        b = self._fetched.pop()
        self._next_deliver = b.seq + 1
        seeds = self._seeds.pop(b.seq)
        bufs = _Buffers(b.bufs, _Lease(self, b), self._dev, self._dim)
        sg = SampledSubgraph(bufs, b.counts, seeds)
        if self.config.subgraph_type != "directional":
            sg = apply_subgraph_type(self.graph, self.config.subgraph_type, sg)
        return int(b.batch_idx), sg

    def next_batch(self):
        """`(batch_idx, subgraph, features)`, or None after `shutdown()`."""
        got = self._take(True)
        if got is None:
            return None
        idx, sg = got
        x = sg.x
        if x is not None and self._host_features:
            x = x.cpu().numpy()
        return idx, sg, x

    def next(self):
        got = self._take(True)
        return None if got is None else got[1]

    def try_next(self):
        got = self._take(False)
        return None if got is None else got[1]

    def next_with_features(self):
        got = self.next_batch()
        return None if got is None else (got[1], got[2])

    def stats(self) -> PrefetchStats:
        s = _lib.LoaderStats()
        if self._composed is not None:
            s.total = s.misses = self._served       # nothing is sampled ahead of time
            s.submitted = self._next_seq
            return PrefetchStats(s)
        _lib.check(_lib.lib().ag_loader_stats_get(self._h, C.byref(s)))
        return PrefetchStats(s)

    def shutdown(self) -> None:
        if self._composed is not None:
            self._closed = True
            return
        if self._h:
            _lib.lib().ag_loader_shutdown(self._h)
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc) -> None:
        self.shutdown()

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                self._fetched = []
                _lib.lib().ag_loader_free(h)
            except Exception:
                pass
            self._h = None

"""Neighbor sampling on the GPU behind the reference's sampler API.

Mirrors `SamplingConfig`, `NeighborSampler` (alias `Sampler`), `SampledSubgraph`
and `ParallelBatchSampler` of the reference (python/aethergraph/sampler.py,
python/aethergraph/_core.pyi:152-288).  Sampling, dedup, relabel and the int64
widening all run in CUDA kernels; results stay in GPU memory (`*_t` tensor
accessors, `x`) and are copied to host numpy arrays only when the numpy
accessors of the reference API are read.
"""
from __future__ import annotations

import ctypes as C
import secrets
from dataclasses import dataclass
from typing import Any, Sequence

import numpy as np

from . import _lib
from ._lib import SamplingError
from .features import FeatureStore
from .graph import CsrGraph

__all__ = ["NeighborSampler", "ParallelBatchSampler", "SampledSubgraph", "Sampler", "SamplingConfig",
           "SamplingError"]

_SUBGRAPH_TYPES = ("directional", "induced", "bidirectional")
_TEMPORAL = ("uniform", "last")


@dataclass
class SamplingConfig:
    """Configuration for neighborhood sampling (same fields and validation as the
    reference, crates/aethergraph-py/src/sampler.rs:116-194), plus `rng_mode`:

    - ``"wyrand_exact"`` (default) reproduces the reference CPU sampler's output
      bit for bit for a given seed.
    - ``"philox"`` keys every draw on (seed, hop, vertex, slot) with
      Philox4x32-10: the same sampling distribution, different samples.
    """

    num_neighbors: list[int]
    replace: bool = False
    seed: int | None = None
    max_degree: int | None = None
    cumulative: bool = False
    weighted: bool = False
    subgraph_type: str = "directional"
    track_edge_ids: bool = True
    temporal_strategy: str | None = None
    disjoint: bool = False
    deterministic: bool = False
    telemetry: Any = None
    rng_mode: str = "wyrand_exact"

    def __post_init__(self) -> None:
        nn = list(self.num_neighbors)
        if len(nn) == 0:
            raise ValueError("num_neighbors must be a non-empty list")
        if any(int(v) < 0 for v in nn):
            raise ValueError(f"num_neighbors values must be non-negative, got {nn}")
        self.num_neighbors = [int(v) for v in nn]
        if self.max_degree is not None and self.max_degree <= 0:
            raise ValueError(f"max_degree must be > 0 if specified, got {self.max_degree}")
        if self.subgraph_type not in _SUBGRAPH_TYPES:
            raise ValueError(f"Invalid subgraph_type '{self.subgraph_type}'. Must be 'directional', "
                             "'induced', or 'bidirectional'")
        if self.temporal_strategy is not None and self.temporal_strategy not in _TEMPORAL:
            raise ValueError(f"Invalid temporal_strategy '{self.temporal_strategy}'. Must be 'uniform' or 'last'")
        if self.seed is not None and not (0 <= int(self.seed) < 2**64):
            raise ValueError(f"seed must fit an unsigned 64-bit integer, got {self.seed}")
        if self.rng_mode not in _lib.RNG_MODE:
            raise ValueError(f"Invalid rng_mode '{self.rng_mode}'. Must be 'wyrand_exact' or 'philox'")

    def _unsupported(self) -> str | None:
        """Modes of the reference this GPU path does not implement."""
        if self.temporal_strategy is not None:
            return "temporal sampling"
        if self.max_degree is not None and self.weighted:
            return "max_degree with weighted sampling"
        if len(self.num_neighbors) > _lib.AG_MAX_HOPS:
            return f"more than {_lib.AG_MAX_HOPS} hops"
        return None

    def _to_c(self, seed: int, max_seeds: int = 0) -> _lib.SamplingConfigC:
        c = _lib.SamplingConfigC()
        c.num_hops = len(self.num_neighbors)
        for i, k in enumerate(self.num_neighbors):
            c.fanout[i] = k
        c.replace, c.weighted, c.track_edge_ids = int(self.replace), int(self.weighted), int(self.track_edge_ids)
        c.seed = seed
        c.rng_mode = _lib.RNG_MODE[self.rng_mode]
        c.max_seeds = max_seeds
        return c


def _align4(n: int) -> int:
    return (max(n, 1) + 3) & ~3


def coerce_seeds(seeds, num_nodes: int) -> np.ndarray:
    """Seed argument -> contiguous uint32 array (crates/aethergraph-py/src/error.rs:115-153):
    uint32 arrays pass through, int64 arrays and sequences are range-checked, and
    an id outside [0, num_nodes) raises SamplingError naming it."""
    a = np.asarray(seeds)
    if a.ndim != 1:
        a = a.reshape(-1)
    if a.dtype != np.uint32:
        if a.size and a.dtype.kind not in "iu":
            raise TypeError(f"seeds must be integers, got dtype {a.dtype}")
        if a.size:
            lo, hi = int(a.min()), int(a.max())
            bad = lo if lo < 0 else (hi if hi > 0xFFFFFFFF else None)
            if bad is not None:
                raise SamplingError(f"seed node {bad} out of u32 range [0, {0xFFFFFFFF}]")
        a = a.astype(np.uint32)
    if not a.flags.c_contiguous:
        a = np.ascontiguousarray(a)
    if a.size and num_nodes < 2**32 and int(a.max()) >= num_nodes:
        p = int(np.nonzero(a >= num_nodes)[0][0])
        raise SamplingError(f"seed node {int(a[p])} (position {p}) is out of range for {num_nodes} nodes")
    return a


class _DevArray:
    """A window of device memory for `torch.as_tensor` (CUDA array interface).  The
    tensor made from it keeps this object — and through `owner` the allocation —
    alive, so a view may outlive the batch object it came from."""

    __slots__ = ("__cuda_array_interface__", "owner")

    def __init__(self, ptr: int, shape: tuple, typestr: str, owner):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 2}
        self.owner = owner


class _Buffers:
    """Device output buffers of one batch: the pointer block handed to the C ABI
    plus whatever keeps the memory alive (torch tensors allocated here, or a lease
    on one of the loader's pooled sets).  Tensor views are made on demand."""

    __slots__ = ("c", "owner", "device", "dim")

    def __init__(self, c: _lib.SubgraphBuffers, owner, device, dim: int | None):
        self.c, self.owner, self.device, self.dim = c, owner, device, dim

    @staticmethod
    def alloc(device, cap_nodes: int, cap_edges: int, cap_seeds: int, track_eids: bool,
              feature_dim: int | None) -> "_Buffers":
        import torch

        cn, ce, cs = _align4(cap_nodes), _align4(cap_edges), _align4(cap_seeds)
        # One allocation per batch: the int64 arrays first (8-byte aligned), the
        # 32-bit arrays behind them.
        n64 = cn + 2 * ce + cs + (ce if track_eids else 0)
        n32 = cn + 4 * ce + cs
        arena = torch.empty(n64 + (n32 + 1) // 2, dtype=torch.int64, device=device)
        x = (torch.empty((max(cap_nodes, 1), feature_dim), dtype=torch.float32, device=device)
             if feature_dim is not None else None)
        base64 = arena.data_ptr()
        base32 = base64 + 8 * n64
        b = _lib.SubgraphBuffers()
        b.cap_nodes, b.cap_edges, b.cap_seeds = max(cap_nodes, 1), max(cap_edges, 1), max(cap_seeds, 1)
        b.nodes = base32
        b.edge_src = base32 + 4 * cn
        b.edge_dst = base32 + 4 * (cn + ce)
        b.src_local = base32 + 4 * (cn + 2 * ce)
        b.dst_local = base32 + 4 * (cn + 3 * ce)
        b.seed_locals = base32 + 4 * (cn + 4 * ce)
        b.n_id = base64
        b.edge_index_local = base64 + 8 * cn
        b.seed_index = base64 + 8 * (cn + 2 * ce)
        b.edge_ids = base64 + 8 * (cn + 2 * ce + cs) if track_eids else None
        b.e_id = None  # int64(edge id) has the same bits as the u64 the kernel writes
        b.x = x.data_ptr() if x is not None else None
        return _Buffers(b, (arena, x), device, feature_dim)

    def view(self, ptr, shape: tuple, typestr: str):
        import torch

        n = 1
        for s in shape:
            n *= s
        if not ptr or n == 0:
            dt = {"<i4": torch.int32, "<i8": torch.int64, "<f4": torch.float32}[typestr]
            return torch.empty(shape, dtype=dt, device=self.device)
        return torch.as_tensor(_DevArray(ptr, shape, typestr, self.owner), device=self.device)

    def record_stream(self, stream) -> None:
        """Torch-allocated buffers only: mark `stream` as a user of the memory."""
        if isinstance(self.owner, tuple):
            for t in self.owner:
                if hasattr(t, "record_stream"):  # not a pool lease
                    t.record_stream(stream)


def _u32_to_i64(t):
    """int32 tensor holding u32 bit patterns -> int64 values."""
    import torch

    return t.to(dtype=torch.int64) & 0xFFFFFFFF


class SampledSubgraph:
    """One sampled subgraph.  numpy accessors follow the reference
    (_core.pyi:207-261): all int64; row 0 of `edge_index` / `edge_index_local` is
    the sampled neighbor and row 1 the node whose row was expanded; `edge_ids[i]`
    is the CSR position of the stored edge row1 -> row0.  The `*_t` accessors
    return the same data as CUDA tensors without a copy."""

    __slots__ = ("_b", "_n", "_e", "_s", "_nodes_per_hop", "_edges_per_hop", "draws", "_seeds", "_cache", "_batch")

    def __init__(self, bufs: _Buffers, counts: _lib.SampleCounts, seeds: np.ndarray):
        self._b = bufs
        self._batch = None
        self._n, self._e, self._s = counts.num_nodes, counts.num_edges, counts.num_seeds
        h = counts.num_hops
        self._nodes_per_hop = counts.nodes_per_hop[:h + 1]
        self._edges_per_hop = counts.edges_per_hop[:h]
        self.draws = counts.draws
        self._seeds = seeds
        self._cache = None

    def _with_edges(self, bufs: "_Buffers", num_edges: int) -> "SampledSubgraph":
        """The same batch with rewritten edge arrays; per-hop counts keep describing
        the sampling pass (crates/aethergraph-core/src/loader/sampler.rs:1533-1536)."""
        out = SampledSubgraph.__new__(SampledSubgraph)
        out._b, out._n, out._e, out._s = bufs, self._n, num_edges, self._s
        out._nodes_per_hop, out._edges_per_hop = self._nodes_per_hop, self._edges_per_hop
        out.draws, out._seeds, out._cache = self.draws, self._seeds, None
        out._batch = self._batch
        return out

    # pooled batches (a loader's): which stream still reads them, and giving them back early
    def record_stream(self, stream) -> None:
        """A batch delivered by a loader lives in pooled memory that the loader writes again
        once the batch is dropped; by default it waits for the work queued on torch's
        CURRENT stream at that moment.  A consumer that reads the tensors on another stream
        names it here (a `torch.cuda.Stream` or a raw `cudaStream_t`)."""
        owner = self._b.owner
        if hasattr(owner, "stream"):
            owner.stream = stream

    def release(self, stream=None) -> None:
        """Give a loader's batch back now.  The loader reuses the memory after the work
        already queued on `stream` (default: the recorded stream, else the current one);
        the tensors of this batch must not be used by work queued later."""
        owner = self._b.owner
        if hasattr(owner, "release"):
            owner.release(stream)

    # counts
    @property
    def num_nodes(self) -> int:
        return self._n

    @property
    def num_edges(self) -> int:
        return self._e

    @property
    def num_seeds(self) -> int:
        return self._s

    def __len__(self) -> int:
        return self._n

    # device tensors
    @property
    def nodes_t(self):
        return self._b.view(self._b.c.n_id, (self._n,), "<i8")

    @property
    def edge_index_local_t(self):
        return self._b.view(self._b.c.edge_index_local, (2, self._e), "<i8")

    @property
    def edge_index_t(self):
        import torch

        b = self._b
        return torch.stack([_u32_to_i64(b.view(b.c.edge_dst, (self._e,), "<i4")),
                            _u32_to_i64(b.view(b.c.edge_src, (self._e,), "<i4"))])

    @property
    def edge_ids_t(self):
        if not self._b.c.edge_ids:
            return None
        return self._b.view(self._b.c.edge_ids, (self._e,), "<i8")

    @property
    def seed_indices_t(self):
        return self._b.view(self._b.c.seed_index, (self._s,), "<i8")

    @property
    def x(self):
        """Gathered feature rows [num_nodes, dim] (CUDA float32), or None."""
        if not self._b.c.x:
            return None
        return self._b.view(self._b.c.x, (self._n, self._b.dim), "<f4")

    def raw_u32(self) -> dict[str, Any]:
        """The core arrays in the reference's native widths (SampledSubgraph,
        crates/aethergraph-core/src/loader/sampler.rs:1512-1543), as host numpy."""
        b, n, e, s = self._b, self._n, self._e, self._s

        def u32(ptr, count):
            return b.view(ptr, (count,), "<i4").cpu().numpy().view(np.uint32)

        out = {"nodes": u32(b.c.nodes, n), "edge_src": u32(b.c.edge_src, e), "edge_dst": u32(b.c.edge_dst, e),
               "src_local": u32(b.c.src_local, e), "dst_local": u32(b.c.dst_local, e),
               "seed_locals": u32(b.c.seed_locals, s)}
        t = self.edge_ids_t
        out["edge_ids"] = t.cpu().numpy().view(np.uint64) if t is not None else None
        out["num_sampled_nodes"] = np.array(self._nodes_per_hop, dtype=np.uint64)
        out["num_sampled_edges"] = np.array(self._edges_per_hop, dtype=np.uint64)
        out["draws"] = int(self.draws)
        return out

    # numpy accessors of the reference API (cached: the same array on every access)
    def _np(self, key, make):
        if self._cache is None:
            self._cache = {}
        if key not in self._cache:
            self._cache[key] = make()
        return self._cache[key]

    @property
    def nodes(self) -> np.ndarray:
        return self._np("nodes", lambda: self.nodes_t.cpu().numpy())

    @property
    def seeds(self) -> np.ndarray:
        return self._np("seeds", lambda: self._seeds.astype(np.int64))

    @property
    def edge_index(self) -> np.ndarray:
        return self._np("edge_index", lambda: self.edge_index_t.cpu().numpy())

    @property
    def edge_index_local(self) -> np.ndarray:
        return self._np("edge_index_local", lambda: self.edge_index_local_t.cpu().numpy())

    @property
    def edge_ids(self) -> np.ndarray:
        def make():
            t = self.edge_ids_t
            return np.empty(0, dtype=np.int64) if t is None else t.cpu().numpy()
        return self._np("edge_ids", make)

    @property
    def seed_indices(self) -> np.ndarray:
        return self._np("seed_indices", lambda: self.seed_indices_t.cpu().numpy())

    @property
    def batch(self):
        """Disjoint sampling: for every node the index of the seed whose block it belongs to
        (int64); None otherwise."""
        return self._batch

    @property
    def num_sampled_nodes_per_hop(self) -> list[int]:
        return list(self._nodes_per_hop)

    @property
    def num_sampled_edges_per_hop(self) -> list[int]:
        return list(self._edges_per_hop)

    def to_dict(self) -> dict[str, Any]:
        return {
            "nodes": self.nodes, "seeds": self.seeds, "edge_index": self.edge_index,
            "edge_index_local": self.edge_index_local, "edge_ids": self.edge_ids,
            "seed_indices": self.seed_indices, "batch": self.batch,
            "num_sampled_nodes_per_hop": self.num_sampled_nodes_per_hop,
            "num_sampled_edges_per_hop": self.num_sampled_edges_per_hop,
        }

    def __repr__(self) -> str:
        return f"SampledSubgraph(num_nodes={self._n}, num_edges={self._e}, num_seeds={self._s})"


def apply_subgraph_type(graph: CsrGraph, subgraph_type: str, sg: SampledSubgraph) -> SampledSubgraph:
    """`subgraph_type` "bidirectional" / "induced" on a finished batch
    (crates/aethergraph-core/src/loader/sampler.rs:964-1040): new edge arrays in GPU
    memory, written by the library's rewrite kernels; nodes, seeds and x are shared
    with the sampled batch."""
    import torch

    if subgraph_type == "directional":
        return sg
    L = _lib.lib()
    b, e = sg._b, sg._e
    dev = b.device
    track = bool(b.c.edge_ids)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        plan = None
        if subgraph_type == "bidirectional":
            cap = max(2 * e, 1)
        else:
            plan, n_out = C.c_void_p(), C.c_uint64()
            _lib.check(L.ag_subgraph_induce_plan(graph._h, b.c.nodes, sg._n, stream, C.byref(plan), C.byref(n_out)))
            cap = max(int(n_out.value), 1)
        try:
            cap4 = _align4(cap)
            n64 = 2 * cap4 + (cap4 if track else 0)
            arena = torch.empty(n64 + 2 * cap4, dtype=torch.int64, device=dev)
            base64 = arena.data_ptr()
            base32 = base64 + 8 * n64
            c = _lib.SubgraphBuffers.from_buffer_copy(b.c)
            c.cap_edges = cap
            c.edge_index_local = base64
            c.edge_ids = base64 + 16 * cap4 if track else None
            c.edge_src, c.edge_dst = base32, base32 + 4 * cap4
            c.src_local, c.dst_local = base32 + 8 * cap4, base32 + 12 * cap4
            nb = _Buffers(c, (*(b.owner if isinstance(b.owner, tuple) else (b.owner,)), arena), dev, b.dim)
            if subgraph_type == "bidirectional":
                for name in ("edge_src", "edge_dst", "src_local", "dst_local"):
                    if e:
                        nb.view(getattr(c, name), (e,), "<i4").copy_(b.view(getattr(b.c, name), (e,), "<i4"))
                if track and e:
                    nb.view(c.edge_ids, (e,), "<i8").copy_(b.view(b.c.edge_ids, (e,), "<i8"))
                n_out = C.c_uint64()
                _lib.check(L.ag_subgraph_mirror(dev.index, e, cap, c.edge_src, c.edge_dst, c.src_local, c.dst_local,
                                                c.edge_ids, c.edge_index_local, C.byref(n_out), stream))
            else:
                _lib.check(L.ag_subgraph_induce_fill(plan, cap, c.edge_src, c.edge_dst, c.src_local, c.dst_local,
                                                     c.edge_ids, c.edge_index_local, stream))
        finally:
            if plan is not None and plan.value:
                L.ag_subgraph_induce_free(plan)
    return sg._with_edges(nb, int(n_out.value))


class _Handle:
    """One ag_sampler: scratch for one group of batches in flight."""

    def __init__(self, graph: CsrGraph, config: SamplingConfig, seed: int, max_seeds: int = 0, group: int = 1):
        import torch

        self.graph, self.config, self.group = graph, config, group
        self.device = torch.device("cuda", graph.device)
        self.h = C.c_void_p()
        self._bounds: dict[int, tuple[int, int]] = {}
        cfg = config._to_c(seed, max_seeds)
        _lib.check(_lib.lib().ag_sampler_create_group(graph._h, C.byref(cfg), group, C.byref(self.h)))

    def __del__(self):
        h = getattr(self, "h", None)
        if h:
            try:
                _lib.lib().ag_sampler_free(h)
            except Exception:
                pass
            self.h = None

    def reseed(self, seed: int) -> None:
        _lib.check(_lib.lib().ag_sampler_reseed(self.h, seed & (2**64 - 1)))

    def bounds(self, n_seeds: int) -> tuple[int, int]:
        b = self._bounds.get(n_seeds)
        if b is None:
            mn, me = C.c_uint64(), C.c_uint64()
            _lib.check(_lib.lib().ag_sampler_bounds(self.h, n_seeds, C.byref(mn), C.byref(me)))
            b = self._bounds[n_seeds] = (mn.value, me.value)
        return b


class _PendingGroup:
    """A group of batches queued as one launch chain; `results()` waits for it."""

    def __init__(self, handle: _Handle, bufs: list[_Buffers], seeds: list[np.ndarray], keep):
        self._handle, self._bufs, self._seeds, self._keep = handle, bufs, seeds, keep
        self._done: list[SampledSubgraph] | None = None

    def __len__(self) -> int:
        return len(self._bufs)

    def results(self) -> list[SampledSubgraph]:
        if self._done is None:
            n = len(self._bufs)
            counts = (_lib.SampleCounts * n)()
            _lib.check(_lib.lib().ag_sample_group_wait(self._handle.h, counts, None))
            kind = self._handle.config.subgraph_type
            self._done = [apply_subgraph_type(self._handle.graph, kind, SampledSubgraph(b, c, s))
                          for b, c, s in zip(self._bufs, counts, self._seeds)]
            self._keep = None
        return self._done


def _submit_group(handle: _Handle, seeds: list[np.ndarray], batch_seeds: list[int] | None,
                  features: FeatureStore | None, stream=None) -> _PendingGroup:
    import torch

    n = len(seeds)
    dev = handle.device
    dim = features.feature_dim if features is not None else None
    bufs = []
    cbufs = (_lib.SubgraphBuffers * n)()
    ptrs = (C.c_void_p * n)()
    lens = (C.c_uint64 * n)()
    bseeds = (C.c_uint64 * n)(*[s & (2**64 - 1) for s in batch_seeds]) if batch_seeds is not None else None
    for i, s in enumerate(seeds):
        mn, me = handle.bounds(len(s))
        b = _Buffers.alloc(dev, mn, me, len(s), handle.config.track_edge_ids, dim)
        bufs.append(b)
        cbufs[i] = b.c
        ptrs[i] = s.ctypes.data if len(s) else None
        lens[i] = len(s)
    st = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().ag_sample_group_into(handle.h, n, ptrs, lens, _lib.AG_MEM_HOST, bseeds,
                                               features._h if features is not None else None, cbufs, st))
    return _PendingGroup(handle, bufs, seeds, (cbufs, ptrs, lens, bseeds))


def _check_config(graph: CsrGraph, config: SamplingConfig, *, pipelined: bool = False) -> None:
    """`pipelined`: the caller runs groups of batches per launch chain (loaders, the parallel
    batch sampler).  Disjoint sampling is sequential seed by seed in the exact mode, so only
    the plain `NeighborSampler` offers it."""
    if not isinstance(config, SamplingConfig):
        raise TypeError("config must be a SamplingConfig")
    bad = config._unsupported()
    if bad is None and pipelined and config.disjoint:
        bad = "disjoint sampling in a parallel batch sampler (use NeighborSampler or NeighborLoader; it runs one seed after the other)"
    if bad is None and pipelined and config.cumulative:
        bad = "cumulative sampling in a parallel batch sampler (use NeighborSampler or NeighborLoader; it runs one launch chain per hop)"
    if bad is None and config.cumulative and config.disjoint:
        bad = "cumulative together with disjoint sampling"
    if bad:
        raise ValueError(f"{bad} is not supported by the GPU minibatch path")
    if config.weighted and not graph.has_weights:
        raise ValueError("weighted sampling requested, but the graph has no edge weights")


class NeighborSampler:
    """Single-graph neighborhood sampler.  The RNG stream advances across
    `sample()` calls, so consecutive batches differ and a fresh sampler with the
    same seed replays the sequence (crates/aethergraph-py/src/sampler.rs:782-785).
    `features` (optional) gathers `x` for every batch in the same launch chain."""

    def __init__(self, graph: CsrGraph, config: SamplingConfig, features: FeatureStore | None = None):
        _check_config(graph, config)
        self.graph, self.config, self.features = graph, config, features
        seed = config.seed if config.seed is not None else secrets.randbits(64)
        self._handle = _Handle(graph, config, seed)
        self._handle_seed = seed
        self._cum_draws = 0   # cumulative mode carries the stream position itself

    def reseed(self, seed: int) -> None:
        """Restart the RNG stream at draw 0 of `seed` (NeighborSampler::reseed, sampler.rs:509-511)."""
        seed = int(seed) & (2**64 - 1)
        self._handle.reseed(seed)
        self._handle_seed, self._cum_draws = seed, 0

    def sample(self, seeds, input_times=None) -> SampledSubgraph:
        if input_times is not None:
            raise SamplingError("temporal sampling: SamplingConfig::temporal_strategy is None")
        s = coerce_seeds(seeds, self.graph.num_nodes)
        if self.config.disjoint:
            return self._sample_disjoint(s)
        if self.config.cumulative:
            return self._sample_cumulative(s)
        return _submit_group(self._handle, [s], None, self.features).results()[0]

    _WYRAND_STEP = 0xA0761D6478BD642F  # the generator's additive constant (internal/genstamp.rs:181-202)

    def _sample_cumulative(self, seeds: np.ndarray) -> SampledSubgraph:
        """Cumulative sampling (crates/aethergraph-core/src/loader/sampler.rs:834-837,
        1250-1258, 1277-1285): every hop expands ALL nodes seen so far, and an edge that an
        earlier hop emitted is refused (repeats within one hop pass).  Composed hop by hop from
        the one-hop sampler: the frontier of hop h is the node list so far, which is exactly
        the distinct-seed prefix of a one-hop batch seeded with it, so local ids agree from hop
        to hop; the refused edges are filtered by edge id on the device.  The RNG stream is
        carried by reseeding: draw d of a WyRand stream seeded s is draw 0 of one seeded
        s + d * step."""
        import torch

        cfg, dev = self.config, self._handle.device
        base = self._handle_seed
        frontier, seed_locals = seeds, None
        kept: list[dict] = []
        nodes_t = None
        emitted = torch.empty(0, dtype=torch.int64, device=dev)
        nodes_per_hop, edges_per_hop = [], []
        for hop, k in enumerate(cfg.num_neighbors):
            h = self._hop_handle(k)
            if cfg.rng_mode == "wyrand_exact":
                h.reseed(base + self._cum_draws * self._WYRAND_STEP)
            else:  # counter-based draws are keyed on (seed, vertex, slot): a key of its own per hop and call
                h.reseed(int(_lib.lib().ag_batch_seed(base, self._cum_draws * 64 + hop)))
            one = _submit_group(h, [np.ascontiguousarray(frontier, dtype=np.uint32)], None, None).results()[0]
            self._cum_draws += int(one.draws) if cfg.rng_mode == "wyrand_exact" else 1
            b, n, e = one._b, one._n, one._e
            if hop == 0:
                nodes_per_hop.append(int(one._nodes_per_hop[0]))
                seed_locals = b.view(b.c.seed_locals, (len(seeds),), "<i4").clone()
            nodes_per_hop.append(int(one._nodes_per_hop[1]))
            nodes_t = b.view(b.c.nodes, (n,), "<i4").clone()
            if e:
                eid = b.view(b.c.edge_ids, (e,), "<i8")
                keep = ~torch.isin(eid, emitted) if emitted.numel() else torch.ones(e, dtype=torch.bool, device=dev)
                part = {name: b.view(getattr(b.c, name), (e,), "<i4")[keep].clone()
                        for name in ("edge_src", "edge_dst", "src_local", "dst_local")}
                part["edge_ids"] = eid[keep].clone()
            else:
                part = {name: torch.empty(0, dtype=torch.int32, device=dev)
                        for name in ("edge_src", "edge_dst", "src_local", "dst_local")}
                part["edge_ids"] = torch.empty(0, dtype=torch.int64, device=dev)
            kept.append(part)
            edges_per_hop.append(int(part["edge_ids"].numel()))
            emitted = torch.unique(torch.cat([emitted, part["edge_ids"]]))
            frontier = nodes_t.cpu().numpy().view(np.uint32)
        n_tot, e_tot, S = int(nodes_t.numel()), sum(edges_per_hop), len(seeds)
        dim = self.features.feature_dim if self.features is not None else None
        out = _Buffers.alloc(dev, max(n_tot, 1), max(e_tot, 1), max(S, 1), cfg.track_edge_ids, dim)
        c = out.c
        out.view(c.nodes, (n_tot,), "<i4").copy_(nodes_t)
        out.view(c.n_id, (n_tot,), "<i8").copy_(_u32_to_i64(nodes_t))
        if S:
            out.view(c.seed_locals, (S,), "<i4").copy_(seed_locals)
            out.view(c.seed_index, (S,), "<i8").copy_(_u32_to_i64(seed_locals))
        if e_tot:
            for name in ("edge_src", "edge_dst", "src_local", "dst_local"):
                out.view(getattr(c, name), (e_tot,), "<i4").copy_(torch.cat([p[name] for p in kept]))
            if cfg.track_edge_ids:
                out.view(c.edge_ids, (e_tot,), "<i8").copy_(torch.cat([p["edge_ids"] for p in kept]))
            ei = out.view(c.edge_index_local, (2, e_tot), "<i8")
            ei[0].copy_(_u32_to_i64(out.view(c.dst_local, (e_tot,), "<i4")))
            ei[1].copy_(_u32_to_i64(out.view(c.src_local, (e_tot,), "<i4")))
        if dim is not None and n_tot:
            self.features.gather(out.view(c.n_id, (n_tot,), "<i8"), out=out.view(c.x, (n_tot, dim), "<f4"))
        torch.cuda.current_stream(dev).synchronize()
        counts = _lib.SampleCounts()
        counts.num_nodes, counts.num_edges, counts.num_seeds, counts.num_hops = n_tot, e_tot, S, len(cfg.num_neighbors)
        for i, v in enumerate(nodes_per_hop):
            counts.nodes_per_hop[i] = v
        for i, v in enumerate(edges_per_hop):
            counts.edges_per_hop[i] = v
        sg = SampledSubgraph(out, counts, seeds)
        return apply_subgraph_type(self.graph, cfg.subgraph_type, sg)

    def _hop_handle(self, fanout: int) -> "_Handle":
        """A one-hop sampler with this fanout and the batch's flags, edge ids on."""
        handles = self.__dict__.setdefault("_hop_handles", {})
        if fanout not in handles:
            one = SamplingConfig(num_neighbors=[fanout], replace=self.config.replace, weighted=self.config.weighted,
                                 track_edge_ids=True, seed=0, rng_mode=self.config.rng_mode)
            handles[fanout] = _Handle(self.graph, one, 0)
        return handles[fanout]

    def _sample_disjoint(self, seeds: np.ndarray) -> SampledSubgraph:
        """Every seed sampled on its own, nothing shared between the blocks, the blocks
        concatenated with their local indices shifted and a `batch` vector naming each node's
        seed (crates/aethergraph-core/src/loader/sampler.rs:600-690).  The reference's RNG
        stream runs on from one seed's tree into the next, and how many draws a tree takes
        depends on what it sampled, so in the exact mode the seeds are inherently sequential:
        one launch chain per seed.  Exact, and slow; `subgraph_type` applies inside each block."""
        import torch

        h = self._handle
        blocks = [_submit_group(h, [seeds[i:i + 1]], None, self.features).results()[0] for i in range(len(seeds))]
        n_tot, e_tot, S = sum(b._n for b in blocks), sum(b._e for b in blocks), len(seeds)
        dim = self.features.feature_dim if self.features is not None else None
        track = self.config.track_edge_ids
        out = _Buffers.alloc(h.device, max(n_tot, 1), max(e_tot, 1), max(S, 1), track, dim)
        c = out.c
        hops = len(self.config.num_neighbors)
        counts = _lib.SampleCounts()
        counts.num_nodes, counts.num_edges, counts.num_seeds, counts.num_hops = n_tot, e_tot, S, hops
        counts.nodes_per_hop[0] = S        # every block contributes its one seed node up front
        n_at = e_at = 0
        batch = np.empty(n_tot, dtype=np.int64)
        for i, b in enumerate(blocks):
            bb, n, e = b._b, b._n, b._e
            if n:
                out.view(c.nodes + 4 * n_at, (n,), "<i4").copy_(bb.view(bb.c.nodes, (n,), "<i4"))
                out.view(c.n_id + 8 * n_at, (n,), "<i8").copy_(bb.view(bb.c.n_id, (n,), "<i8"))
                if dim is not None:
                    out.view(c.x + 4 * dim * n_at, (n, dim), "<f4").copy_(bb.view(bb.c.x, (n, dim), "<f4"))
            if e:
                for name in ("edge_src", "edge_dst"):
                    out.view(getattr(c, name) + 4 * e_at, (e,), "<i4").copy_(bb.view(getattr(bb.c, name), (e,), "<i4"))
                for name in ("src_local", "dst_local"):
                    out.view(getattr(c, name) + 4 * e_at, (e,), "<i4").copy_(bb.view(getattr(bb.c, name), (e,), "<i4") + n_at)
                if track:
                    out.view(c.edge_ids + 8 * e_at, (e,), "<i8").copy_(bb.view(bb.c.edge_ids, (e,), "<i8"))
            out.view(c.seed_locals + 4 * i, (1,), "<i4").copy_(bb.view(bb.c.seed_locals, (1,), "<i4") + n_at)
            out.view(c.seed_index + 8 * i, (1,), "<i8").copy_(bb.view(bb.c.seed_index, (1,), "<i8") + n_at)
            for k in range(hops):
                counts.nodes_per_hop[k + 1] += b._nodes_per_hop[k + 1]
                counts.edges_per_hop[k] += b._edges_per_hop[k]
            counts.draws += b.draws
            batch[n_at:n_at + n] = i
            n_at += n
            e_at += e
        # the packed [2, E] int64 edge index of the whole batch: neighbour row, then expanded-node row
        if e_tot:
            ei = out.view(c.edge_index_local, (2, e_tot), "<i8")
            ei[0].copy_(_u32_to_i64(out.view(c.dst_local, (e_tot,), "<i4")))
            ei[1].copy_(_u32_to_i64(out.view(c.src_local, (e_tot,), "<i4")))
        torch.cuda.current_stream(h.device).synchronize()
        sg = SampledSubgraph(out, counts, seeds)
        sg._batch = batch
        return sg

    def __repr__(self) -> str:
        return f"NeighborSampler(num_neighbors={self.config.num_neighbors}, replace={self.config.replace})"


Sampler = NeighborSampler


class ParallelBatchSampler:
    """Samples many batches concurrently.  The batch at stream position p (counted
    over every batch this sampler has handled) draws from
    `batch_seed(config.seed, p)`, so a fixed seed gives the same output however
    the batches are scheduled (crates/aethergraph-core/src/loader/sampler.rs:1726-1751).
    Here the parallelism is on the device: up to `group` batches ride one launch
    chain (each kernel's grid has the batch as a second dimension), and `streams`
    such chains overlap on their own CUDA streams."""

    def __init__(self, graph: CsrGraph, config: SamplingConfig, features: FeatureStore | None = None,
                 streams: int = 2, group: int = 16):
        import torch

        _check_config(graph, config, pipelined=True)
        self.graph, self.config, self.features = graph, config, features
        self._base = config.seed if config.seed is not None else secrets.randbits(64)
        self._next = 0
        self._group = max(1, int(group))
        dev = torch.device("cuda", graph.device)
        self._handles = [_Handle(graph, config, self._base, group=self._group) for _ in range(max(1, streams))]
        self._streams = [torch.cuda.Stream(dev) for _ in self._handles]

    def sample_batches(self, batches: Sequence) -> list[SampledSubgraph]:
        import torch

        seeds = [coerce_seeds(b, self.graph.num_nodes) for b in batches]
        first = self._next
        self._next += len(seeds)
        out: list[SampledSubgraph | None] = [None] * len(seeds)
        pending: list[tuple[int, _PendingGroup] | None] = [None] * len(self._handles)
        cur = torch.cuda.current_stream()
        G = self._group
        for c, lo in enumerate(range(0, len(seeds), G)):
            k = c % len(self._handles)
            if pending[k] is not None:
                i, p = pending[k]
                out[i:i + len(p)] = p.results()
            h, st = self._handles[k], self._streams[k]
            chunk = seeds[lo:lo + G]
            bseeds = [_lib.lib().ag_batch_seed(self._base, first + lo + j) for j in range(len(chunk))]
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                pending[k] = (lo, _submit_group(h, chunk, bseeds, self.features, st.cuda_stream))
        for slot in pending:
            if slot is not None:
                i, p = slot
                out[i:i + len(p)] = p.results()
        for st in self._streams:
            cur.wait_stream(st)
        for sg in out:
            # The buffers were allocated on a side stream; tell the allocator the
            # caller's stream uses them too before it may recycle them.
            sg._b.record_stream(cur)  # type: ignore[union-attr]
        return out  # type: ignore[return-value]


SAMPLE_PAD = 0xFFFFFFFF


def reservoir_hop(graph: CsrGraph, nodes, fanout: int, seed: int, layer: int = 0):
    """One hop of the reference's Philox fast mode for a list of nodes: returns
    `(neighbors [n, fanout] int32 CUDA tensor holding u32 ids, counts [n])`, bit for
    bit what `reservoir_sample` (crates/aethergraph-core/src/internal/philox.rs:59-82)
    and the `warp_sample_neighbors` kernel give; unused slots hold SAMPLE_PAD."""
    import torch

    dev = torch.device("cuda", graph.device)
    if isinstance(nodes, torch.Tensor):
        ids = nodes.to(device=dev, dtype=torch.int64).contiguous()
    else:
        ids = torch.from_numpy(np.ascontiguousarray(np.asarray(nodes).astype(np.uint64)).view(np.int64)).to(dev)
    n = int(ids.numel())
    out = torch.empty((n, int(fanout)), dtype=torch.int32, device=dev)
    counts = torch.empty((n,), dtype=torch.int32, device=dev)
    _lib.check(_lib.lib().ag_sample_hop_reservoir(graph._h, ids.data_ptr() if n else None, n, int(fanout),
                                                  int(seed) & (2**64 - 1), int(layer), out.data_ptr(),
                                                  counts.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return out, counts

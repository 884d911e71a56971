"""Epoch driver: iterate a graph's seed nodes in batches and yield sampled
subgraphs with their feature rows, all of it already in GPU memory.

Same constructor arguments, batch order, per-epoch seeding and batch attributes
as the reference's `aethergraph.pytorch.NeighborLoader`
(python/aethergraph/pytorch/loader.py:386-1079):

- seed batches: slices of `input_nodes` (optionally through a permutation), or,
  for all nodes with `shuffle`, an O(1)-memory coprime-stride walk (`:140-184`);
  the numpy `Generator` is consumed call for call like the reference's, so a
  given `seed` yields the same batches;
- the sampler seed of an epoch is the next child of `SeedSequence(seed)`
  (`:195-205`); inside an epoch batch number b is sampled from
  `batch_seed(epoch_seed, b)` and batches arrive in order;
- a sliding window of submitted batches keeps the native loader busy (`:817-897`).

The batch object is a `torch_geometric.data.Data` when PyG is installed and the
attribute-compatible `Batch` below otherwise.  Every tensor is a CUDA tensor on
the graph's device: nothing is copied to the host.
"""
from __future__ import annotations

import dataclasses
import math
import os
import time
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator

import numpy as np

from ..features import FeatureStore
from ..graph import CsrGraph
from ..loader import NeighborLoader as NativeLoader
from ..sampler import SamplingConfig

__all__ = ["Batch", "LoaderMetrics", "NeighborLoader", "epoch_sampling_seed", "make_batch_getter",
           "normalize_input_nodes"]


class Batch:
    """Attribute bag with the fields the reference puts on a PyG `Data`
    (loader.py:935-951): x, edge_index, e_id, n_id, batch_size, input_id,
    seed_index, num_nodes, num_sampled_nodes, num_sampled_edges."""

    def __init__(self, **kw: Any):
        self.__dict__.update(kw)

    def keys(self) -> list[str]:
        return [k for k, v in self.__dict__.items() if v is not None]

    def to(self, device, non_blocking: bool = False) -> "Batch":
        import torch

        return Batch(**{k: (v.to(device, non_blocking=non_blocking) if isinstance(v, torch.Tensor) else v)
                        for k, v in self.__dict__.items()})

    def __repr__(self) -> str:
        import torch

        parts = [f"{k}={list(v.shape)}" if isinstance(v, torch.Tensor) else f"{k}={v}" for k, v in self.__dict__.items()
                 if v is not None]
        return "Batch(" + ", ".join(parts) + ")"


def _make_data(**kw):
    try:
        from torch_geometric.data import Data  # type: ignore
    except ImportError:
        return Batch(**kw)
    return Data(**kw)


def normalize_input_nodes(input_nodes, *, num_nodes: int, what: str = "input_nodes") -> np.ndarray:
    """Mask or explicit ids -> contiguous 1D int64 ids in [0, num_nodes)
    (loader.py:54-111: a bool array is a mask; floats are rejected)."""
    import torch

    if isinstance(input_nodes, torch.Tensor):
        if input_nodes.dtype.is_floating_point:
            raise ValueError(f"{what} must be integer or bool IDs, got dtype {input_nodes.dtype}")
        a = input_nodes.cpu().numpy()
    else:
        a = np.asarray(input_nodes)
    if a.dtype == np.bool_:
        arr = np.nonzero(a)[0].astype(np.int64)
    elif np.issubdtype(a.dtype, np.integer):
        arr = a.astype(np.int64, copy=False)
    else:
        raise ValueError(f"{what} must be integer or bool IDs, got dtype {a.dtype}")
    if arr.ndim != 1:
        raise ValueError(f"{what} must be a 1D array-like, got shape {arr.shape}")
    if arr.size:
        lo, hi = int(arr.min()), int(arr.max())
        if lo < 0:
            raise ValueError(f"{what} must contain non-negative node IDs (min {lo})")
        if hi >= num_nodes:
            raise ValueError(f"{what} contains out-of-range node IDs (max {hi} >= num_nodes={num_nodes})")
    return np.ascontiguousarray(arr)


def make_batch_getter(input_nodes: np.ndarray | None, num_nodes: int, batch_size: int, shuffle: bool,
                      rng: np.random.Generator) -> Callable[[int], tuple[np.ndarray, np.ndarray]]:
    """`batch_idx -> (seeds, input_id)` for one epoch (loader.py:140-192).  The
    generator calls (permutation; or integers + coprime stride search) are the
    reference's, in its order."""
    def bounds(b: int) -> tuple[int, int]:
        start = b * batch_size
        return start, min(start + batch_size, num_nodes)

    if input_nodes is not None:
        order = rng.permutation(num_nodes) if shuffle else None

        def sliced(b: int):
            start, end = bounds(b)
            if order is None:
                return input_nodes[start:end], np.arange(start, end, dtype=np.int64)
            pos = order[start:end]
            return input_nodes[pos], pos

        return sliced
    if shuffle and num_nodes > 0:
        offset = int(rng.integers(0, num_nodes))
        stride = 1
        while num_nodes > 1:  # a random stride coprime with num_nodes walks a full permutation
            stride = int(rng.integers(1, num_nodes))
            if math.gcd(stride, num_nodes) == 1:
                break

        def strided(b: int):
            start, end = bounds(b)
            idx = (np.arange(start, end, dtype=np.int64) * stride + offset) % num_nodes
            return idx, idx

        return strided

    def ranged(b: int):
        start, end = bounds(b)
        idx = np.arange(start, end, dtype=np.int64)
        return idx, idx

    return ranged


def epoch_sampling_seed(seeds: np.random.SeedSequence | None) -> int | None:
    """The next epoch's sampler seed (loader.py:195-205); None stays None."""
    if seeds is None:
        return None
    (child,) = seeds.spawn(1)
    return int(child.generate_state(1, dtype=np.uint64)[0])


@dataclass
class LoaderMetrics:
    """Counters of the most recent epoch (loader.py:296-341)."""

    batches_processed: int = 0
    total_time_ms: float = 0.0
    avg_batch_time_ms: float = 0.0
    prefetch_hit_rate: float = 0.0
    prefetch_hits: int = 0
    prefetch_misses: int = 0
    _epoch_start: float = field(default=0.0, repr=False)

    def to_dict(self) -> dict[str, float | int]:
        return {k: getattr(self, k) for k in ("batches_processed", "total_time_ms", "avg_batch_time_ms",
                                              "prefetch_hit_rate", "prefetch_hits", "prefetch_misses")}


class NeighborLoader:
    """Drop-in for `aethergraph.pytorch.NeighborLoader` on a GPU-resident graph.

    `features` may be a `FeatureStore`, a float32 `[num_nodes, dim]` array (kept in
    GPU memory as f32) or left out in favour of `feature_path` (an AETHFEAT file).
    `num_workers` is the number of native sampler threads (0 and 1 both mean one).
    Not available on this path: `DynamicGraph` inputs, `feature_source`
    (`rdma://`), `input_time`, and the sampling modes `SamplingConfig` rejects.
    """

    def __init__(self, data: CsrGraph, num_neighbors: list[int], input_nodes=None, batch_size: int = 128,
                 shuffle: bool = True, replace: bool = False, weighted: bool = False, num_workers: int = 0,
                 prefetch_factor: int = 3, pin_memory: bool = False, device: str | None = None,
                 transfer_depth: int = 2, transform: Callable | None = None, feature_source: str | None = None,
                 gpu_id: int = 0, input_time=None, temporal_strategy: str | None = None, disjoint: bool = False,
                 seed: int | None = None, generator: np.random.Generator | None = None,
                 max_degree: int | None = None, cumulative: bool = False, subgraph_type: str = "directional",
                 track_edge_ids: bool = True, neighbor_sampler: Callable | None = None, features=None,
                 feature_path=None, group: int = 8, rng_mode: str = "wyrand_exact"):
        if not isinstance(data, CsrGraph):
            raise TypeError(f"data must be an aethergraph_b200 Graph resident on the GPU, got {type(data).__name__}")
        if batch_size < 1:
            raise ValueError("batch_size must be >= 1")
        if prefetch_factor < 1:
            raise ValueError("prefetch_factor must be >= 1")
        if feature_source is not None:
            if not str(feature_source).startswith("rdma://"):
                raise ValueError(f"unrecognized feature_source {feature_source!r}: expected 'rdma://host:port'")
            raise RuntimeError("feature_source='rdma://' is not available: features are gathered from GPU memory")
        if input_time is not None:
            raise NotImplementedError("per-seed input_time is not supported by NeighborLoader's prefetch pipeline")
        if features is not None and feature_path is not None:
            raise ValueError("pass either `features` or `feature_path`, not both")
        self.graph = data
        self.num_neighbors = list(num_neighbors)
        self.batch_size, self.shuffle, self.replace, self.weighted = batch_size, shuffle, replace, weighted
        self.prefetch_factor, self.pin_memory, self.transform = prefetch_factor, pin_memory, transform
        self._neighbor_sampler = neighbor_sampler
        self._threads = max(1, int(num_workers))
        self._group = max(1, int(group))
        self._track_edge_ids = track_edge_ids
        self._sampling = SamplingConfig(num_neighbors=self.num_neighbors, replace=replace, seed=seed,
                                        max_degree=max_degree, cumulative=cumulative, weighted=weighted,
                                        subgraph_type=subgraph_type, track_edge_ids=track_edge_ids,
                                        temporal_strategy=temporal_strategy, disjoint=disjoint, rng_mode=rng_mode)
        n = data.num_nodes
        if features is None and feature_path is None:
            features = getattr(data, "features", None)  # attached by Graph.load_features
        if features is None and feature_path is not None:
            features = FeatureStore.load(os.fspath(feature_path), device=data.device)
        if features is not None and not isinstance(features, FeatureStore):
            arr = np.asarray(features)
            if arr.dtype != np.float32:
                raise ValueError(f"features must be float32 (got {arr.dtype}); cast explicitly before passing")
            if arr.ndim != 2:
                raise ValueError(f"features must be 2D, got shape {arr.shape}")
            if arr.shape[0] != n:
                raise ValueError(f"features.shape[0]={arr.shape[0]} does not match graph num_nodes={n}")
            features = FeatureStore.from_array(np.ascontiguousarray(arr), dtype="f32", device=data.device)
        self._features: FeatureStore | None = features
        if input_nodes is None:
            self._input_nodes, self._num_input_nodes = None, n
        else:
            self._input_nodes = normalize_input_nodes(input_nodes, num_nodes=n)
            self._num_input_nodes = len(self._input_nodes)
        self._out_device = device
        self._rng = generator if generator is not None else np.random.default_rng(seed)
        self._sampling_seeds = np.random.SeedSequence(seed) if seed is not None else None
        self._metrics = LoaderMetrics()

    @property
    def metrics(self) -> LoaderMetrics:
        return self._metrics

    def __len__(self) -> int:
        return (self._num_input_nodes + self.batch_size - 1) // self.batch_size

    def __repr__(self) -> str:
        return (f"NeighborLoader(num_nodes={self._num_input_nodes}, num_neighbors={self.num_neighbors}, "
                f"batch_size={self.batch_size})")

    def __iter__(self) -> Iterator:
        num_batches = len(self)
        rng = self._rng.spawn(1)[0]
        get_batch = make_batch_getter(self._input_nodes, self._num_input_nodes, self.batch_size, self.shuffle, rng)
        if self._neighbor_sampler is not None:  # a user-supplied sampler bypasses the native path (loader.py:715-721)
            for b in range(num_batches):
                out = self._neighbor_sampler(self.graph, get_batch(b)[0])
                yield self.transform(out) if self.transform is not None else out
            return
        sampling = dataclasses.replace(self._sampling, seed=epoch_sampling_seed(self._sampling_seeds))
        native = NativeLoader(self.graph, sampling, self.prefetch_factor, self._threads, features=self._features,
                              group=self._group)
        yield from self._drive_epoch(native, num_batches, get_batch)

    def _drive_epoch(self, native: NativeLoader, num_batches: int, get_batch) -> Iterator:
        """Prime a window of submissions, then receive / resubmit one for one
        (loader.py:817-897).  The window is at least `prefetch_factor` and at least
        what the native workers can hold in flight (threads x group)."""
        import torch

        window = max(self.prefetch_factor, self._threads * self._group)
        window = min(window, 8 * self.prefetch_factor)  # never more than the native work queue holds
        submitted = received = 0
        input_ids: dict[int, np.ndarray] = {}
        start = time.perf_counter()
        dev = torch.device("cuda", self.graph.device)
        try:
            while received < num_batches:
                while submitted < num_batches and submitted - received < window:
                    seeds, input_id = get_batch(submitted)
                    input_ids[submitted] = input_id
                    native.submit(submitted, seeds)
                    submitted += 1
                got = native.next_batch()
                if got is None:
                    raise RuntimeError(f"NeighborLoader backend stopped early: received {received} of "
                                       f"{num_batches} batches")
                batch_idx, sg, x = got
                received += 1
                input_id = torch.from_numpy(np.ascontiguousarray(input_ids.pop(batch_idx))).to(dev, non_blocking=True)
                seed_index = sg.seed_indices_t
                data = _make_data(
                    x=x, edge_index=sg.edge_index_local_t, e_id=sg.edge_ids_t if self._track_edge_ids else None,
                    n_id=sg.nodes_t, batch_size=int(seed_index.shape[0]), input_id=input_id, seed_index=seed_index,
                    num_nodes=sg.num_nodes, num_sampled_nodes=sg.num_sampled_nodes_per_hop,
                    num_sampled_edges=sg.num_sampled_edges_per_hop)
                if sg.batch is not None:  # disjoint batches: which seed's block a node belongs to (loader.py:985-991)
                    data.batch = torch.from_numpy(sg.batch).to(dev, non_blocking=True)
                if self._out_device is not None and torch.device(self._out_device).type != "cuda":
                    data = data.to(self._out_device)
                if self.transform is not None:
                    data = self.transform(data)
                yield data
        finally:
            stats = native.stats()
            native.shutdown()
            total = (time.perf_counter() - start) * 1000
            self._metrics = LoaderMetrics(batches_processed=received, total_time_ms=total,
                                          avg_batch_time_ms=total / received if received else 0.0,
                                          prefetch_hit_rate=stats.hit_rate, prefetch_hits=stats.hits,
                                          prefetch_misses=stats.misses)

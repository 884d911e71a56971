"""Epoch driver for heterogeneous graphs: the surface of the reference's
`aethergraph.pytorch.HeteroNeighborLoader`
(python/aethergraph/pytorch/hetero_loader.py:65-515) over the GPU sampler.

Same arguments, seed batching (`make_batch_getter`), per-epoch sampler seed and
per-batch reseed as the reference; every batch carries, per node type, `n_id`,
`num_nodes` and (when features were given) `x`; per edge type `edge_index`
(row 0 indexes the source type's `n_id`, row 1 the destination type's); and on
the seed type `batch_size`, `seed_index`, `input_id`.  All tensors are CUDA
tensors on the graph's device.  The batch object is a PyG `HeteroData` when
`torch_geometric` is installed and the attribute-compatible `HeteroBatch`
otherwise.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable, Iterator

import numpy as np

from ..features import FeatureStore
from ..hetero import HeteroCsrGraph, HeteroNeighborLoader as NativeHeteroLoader, HeteroSamplingConfig
from .loader import Batch, epoch_sampling_seed, make_batch_getter, normalize_input_nodes

__all__ = ["HeteroBatch", "HeteroLoaderMetrics", "HeteroNeighborLoader"]


class HeteroBatch:
    """`data[node_type]` / `data[src, rel, dst]` attribute stores, like PyG's HeteroData."""

    def __init__(self) -> None:
        self._stores: dict[Any, Batch] = {}

    def __getitem__(self, key) -> Batch:
        if key not in self._stores:
            self._stores[key] = Batch()
        return self._stores[key]

    @property
    def node_types(self) -> list[str]:
        return [k for k in self._stores if isinstance(k, str)]

    @property
    def edge_types(self) -> list[tuple]:
        return [k for k in self._stores if isinstance(k, tuple)]

    def to(self, device, non_blocking: bool = False) -> "HeteroBatch":
        out = HeteroBatch()
        out._stores = {k: v.to(device, non_blocking=non_blocking) for k, v in self._stores.items()}
        return out

    def __repr__(self) -> str:
        return "HeteroBatch(" + ", ".join(f"{k}: {v!r}" for k, v in self._stores.items()) + ")"


def _new_hetero_data():
    try:
        from torch_geometric.data import HeteroData  # type: ignore
    except ImportError:
        return HeteroBatch()
    return HeteroData()


@dataclass
class HeteroLoaderMetrics:
    """Counters of the most recent epoch (hetero_loader.py:45-63)."""

    batches_processed: int = 0
    total_time_ms: float = 0.0
    avg_batch_time_ms: float = 0.0
    _epoch_start: float = field(default=0.0, repr=False)

    def to_dict(self) -> dict[str, float | int]:
        return {"batches_processed": self.batches_processed, "total_time_ms": self.total_time_ms,
                "avg_batch_time_ms": self.avg_batch_time_ms}


class HeteroNeighborLoader:
    """Drop-in for `aethergraph.pytorch.HeteroNeighborLoader` on a GPU-resident
    `HeteroCsrGraph`.  `features` maps node types to a `FeatureStore` or a float32
    `[num_nodes(type), dim]` array (kept in GPU memory); `x` of a batch is gathered
    on the GPU from the batch's `n_id`."""

    def __init__(self, data: HeteroCsrGraph, num_neighbors: dict[tuple[str, str, str], list[int]],
                 input_nodes=None, batch_size: int = 128, shuffle: bool = True, replace: bool = False,
                 num_workers: int = 0, pin_memory: bool = False, device: str | None = None,
                 transfer_depth: int = 2, prefetch_factor: int = 2, seed: int | None = None,
                 max_degree: int | None = None, transform: Callable | None = None, features: dict | None = None):
        if num_workers < 0:
            raise ValueError(f"num_workers must be >= 0, got {num_workers}")
        if not num_neighbors:
            raise ValueError("num_neighbors must be a non-empty dict")
        hop_lens = {len(h) for h in num_neighbors.values()}
        if len(hop_lens) != 1:
            raise ValueError("all edge types in num_neighbors must have the same number of hops, "
                             f"got lengths {sorted(hop_lens)}")
        for et, hops in num_neighbors.items():
            if not hops:
                raise ValueError(f"num_neighbors[{et!r}] must be a non-empty list, got {hops!r}")
            if any(n < 0 for n in hops):
                raise ValueError(f"num_neighbors values must be non-negative, got {hops} for {et!r}")
        if max_degree is not None and max_degree <= 0:
            raise ValueError(f"max_degree must be > 0 if specified, got {max_degree}")
        if input_nodes is None:
            raise ValueError("input_nodes is required for HeteroNeighborLoader. Pass a (node_type, node_ids) tuple.")
        try:
            seed_type, node_ids = input_nodes
        except (TypeError, ValueError) as e:
            raise ValueError("input_nodes must be a (node_type, node_ids) tuple, "
                             f"got {type(input_nodes).__name__}") from e
        if not isinstance(data, HeteroCsrGraph):
            raise TypeError(f"data must be an aethergraph_b200 HeteroCsrGraph, got {type(data).__name__}")
        self.graph, self.num_neighbors = data, num_neighbors
        self.batch_size, self.shuffle, self.replace, self.pin_memory = batch_size, shuffle, replace, pin_memory
        self.prefetch_factor, self.transform = max(1, prefetch_factor), transform
        self._threads = max(1, num_workers)
        self._seed, self._max_degree, self._out_device = seed, max_degree, device
        self._node_types, self._edge_types = data.node_types(), data.edge_types()
        self._seed_type = seed_type
        self._stores: dict[str, FeatureStore] = {}
        for nt, f in (features or {}).items():
            if isinstance(f, FeatureStore):
                self._stores[nt] = f
                continue
            arr = np.asarray(f)
            if arr.dtype != np.float32:
                raise ValueError(f"features must be float32 (got {arr.dtype}); cast explicitly before passing")
            if arr.ndim != 2:
                raise ValueError(f"features must be 2D, got shape {arr.shape}")
            if arr.shape[0] != data.num_nodes(nt):
                raise ValueError(f"features.shape[0]={arr.shape[0]} does not match graph num_nodes={data.num_nodes(nt)}")
            self._stores[nt] = FeatureStore.from_array(np.ascontiguousarray(arr), dtype="f32", device=data.device)
        n_type = data.num_nodes(seed_type)
        if node_ids is None:
            self._input_nodes, self._num_input_nodes = None, n_type
        else:
            self._input_nodes = normalize_input_nodes(node_ids, num_nodes=n_type,
                                                      what=f"input_nodes for node type '{seed_type}'")
            self._num_input_nodes = len(self._input_nodes)
        self._rng = np.random.default_rng(seed)
        self._sampling_seeds = np.random.SeedSequence(seed) if seed is not None else None
        self._metrics = HeteroLoaderMetrics()

    @property
    def metrics(self) -> HeteroLoaderMetrics:
        return self._metrics

    def __len__(self) -> int:
        return (self._num_input_nodes + self.batch_size - 1) // self.batch_size

    def __repr__(self) -> str:
        return (f"HeteroNeighborLoader(seed_type='{self._seed_type}', num_input_nodes={self._num_input_nodes}, "
                f"num_neighbors=<{len(self.num_neighbors)} edge types>, batch_size={self.batch_size})")

    def __iter__(self) -> Iterator:
        import torch

        num_batches = len(self)
        rng = self._rng.spawn(1)[0]
        get_batch = make_batch_getter(self._input_nodes, self._num_input_nodes, self.batch_size, self.shuffle, rng)
        cfg = HeteroSamplingConfig(self.num_neighbors, replace=self.replace,
                                   seed=epoch_sampling_seed(self._sampling_seeds), max_degree=self._max_degree)
        native = NativeHeteroLoader(self.graph, cfg, self._seed_type, prefetch_depth=self.prefetch_factor,
                                    sampler_threads=self._threads, features=self._stores or None)
        dev = torch.device("cuda", self.graph.device)
        submitted = received = 0
        input_ids: dict[int, np.ndarray] = {}
        start = time.perf_counter()
        try:
            while received < num_batches:
                while submitted < num_batches and submitted - received < self.prefetch_factor:
                    seeds, input_id = get_batch(submitted)
                    input_ids[submitted] = input_id
                    native.submit(submitted, seeds)
                    submitted += 1
                got = native.next_batch()
                if got is None:
                    raise RuntimeError(f"hetero sampler stopped early: received {received} of {num_batches} batches")
                batch_idx, sg = got
                received += 1
                data = _new_hetero_data()
                for nt in self._node_types:
                    n_id = sg.nodes_t(nt)
                    store = data[nt]
                    store.n_id = n_id
                    store.num_nodes = int(n_id.shape[0])
                    if nt in self._stores:
                        store.x = sg.x_t(nt)  # gathered on the GPU in the sampling launch chain
                for et in self._edge_types:
                    data[et].edge_index = sg.edge_index_local_t(*et)
                seed_store = data[self._seed_type]
                seed_index = sg.seed_indices_t
                seed_store.batch_size = int(seed_index.shape[0])
                seed_store.seed_index = seed_index
                seed_store.input_id = torch.from_numpy(np.ascontiguousarray(input_ids.pop(batch_idx))).to(dev)
                if self._out_device is not None and torch.device(self._out_device).type != "cuda":
                    data = data.to(self._out_device)
                if self.transform is not None:
                    data = self.transform(data)
                yield data
        finally:
            native.shutdown()
            total = (time.perf_counter() - start) * 1000
            self._metrics = HeteroLoaderMetrics(batches_processed=received, total_time_ms=total,
                                                avg_batch_time_ms=total / received if received else 0.0)

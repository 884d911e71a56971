"""`CsrGraph` / `Graph`: a static CSR graph resident in GPU memory.

Mirrors the reference's `aethergraph._core.CsrGraph` (python/aethergraph/_core.pyi:68-131;
crates/aethergraph-py/src/graph.rs) for the methods the minibatch path uses.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Any

import numpy as np

from . import _lib
from ._ids import to_uint32_ids

__all__ = ["CsrGraph", "Graph", "partition_aligned_batches"]


def _current_device() -> int:
    import torch

    if not torch.cuda.is_available():
        raise RuntimeError("aethergraph_b200 needs a CUDA device; there is no CPU path")
    return torch.cuda.current_device()


class CsrGraph:
    """Compressed-sparse-row graph (u64 offsets, u32 destinations, optional f32
    weights) held in HBM.  Construct with `load`, `from_edges` or `from_csr`."""

    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)
        n, e, w, d = C.c_uint64(), C.c_uint64(), C.c_int32(), C.c_int32()
        _lib.check(_lib.lib().ag_graph_info(self._h, C.byref(n), C.byref(e), C.byref(w), C.byref(d)))
        self._n, self._e, self._w, self._device = n.value, e.value, bool(w.value), d.value

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _lib.lib().ag_graph_free(h)
            except Exception:
                pass
            self._h = None

    # -- constructors ------------------------------------------------------
    @staticmethod
    def load(path, *, storage: str = "auto", validation: str = "auto", device: int | None = None) -> "CsrGraph":
        """Load an AETH file (flat version 1, or the compressed version 2, which is decoded
        on the GPU and always fully validated) into GPU memory.

        `storage` is accepted for signature compatibility; the CSR always
        lives in HBM.  `validation` picks whether the body checksum is
        verified ("full", or "auto" below 512 MiB); destinations are always
        proven in range because the sampler indexes by them.
        """
        if storage not in ("auto", "mmap", "owned"):
            raise ValueError(f"Invalid storage '{storage}'. Must be 'auto', 'mmap', or 'owned'")
        if validation not in _lib.VALIDATION:
            raise ValueError(f"Invalid validation '{validation}'. Must be 'auto', 'header_only', "
                             "'offsets_only', or 'full'")
        dev = _current_device() if device is None else device
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_graph_load(os.fspath(path).encode(), _lib.VALIDATION[validation], dev,
                                            C.byref(out)))
        return CsrGraph(out.value)

    def load_features(self, path):
        """Load an AETHFEAT file into this graph's GPU and attach it: the store is
        returned and kept as `graph.features`, where `aethergraph_b200.pytorch.NeighborLoader`
        finds it when neither `features` nor `feature_path` is passed.  (The reference's
        README spells the workflow `graph = Graph.load(p); graph.load_features(f)`; its
        current loaders take the same file as `feature_path`, which works here too.)"""
        from .features import FeatureStore

        store = FeatureStore.load(os.fspath(path), device=self.device)
        if store.num_nodes < self.num_nodes:
            raise ValueError(f"feature file has {store.num_nodes} rows but the graph has {self.num_nodes} nodes")
        self.features = store
        return store

    @staticmethod
    def from_edges(num_nodes: int, src, dst, weights=None, *, device: int | None = None) -> "CsrGraph":
        """Build from an edge list; edges keep their input order within a row."""
        s = np.ascontiguousarray(to_uint32_ids(np.asarray(src), "src"))
        d = np.ascontiguousarray(to_uint32_ids(np.asarray(dst), "dst"))
        if s.shape != d.shape or s.ndim != 1:
            raise ValueError(f"src and dst must be 1-d arrays of equal length, got {s.shape} and {d.shape}")
        w = None
        if weights is not None:
            w = np.ascontiguousarray(weights, dtype=np.float32)
            if w.shape != s.shape:
                raise ValueError(f"weights length {w.shape} does not match the edge count {s.shape}")
        dev = _current_device() if device is None else device
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_graph_from_edges(num_nodes, s.ctypes.data, d.ctypes.data,
                                                  w.ctypes.data if w is not None else None, len(s), dev,
                                                  C.byref(out)))
        return CsrGraph(out.value)

    @staticmethod
    def from_csr(offsets, dst, weights=None, *, device: int | None = None) -> "CsrGraph":
        """Build from CSR arrays (numpy, or CUDA torch tensors of dtype int64 / int32 /
        float32 holding the u64 / u32 / f32 bit patterns)."""
        import torch

        dev = _current_device() if device is None else device
        out = C.c_void_p()
        if isinstance(offsets, torch.Tensor):
            if not (offsets.is_cuda and dst.is_cuda and offsets.is_contiguous() and dst.is_contiguous()):
                raise ValueError("tensor CSR arrays must be contiguous CUDA tensors")
            if offsets.dtype != torch.int64 or dst.dtype != torch.int32:
                raise ValueError("tensor CSR: offsets must be int64 and dst int32 (bit patterns of u64 / u32)")
            n, e = offsets.numel() - 1, dst.numel()
            wp = None
            if weights is not None:
                if weights.dtype != torch.float32 or not weights.is_cuda or weights.numel() != e:
                    raise ValueError("tensor CSR: weights must be a float32 CUDA tensor with one entry per edge")
                wp = weights.data_ptr()
            _lib.check(_lib.lib().ag_graph_from_csr(n, e, offsets.data_ptr(), dst.data_ptr() if e else None, wp,
                                                    _lib.AG_MEM_DEVICE, dev, C.byref(out)))
            return CsrGraph(out.value)
        off = np.ascontiguousarray(offsets, dtype=np.uint64)
        d = np.ascontiguousarray(dst, dtype=np.uint32)
        w = np.ascontiguousarray(weights, dtype=np.float32) if weights is not None else None
        _lib.check(_lib.lib().ag_graph_from_csr(len(off) - 1, len(d), off.ctypes.data, d.ctypes.data if len(d) else None,
                                                w.ctypes.data if w is not None else None, _lib.AG_MEM_HOST, dev,
                                                C.byref(out)))
        return CsrGraph(out.value)

    # -- locality reordering (python/aethergraph/_core.pyi:121-130) ----------
    def reorder_rabbit_with_partitions(self) -> tuple[np.ndarray, np.ndarray]:
        """`(perm, partitions)` of Rabbit Order community detection in one pass: `perm[new_id] =
        old_id` keeps every community of the dendrogram contiguous, `partitions[v]` is the dense
        id of v's top-level community.  Deterministic; the merge itself is sequential and runs on
        the host (crates/aethergraph-core/src/graph/reorder.rs:142-262)."""
        perm = np.empty(self._n, dtype=np.uint32)
        parts = np.empty(self._n, dtype=np.uint32)
        _lib.check(_lib.lib().ag_graph_rabbit_order(self._h, perm.ctypes.data if self._n else None,
                                                    parts.ctypes.data if self._n else None))
        return perm, parts

    def reorder_rabbit(self) -> np.ndarray:
        return self.reorder_rabbit_with_partitions()[0]

    def rabbit_partitions(self) -> np.ndarray:
        return self.reorder_rabbit_with_partitions()[1]

    def permute(self, perm) -> "CsrGraph":
        """The graph relabelled by `perm[new_id] = old_id`, built on the GPU; rows keep their
        edge order and weights (reorder.rs:297-383)."""
        p = np.ascontiguousarray(perm)
        if p.ndim != 1 or p.dtype.kind not in "iu" or (p.size and (p.min() < 0 or p.max() > 0xFFFFFFFF)):
            raise ValueError("perm must be a 1-D array of node ids")
        p = p.astype(np.uint32, copy=False)
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_graph_permute(self._h, p.ctypes.data if p.size else None, p.size, C.byref(out)))
        return CsrGraph(out.value)

    def save(self, path, *, compressed: bool = False) -> None:
        """Write the graph: the flat AETH v1 file, or with `compressed=True` the succinct-coded
        version 2 (Elias-Fano offsets, StreamVByte edge deltas; python/aethergraph/_core.pyi:95-99).
        `Graph.load` reads either."""
        fn = _lib.lib().ag_graph_save_compressed if compressed else _lib.lib().ag_graph_save
        _lib.check(fn(self._h, os.fspath(path).encode()))

    # -- properties --------------------------------------------------------
    @property
    def num_nodes(self) -> int:
        return self._n

    @property
    def num_edges(self) -> int:
        return self._e

    @property
    def has_weights(self) -> bool:
        return self._w

    @property
    def has_timestamps(self) -> bool:
        return False

    @property
    def device(self) -> int:
        return self._device

    def device_ptrs(self) -> tuple[int, int, int]:
        """(offsets, destinations, weights) device addresses; weights is 0 if absent."""
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _lib.check(_lib.lib().ag_graph_device_ptrs(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value or 0, b.value or 0, c.value or 0

    def to_host(self):
        """(offsets u64, destinations u32, weights f32 | None) copied back to host numpy arrays."""
        off = np.empty(self._n + 1, dtype=np.uint64)
        dst = np.empty(self._e, dtype=np.uint32)
        w = np.empty(self._e, dtype=np.float32) if self._w else None
        _lib.check(_lib.lib().ag_graph_copy_to_host(self._h, off.ctypes.data, dst.ctypes.data if self._e else None,
                                                    w.ctypes.data if (w is not None and self._e) else None))
        return off, dst, w

    # -- row access --------------------------------------------------------
    def degrees(self) -> np.ndarray:
        out = np.empty(self._n, dtype=np.uint32)
        _lib.check(_lib.lib().ag_graph_degrees(self._h, None, self._n, out.ctypes.data))
        return out

    def degrees_of(self, nodes) -> np.ndarray:
        ids = np.ascontiguousarray(to_uint32_ids(np.asarray(nodes), "nodes"))
        out = np.empty(len(ids), dtype=np.uint32)
        _lib.check(_lib.lib().ag_graph_degrees(self._h, ids.ctypes.data, len(ids), out.ctypes.data))
        return out

    def degree(self, node: int) -> int:
        if node < 0 or node >= self._n:
            return 0
        return int(self.degrees_of(np.array([node], dtype=np.uint32))[0])

    def _row(self, node: int, want_weights: bool):
        if node < 0 or node >= 2**32:
            return np.empty(0, dtype=np.uint32), (np.empty(0, dtype=np.float32) if want_weights else None)
        deg = C.c_uint64()
        _lib.check(_lib.lib().ag_graph_neighbors(self._h, node, None, None, 0, C.byref(deg)))
        out = np.empty(deg.value, dtype=np.uint32)
        w = np.empty(deg.value, dtype=np.float32) if (want_weights and self._w) else None
        if deg.value:
            _lib.check(_lib.lib().ag_graph_neighbors(self._h, node, out.ctypes.data,
                                                     w.ctypes.data if w is not None else None, deg.value,
                                                     C.byref(deg)))
        return out, w

    def neighbors(self, node: int) -> np.ndarray:
        return self._row(int(node), False)[0]

    def neighbor_weights(self, node: int):
        if not self._w:
            return None
        return self._row(int(node), True)[1]

    def batch_neighbors(self, nodes) -> list[np.ndarray]:
        return [self.neighbors(int(v)) for v in nodes]

    def stats(self) -> dict[str, Any]:
        deg = self.degrees()
        return {
            "num_nodes": self._n, "num_edges": self._e,
            "avg_degree": float(self._e) / self._n if self._n else 0.0,
            "max_degree": int(deg.max()) if self._n else 0,
            "min_degree": int(deg.min()) if self._n else 0,
            "has_weights": self._w,
        }

    def __len__(self) -> int:
        return self._n

    def __getitem__(self, node: int) -> np.ndarray:
        return self.neighbors(node)

    def __repr__(self) -> str:
        return f"CsrGraph(num_nodes={self._n}, num_edges={self._e}, device=cuda:{self._device})"


Graph = CsrGraph


def partition_aligned_batches(partitions, seeds, batch_size: int, shuffle_partitions: bool = False,
                              seed: int = 0) -> list[np.ndarray]:
    """Seed batches that follow the Rabbit partitions: seeds of one community land in the
    same batch, so their sampled neighbourhoods (and feature rows, on a reordered graph)
    overlap.  Seeds are grouped by partition, keeping their order inside one; the partitions
    are visited in id order, or shuffled by the reference's LCG Fisher-Yates; batches of
    `batch_size` are cut from that sequence (crates/aethergraph-core/src/graph/reorder.rs:385-463)."""
    if batch_size < 1:
        raise ValueError("batch_size must be >= 1")
    parts = np.ascontiguousarray(partitions, dtype=np.uint32)
    s = np.ascontiguousarray(seeds).astype(np.int64, copy=False)
    if s.size and (s.min() < 0 or s.max() >= parts.size):
        bad = int(s[(s < 0) | (s >= parts.size)][0])
        raise ValueError(f"seed {bad} is out of range for partitions of length {parts.size}")
    keyed = np.sort((parts[s].astype(np.uint64) << np.uint64(32)) | np.arange(s.size, dtype=np.uint64))
    run_id = keyed >> np.uint64(32)
    starts = np.flatnonzero(np.concatenate([[True], run_id[1:] != run_id[:-1]])) if s.size else np.zeros(0, np.int64)
    ends = np.concatenate([starts[1:], [s.size]]) if s.size else np.zeros(0, np.int64)
    runs = list(zip(starts.tolist(), ends.tolist()))
    if shuffle_partitions:
        mask, mul = (1 << 64) - 1, 0x517CC1B727220A95
        rng = (seed * mul + 1) & mask
        for i in range(len(runs) - 1, 0, -1):
            rng = (rng * mul + 1) & mask
            j = (rng >> 33) % (i + 1)
            runs[i], runs[j] = runs[j], runs[i]
    order = np.concatenate([keyed[a:b] for a, b in runs]) if runs else np.zeros(0, np.uint64)
    picked = s[(order & np.uint64(0xFFFFFFFF)).astype(np.int64)].astype(np.uint32)
    return [picked[i:i + batch_size] for i in range(0, picked.size, batch_size)]

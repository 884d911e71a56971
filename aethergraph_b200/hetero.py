"""Heterogeneous neighbor sampling on the GPU behind the reference's API.

Mirrors `HeteroCsrGraph`, `HeteroSamplingConfig`, `HeteroSampledSubgraph`,
`HeteroNeighborSampler` and `HeteroNeighborLoader`
(python/aethergraph/_core.pyi:609-720, crates/aethergraph-py/src/hetero.rs).
The transposed adjacency is built and kept in GPU memory; sampling, per-type
dedup, relabel and the int64 widening run in CUDA kernels.  For the same seed
the arrays are the reference CPU sampler's, bit for bit.
"""
from __future__ import annotations

import ctypes as C
import secrets
import threading
from typing import Sequence

import numpy as np

from . import _lib
from ._lib import SamplingError
from .loader import _FETCH, PrefetchStats, _raw_current_stream
from .sampler import _DevArray, coerce_seeds

__all__ = ["HeteroCsrGraph", "HeteroNeighborLoader", "HeteroNeighborSampler", "HeteroSampledSubgraph",
           "HeteroSamplingConfig"]

EdgeType = tuple[str, str, str]


def _ptr_array(arrays: Sequence[np.ndarray | None]):
    out = (C.c_void_p * max(len(arrays), 1))()
    for i, a in enumerate(arrays):
        out[i] = a.ctypes.data if a is not None and a.size else None
    return out


class HeteroCsrGraph:
    """Heterogeneous graph: several node types and edge types, resident in GPU memory
    as one transposed adjacency per edge type (crates/aethergraph-core/src/graph/hetero.rs:70-97)."""

    def __init__(self, handle: int, node_types: list[tuple[str, int]], edge_types: list[EdgeType],
                 num_edges: list[int], device: int):
        self._h = handle
        self._node_types = node_types
        self._edge_types = edge_types
        self._num_edges = num_edges
        self.device = device
        self._nt_id = {name: i for i, (name, _) in enumerate(node_types)}
        self._et_id = {et: i for i, et in enumerate(edge_types)}

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.lib().ag_hetero_free(h)
            except Exception:
                pass

    @staticmethod
    def from_edge_arrays(node_types: dict[str, int], edge_types: list[tuple], device: int | None = None) -> "HeteroCsrGraph":
        """Build from per-edge-type COO arrays `(src_type, rel, dst_type, src_ids, dst_ids)`.

        Raises ValueError for mismatched array lengths, an unknown node type, an
        endpoint outside its type's node count or a repeated edge type
        (crates/aethergraph-py/src/hetero.rs:56-134), and for more node / edge
        types than the GPU sampler supports (8 / 16)."""
        import torch

        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        nt = [(str(k), int(v)) for k, v in node_types.items()]
        nt_id = {name: i for i, (name, _) in enumerate(nt)}
        names: list[EdgeType] = []
        src_t, dst_t, srcs, dsts = [], [], [], []
        for (s, rel, d, src_ids, dst_ids) in edge_types:
            a = np.ascontiguousarray(np.asarray(src_ids), dtype=np.uint32).reshape(-1)
            b = np.ascontiguousarray(np.asarray(dst_ids), dtype=np.uint32).reshape(-1)
            if a.size != b.size:
                raise ValueError(f"src and dst arrays must have the same length for ({s}, {rel}, {d})")
            if s not in nt_id:
                raise ValueError(f"unknown source type '{s}' in ({s}, {rel}, {d})")
            if d not in nt_id:
                raise ValueError(f"unknown dest type '{d}' in ({s}, {rel}, {d})")
            if (s, rel, d) in names:
                raise ValueError(f"duplicate edge type ({s}, {rel}, {d})")
            names.append((s, rel, d))
            src_t.append(nt_id[s]); dst_t.append(nt_id[d]); srcs.append(a); dsts.append(b)
        for (s, rel, d), a, b, si, di in zip(names, srcs, dsts, src_t, dst_t):
            # the reference's bipartite builder names the relation in its error
            if a.size and (int(a.max()) >= nt[si][1] or int(b.max()) >= nt[di][1]):
                raise ValueError(f"failed to build CSR for ({s}, {rel}, {d}): endpoint outside the node range")
        num_nodes = np.array([c for _, c in nt], dtype=np.uint64)
        st = np.array(src_t, dtype=np.uint32)
        dt = np.array(dst_t, dtype=np.uint32)
        ne = np.array([a.size for a in srcs], dtype=np.uint64)
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_hetero_create(len(nt), num_nodes.ctypes.data, len(names), st.ctypes.data,
                                               dt.ctypes.data, None, _ptr_array(srcs), _ptr_array(dsts),
                                               ne.ctypes.data, _lib.AG_MEM_HOST, device, C.byref(out)))
        return HeteroCsrGraph(out.value, nt, names, [int(v) for v in ne], device)

    @staticmethod
    def load(path, device: int | None = None) -> "HeteroCsrGraph":
        """Load an AETHHETG v1 file (crates/aethergraph-core/src/internal/mmap_hetero.rs:1-45)
        into GPU memory.  Every relation is validated in full; a malformed file raises
        GraphLoadError."""
        import os

        import torch

        if device is None:
            device = torch.cuda.current_device() if torch.cuda.is_available() else 0
        out, names = C.c_void_p(), _lib.HeteroNames()
        _lib.check(_lib.lib().ag_hetero_load(os.fspath(path).encode(), device, C.byref(out), C.byref(names)))
        nt_n, et_n = names.num_node_types, names.num_edge_types
        counts = (C.c_uint64 * _lib.AG_MAX_NODE_TYPES)()
        edges = (C.c_uint64 * _lib.AG_MAX_EDGE_TYPES)()
        _lib.check(_lib.lib().ag_hetero_info(out, None, None, counts, edges, None))
        nt = [(names.node_type[t].value.decode(), int(counts[t])) for t in range(nt_n)]
        ets = [(names.src[e].value.decode(), names.rel[e].value.decode(), names.dst[e].value.decode()) for e in range(et_n)]
        return HeteroCsrGraph(out.value, nt, ets, [int(edges[e]) for e in range(et_n)], device)

    def save(self, path) -> None:
        """Write the graph as an AETHHETG v1 file, atomically.  Rows of the stored forward
        CSR are sorted by destination id (the sampler never observes the order within a
        forward row: it walks the transposed adjacency)."""
        import os

        names = _lib.HeteroNames()
        names.num_node_types, names.num_edge_types = len(self._node_types), len(self._edge_types)
        for t, (name, _) in enumerate(self._node_types):
            b = name.encode()
            if len(b) >= 64:
                raise ValueError(f"type name too long: {name}")
            names.node_type[t].value = b
        for e, (s, rel, d) in enumerate(self._edge_types):
            for field, text in ((names.src, s), (names.rel, rel), (names.dst, d)):
                b = text.encode()
                if len(b) >= 64:
                    raise ValueError(f"type name too long: {text}")
                field[e].value = b
        _lib.check(_lib.lib().ag_hetero_save(self._h, C.byref(names), os.fspath(path).encode()))

    @staticmethod
    def from_device_edges(node_types: dict[str, int], edge_types: list[tuple], device: int | None = None) -> "HeteroCsrGraph":
        """Like `from_edge_arrays` with the COO arrays already in GPU memory: every
        `src_ids` / `dst_ids` is a contiguous int32 CUDA tensor holding u32 ids."""
        import torch

        if device is None:
            device = torch.cuda.current_device()
        nt = [(str(k), int(v)) for k, v in node_types.items()]
        nt_id = {name: i for i, (name, _) in enumerate(nt)}
        names, src_t, dst_t, srcs, dsts = [], [], [], [], []
        for (s, rel, d, a, b) in edge_types:
            if s not in nt_id or d not in nt_id:
                raise ValueError(f"unknown node type in ({s}, {rel}, {d})")
            if (s, rel, d) in names:
                raise ValueError(f"duplicate edge type ({s}, {rel}, {d})")
            for t in (a, b):
                if not (t.is_cuda and t.is_contiguous() and t.dtype == torch.int32 and t.dim() == 1):
                    raise ValueError("edge arrays must be contiguous 1-d int32 CUDA tensors")
            if a.numel() != b.numel():
                raise ValueError(f"src and dst arrays must have the same length for ({s}, {rel}, {d})")
            names.append((s, rel, d)); src_t.append(nt_id[s]); dst_t.append(nt_id[d]); srcs.append(a); dsts.append(b)
        num_nodes = np.array([c for _, c in nt], dtype=np.uint64)
        st, dt = np.array(src_t, dtype=np.uint32), np.array(dst_t, dtype=np.uint32)
        ne = np.array([a.numel() for a in srcs], dtype=np.uint64)
        pa = (C.c_void_p * max(len(srcs), 1))(*[a.data_ptr() if a.numel() else None for a in srcs])
        pb = (C.c_void_p * max(len(dsts), 1))(*[b.data_ptr() if b.numel() else None for b in dsts])
        out = C.c_void_p()
        torch.cuda.synchronize(device)
        _lib.check(_lib.lib().ag_hetero_create(len(nt), num_nodes.ctypes.data, len(names), st.ctypes.data, dt.ctypes.data,
                                               None, pa, pb, ne.ctypes.data, _lib.AG_MEM_DEVICE, device, C.byref(out)))
        return HeteroCsrGraph(out.value, nt, names, [int(v) for v in ne], device)

    def node_types(self) -> list[str]:
        return [n for n, _ in self._node_types]

    def edge_types(self) -> list[EdgeType]:
        return list(self._edge_types)

    def num_nodes(self, node_type: str) -> int:
        if node_type not in self._nt_id:
            raise KeyError(f"unknown node type '{node_type}'")
        return self._node_types[self._nt_id[node_type]][1]

    def num_edges(self, src_type: str, rel: str, dst_type: str) -> int:
        if (src_type, rel, dst_type) not in self._et_id:
            raise KeyError(f"unknown edge type ('{src_type}', '{rel}', '{dst_type}')")
        return self._num_edges[self._et_id[(src_type, rel, dst_type)]]

    def total_nodes(self) -> int:
        return sum(c for _, c in self._node_types)

    def total_edges(self) -> int:
        return sum(self._num_edges)

    def in_adjacency(self, src_type: str, rel: str, dst_type: str) -> tuple[np.ndarray, np.ndarray]:
        """Host copy of the transposed adjacency of one edge type: `(offsets, sources)`
        over the destination type's nodes."""
        if (src_type, rel, dst_type) not in self._et_id:
            raise KeyError(f"unknown edge type ('{src_type}', '{rel}', '{dst_type}')")
        e = self._et_id[(src_type, rel, dst_type)]
        offsets = np.zeros(self.num_nodes(dst_type) + 1, dtype=np.uint64)
        sources = np.zeros(self._num_edges[e], dtype=np.uint32)
        _lib.check(_lib.lib().ag_hetero_in_adjacency(self._h, e, offsets.ctypes.data,
                                                     sources.ctypes.data if sources.size else None))
        return offsets, sources

    def __repr__(self) -> str:
        return (f"HeteroCsrGraph(node_types={len(self._node_types)}, edge_types={len(self._edge_types)}, "
                f"total_nodes={self.total_nodes()}, total_edges={self.total_edges()})")


class HeteroSamplingConfig:
    """`num_neighbors[(src, rel, dst)]` is, per hop, how many `src` nodes with an
    edge into each expanded `dst` node to draw; edge types left out draw nothing.
    `max_degree` has no effect (crates/aethergraph-py/src/hetero.rs:209-262)."""

    def __init__(self, num_neighbors: dict[EdgeType, list[int]], replace: bool = False, seed: int | None = None,
                 max_degree: int | None = None, rng_mode: str = "wyrand_exact"):
        if not num_neighbors:
            raise ValueError("num_neighbors must not be empty")
        hops = [len(v) for v in num_neighbors.values()]
        if hops[0] == 0:
            raise ValueError("num_neighbors hop lists must be non-empty")
        if any(h != hops[0] for h in hops):
            raise ValueError("all edge types must have the same number of hops")
        if max_degree is not None and max_degree == 0:
            raise ValueError("max_degree must be > 0 if specified")
        if seed is not None and not (0 <= int(seed) < 2**64):
            raise ValueError(f"seed must fit an unsigned 64-bit integer, got {seed}")
        if rng_mode not in _lib.RNG_MODE:
            raise ValueError(f"Invalid rng_mode '{rng_mode}'. Must be 'wyrand_exact' or 'philox'")
        self._nn = {tuple(k): [int(x) for x in v] for k, v in num_neighbors.items()}
        if any(x < 0 for v in self._nn.values() for x in v):
            raise ValueError("num_neighbors values must be non-negative")
        self._replace, self._seed, self._max_degree, self.rng_mode = bool(replace), seed, max_degree, rng_mode

    num_neighbors = property(lambda self: {k: list(v) for k, v in self._nn.items()})
    replace = property(lambda self: self._replace)
    seed = property(lambda self: self._seed)
    max_degree = property(lambda self: self._max_degree)
    num_hops = property(lambda self: len(next(iter(self._nn.values()))))

    def _fanout(self, graph: HeteroCsrGraph) -> np.ndarray:
        """[edge types][hops], zeros for edge types left out (hetero.rs:309-328)."""
        f = np.zeros((len(graph._edge_types), self.num_hops), dtype=np.uint32)
        for et, hops in self._nn.items():
            if et not in graph._et_id:
                raise SamplingError(f"unknown edge type ('{et[0]}', '{et[1]}', '{et[2]}')")
            f[graph._et_id[et]] = hops
        return f

    def __repr__(self) -> str:
        return f"HeteroSamplingConfig(edge_types={len(self._nn)}, num_hops={self.num_hops}, replace={self._replace})"


class HeteroSampledSubgraph:
    """One heterogeneous batch.  The arrays live in GPU memory; `*_t` accessors
    return CUDA tensors over it without a copy, the reference's accessors
    (`nodes`, `nodes_u32`, `edge_index_local`, `seeds`, `seed_indices`) return
    fresh host numpy arrays (crates/aethergraph-py/src/hetero.rs:349-470)."""

    def __init__(self, graph: HeteroCsrGraph, seed_type: int, seeds: np.ndarray, counts: _lib.HeteroCounts,
                 bufs: _lib.HeteroBuffers, owner, dims=None):
        self._g, self._seed_type, self._seeds, self._c, self._b, self._owner = graph, seed_type, seeds, counts, bufs, owner
        self._dims = dims or [0] * len(graph._node_types)
        self._x_override: dict[int, object] = {}
        self._n = list(counts.nodes[:len(graph._node_types)])
        self._e = list(counts.edges[:len(graph._edge_types)])
        self._n_start, self._e_start = [0], [0]  # segment starts: prefix sums of the per-type counts
        for v in self._n:
            self._n_start.append(self._n_start[-1] + v)
        for v in self._e:
            self._e_start.append(self._e_start[-1] + v)

    # -- reference API ------------------------------------------------------
    @property
    def node_types(self) -> list[str]:
        return [name for (name, _), n in zip(self._g._node_types, self._n) if n]

    @property
    def edge_types(self) -> list[EdgeType]:
        return [et for et, n in zip(self._g._edge_types, self._e) if n]

    @property
    def seed_type(self) -> str:
        return self._g._node_types[self._seed_type][0]

    @property
    def seeds(self) -> np.ndarray:
        return self._seeds.astype(np.int64)

    @property
    def seed_indices(self) -> np.ndarray:
        return self.seed_indices_t.cpu().numpy()

    def nodes(self, node_type: str) -> np.ndarray:
        return self.nodes_t(node_type).cpu().numpy()

    def nodes_u32(self, node_type: str) -> np.ndarray:
        import torch

        t = self._nt(node_type)
        v = torch.as_tensor(_DevArray(self._b.nodes + 4 * int(self._n_start[t]), (self._n[t],), "<i4", self._owner),
                            device=self._dev()) if self._n[t] else torch.empty(0, dtype=torch.int32)
        return v.cpu().numpy().view(np.uint32)

    def edge_index_local(self, src: str, rel: str, dst: str) -> np.ndarray:
        return self.edge_index_local_t(src, rel, dst).cpu().numpy()

    # -- device views -------------------------------------------------------
    def _dev(self):
        import torch

        return torch.device("cuda", self._g.device)

    def _nt(self, node_type: str) -> int:
        if node_type not in self._g._nt_id:
            raise KeyError(f"unknown node type '{node_type}'")
        return self._g._nt_id[node_type]

    def nodes_t(self, node_type: str):
        """int64 CUDA tensor of the sampled ids of `node_type`, in discovery order."""
        import torch

        t = self._nt(node_type)
        if not self._n[t]:
            return torch.empty(0, dtype=torch.int64, device=self._dev())
        return torch.as_tensor(_DevArray(self._b.n_id + 8 * int(self._n_start[t]), (self._n[t],), "<i8", self._owner),
                               device=self._dev())

    def x_t(self, node_type: str):
        """float32 CUDA tensor [num nodes of the type, dim]: the feature rows of
        `nodes(node_type)`, gathered in the sampling launch chain; None when the
        sampler was built without a feature store for this type."""
        import torch

        t = self._nt(node_type)
        if t in self._x_override:
            return self._x_override[t]
        if not self._dims[t] or not self._b.x[t]:
            return None
        if not self._n[t]:
            return torch.empty((0, self._dims[t]), dtype=torch.float32, device=self._dev())
        return torch.as_tensor(_DevArray(self._b.x[t], (self._n[t], self._dims[t]), "<f4", self._owner), device=self._dev())

    def edge_index_local_t(self, src: str, rel: str, dst: str):
        """int64 CUDA tensor [2, E]: row 0 indexes `nodes(src)`, row 1 `nodes(dst)`."""
        import torch

        if (src, rel, dst) not in self._g._et_id:
            raise KeyError(f"unknown edge type ('{src}', '{rel}', '{dst}')")
        e = self._g._et_id[(src, rel, dst)]
        if not self._e[e]:
            return torch.empty((2, 0), dtype=torch.int64, device=self._dev())
        return torch.as_tensor(_DevArray(self._b.edge_index_local + 16 * int(self._e_start[e]), (2, self._e[e]), "<i8",
                                         self._owner), device=self._dev())

    @property
    def seed_indices_t(self):
        import torch

        n = int(self._c.num_seeds)
        if not n:
            return torch.empty(0, dtype=torch.int64, device=self._dev())
        return torch.as_tensor(_DevArray(self._b.seed_index, (n,), "<i8", self._owner), device=self._dev())

    def raw_u32(self) -> dict:
        """The u32 arrays the C ABI wrote, per type, as host numpy (parity tests)."""
        import torch

        def u32(ptr, start, n):
            if not n:
                return np.zeros(0, dtype=np.uint32)
            t = torch.as_tensor(_DevArray(ptr + 4 * int(start), (n,), "<i4", self._owner), device=self._dev())
            return t.cpu().numpy().view(np.uint32)

        return {
            "nodes": [u32(self._b.nodes, self._n_start[t], self._n[t]) for t in range(len(self._n))],
            "edge_src_local": [u32(self._b.edge_src_local, self._e_start[e], self._e[e]) for e in range(len(self._e))],
            "edge_dst_local": [u32(self._b.edge_dst_local, self._e_start[e], self._e[e]) for e in range(len(self._e))],
            "seed_indices": u32(self._b.seed_indices, 0, int(self._c.num_seeds)),
            "draws": int(self._c.draws),
        }

    def __repr__(self) -> str:
        return (f"HeteroSampledSubgraph(node_types={len(self.node_types)}, edge_types={len(self.edge_types)}, "
                f"seed_type='{self.seed_type}')")


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class _HeteroHandle:
    """One native hetero sampler handle (scratch for `group` batches per launch
    chain) plus the allocation of its output buffers."""

    def __init__(self, graph: HeteroCsrGraph, config: HeteroSamplingConfig, seed: int, group: int = 1,
                 features: dict | None = None):
        self.graph, self.config, self.group = graph, config, max(1, int(group))
        fan = np.ascontiguousarray(config._fanout(graph))
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_hetero_sampler_create_group(graph._h, fan.ctypes.data, config.num_hops,
                                                             int(config.replace), seed, _lib.RNG_MODE[config.rng_mode],
                                                             self.group, C.byref(out)))
        self._h = out.value
        # per node type: the feature store whose rows ride along as x, or None
        self._stores = [None] * len(graph._node_types)
        for name, store in (features or {}).items():
            if name not in graph._nt_id:
                raise KeyError(f"unknown node type '{name}'")
            self._stores[graph._nt_id[name]] = store
        self._feat_ptrs = None
        if any(st is not None for st in self._stores):
            self._feat_ptrs = (C.c_void_p * len(self._stores))(*[st._h if st is not None else None for st in self._stores])
        self._bounds: dict[int, tuple[int, int]] = {}
        # rows of x reserved per node type: the worst-case bound until batches have been
        # seen, then 1.5 x the largest count observed (a batch that outgrows it is
        # gathered again at its exact size)
        self._x_rows: list[int | None] = [None] * len(self._stores)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib.lib().ag_hetero_sampler_free(h)
            except Exception:
                pass

    def reseed(self, seed: int) -> None:
        _lib.check(_lib.lib().ag_hetero_sampler_reseed(self._h, seed))

    def _bound(self, n: int) -> tuple[int, int]:
        if n not in self._bounds:
            mn, me = C.c_uint64(), C.c_uint64()
            _lib.check(_lib.lib().ag_hetero_sampler_bounds(self._h, n, C.byref(mn), C.byref(me)))
            self._bounds[n] = (max(int(mn.value), 1), max(int(me.value), 1))
        return self._bounds[n]

    def sample_group(self, seed_type: int, seeds: list[np.ndarray], batch_seeds: list[int] | None, stream=None,
                     return_errors: bool = False) -> list:
        """One launch chain for up to `group` batches; returns one HeteroSampledSubgraph per batch."""
        import torch

        L = _lib.lib()
        nb = len(seeds)
        dev = torch.device("cuda", self.graph.device)
        dims = [st.feature_dim if st is not None else 0 for st in self._stores]
        layouts, total = [], 0
        for sd in seeds:
            n = int(sd.size)
            cap_n, cap_e = self._bound(n)
            cap_s = max(n, 1)
            sizes = [4 * cap_n, 4 * cap_e, 4 * cap_e, 4 * cap_s, 8 * cap_n, 16 * cap_e, 8 * cap_s]
            x_caps = [min(cap_n, self.graph._node_types[t][1], self._x_rows[t] or cap_n) if d else 0
                      for t, d in enumerate(dims)]
            sizes += [4 * c * d for c, d in zip(x_caps, dims)]
            offs = []
            for sz in sizes:
                offs.append(total)
                total += _align(sz)
            layouts.append((cap_n, cap_e, cap_s, offs, x_caps))
        block = torch.empty(max(total, 1), dtype=torch.uint8, device=dev)
        base = block.data_ptr()
        bufs = (_lib.HeteroBuffers * nb)()
        for i, (cap_n, cap_e, cap_s, offs, x_caps) in enumerate(layouts):
            b = bufs[i]
            b.cap_nodes, b.cap_edges, b.cap_seeds = cap_n, cap_e, cap_s
            (b.nodes, b.edge_src_local, b.edge_dst_local, b.seed_indices, b.n_id, b.edge_index_local,
             b.seed_index) = (base + o for o in offs[:7])
            for t, d in enumerate(dims):
                b.x[t] = base + offs[7 + t] if d else None
                b.cap_x[t] = x_caps[t]
        ptrs = (C.c_void_p * nb)(*[sd.ctypes.data if sd.size else None for sd in seeds])
        lens = (C.c_uint64 * nb)(*[int(sd.size) for sd in seeds])
        bseeds = (C.c_uint64 * nb)(*batch_seeds) if batch_seeds is not None else None
        st = stream if stream is not None else torch.cuda.current_stream(dev)
        _lib.check(L.ag_hetero_sample_group_into(self._h, nb, seed_type, ptrs, lens, bseeds, self._feat_ptrs, bufs,
                                                 st.cuda_stream))
        counts = (_lib.HeteroCounts * nb)()
        statuses = (C.c_int32 * nb)()
        rc = L.ag_hetero_sample_group_wait(self._h, counts, statuses)
        if rc != _lib.AG_OK and not return_errors:
            _lib.check(rc)
        out = []
        for i in range(nb):
            cb = _lib.HeteroBuffers.from_buffer_copy(bufs[i])
            cc = _lib.HeteroCounts.from_buffer_copy(counts[i])
            sg = HeteroSampledSubgraph(self.graph, seed_type, seeds[i], cc, cb, block, dims)
            for t, d in enumerate(dims):
                if not d:
                    continue
                n_t = int(cc.nodes[t])
                if n_t > layouts[i][4][t]:  # outgrew the reserved rows: gather this type again, exactly
                    sg._x_override[t] = self._stores[t].gather(sg.nodes_t(self.graph._node_types[t][0]))
                self._x_rows[t] = max(self._x_rows[t] or 0, n_t + n_t // 2 + 1024)
            out.append(sg)
        return (out, list(statuses), _lib.last_error() if rc != _lib.AG_OK else "") if return_errors else out

    def sample(self, seed_type: int, seeds: np.ndarray, stream=None) -> HeteroSampledSubgraph:
        return self.sample_group(seed_type, [seeds], None, stream)[0]


class HeteroNeighborSampler:
    """Heterogeneous neighborhood sampler; `sample` raises SamplingError for an
    unknown seed type or a seed outside the seed type's node range
    (crates/aethergraph-py/src/hetero.rs:544-581)."""

    def __init__(self, graph: HeteroCsrGraph, config: HeteroSamplingConfig, features: dict | None = None):
        self._graph = graph
        seed = config.seed if config.seed is not None else secrets.randbits(64)
        self._handle = _HeteroHandle(graph, config, int(seed), 1, features)

    def sample(self, seed_type: str, seeds) -> HeteroSampledSubgraph:
        if seed_type not in self._graph._nt_id:
            raise SamplingError(f"unknown seed type '{seed_type}'")
        t = self._graph._nt_id[seed_type]
        return self._handle.sample(t, coerce_seeds(seeds, self._graph._node_types[t][1]))

    def __repr__(self) -> str:
        return f"HeteroNeighborSampler(edge_types={len(self._graph._edge_types)})"


class _HeteroLease:
    """Holds one pooled heterogeneous batch; hands it back to the loader when nothing
    refers to it any more, recording the consumer's current stream as its last use."""

    __slots__ = ("loader", "batch")

    def __init__(self, loader: "HeteroNeighborLoader", batch: _lib.HeteroBatch):
        self.loader, self.batch = loader, batch

    def __del__(self):
        ld = self.loader
        if ld is None or not ld._h:
            return
        try:
            ld._release(ld._h, C.byref(self.batch), _raw_current_stream(ld._dev_index))
        except Exception:
            pass


class HeteroNeighborLoader:
    """Prefetching heterogeneous loader over the native worker pool: `sampler_threads`
    host threads, each with its own sampler handle and CUDA stream, run up to `group`
    queued batches as one launch chain; the same ordering, per-batch reseed
    (`batch_seed(seed, seq)` when the config has a seed), timeout and shutdown
    contract as `NeighborLoader`
    (crates/aethergraph-core/src/loader/prefetch.rs:984-1022, 1940-2060)."""

    def __init__(self, graph: HeteroCsrGraph, config: HeteroSamplingConfig, seed_type: str, prefetch_depth: int = 2,
                 sampler_threads: int = 1, *, features: dict | None = None, group: int = 8):
        if prefetch_depth < 1:
            raise RuntimeError("Failed to create HeteroNeighborLoader: prefetch_depth must be >= 1")
        if seed_type not in graph._nt_id:
            raise SamplingError(f"unknown seed type '{seed_type}'")
        self._graph, self._config = graph, config
        self._seed_type = graph._nt_id[seed_type]
        self._seed_nodes = graph._node_types[self._seed_type][1]
        self._depth = prefetch_depth
        self._seeded = config.seed is not None
        self._stores = [None] * len(graph._node_types)
        for name, store in (features or {}).items():
            if name not in graph._nt_id:
                raise KeyError(f"unknown node type '{name}'")
            self._stores[graph._nt_id[name]] = store
        self._dims = [st.feature_dim if st is not None else 0 for st in self._stores]
        feat_ptrs = None
        if any(st is not None for st in self._stores):
            feat_ptrs = (C.c_void_p * len(self._stores))(*[st._h if st is not None else None for st in self._stores])
        fan = np.ascontiguousarray(config._fanout(graph))
        seed = config.seed if self._seeded else secrets.randbits(64)
        self._h = C.c_void_p()
        _lib.check(_lib.lib().ag_hetero_loader_create(graph._h, self._seed_type, fan.ctypes.data, config.num_hops,
                                                      int(config.replace), int(seed), _lib.RNG_MODE[config.rng_mode],
                                                      int(self._seeded), feat_ptrs, prefetch_depth,
                                                      max(1, int(sampler_threads)), max(1, min(int(group), 64)),
                                                      C.byref(self._h)))
        self._dev_index = int(graph.device)
        self._release = _lib.lib().ag_hetero_loader_release_batch
        self._lock = threading.Lock()
        self._next_seq = 0
        self._seeds: dict[int, np.ndarray] = {}
        self._fetched: list = []
        self._fetch_buf = (_lib.HeteroBatch * _FETCH)()
        self._closed = False

    def submit(self, batch_idx: int, seeds) -> None:
        if self._closed:
            raise SamplingError("Submit failed: loader is shut down")
        s = coerce_seeds(seeds, self._seed_nodes)
        with self._lock:
            # The C call blocks while the work queue is full; the lock keeps the
            # Python-side sequence counter in step with the library's.
            seq = self._next_seq
            self._seeds[seq] = s
            rc = _lib.lib().ag_hetero_loader_submit(self._h, int(batch_idx), s.ctypes.data if len(s) else None, len(s))
            if rc != _lib.AG_OK:
                del self._seeds[seq]
                _lib.check(rc)
            self._next_seq += 1

    def next_batch(self):
        """`(batch_idx, subgraph)`, or None after `shutdown()`; TimeoutError when
        nothing arrived within 30 s; RuntimeError once a worker failed."""
        if not self._fetched:
            if self._closed:
                return None
            got = C.c_uint32()
            rc = _lib.lib().ag_hetero_loader_next_many(self._h, -1, _FETCH, self._fetch_buf, C.byref(got))
            if rc == _lib.AG_ERR_SHUTDOWN:
                return None
            _lib.check(rc)
            for i in range(got.value - 1, -1, -1):  # reversed: pop() hands them out in order
                self._fetched.append(_lib.HeteroBatch.from_buffer_copy(self._fetch_buf[i]))
        b = self._fetched.pop()
        seeds = self._seeds.pop(b.seq)
        sg = HeteroSampledSubgraph(self._graph, self._seed_type, seeds, b.counts, b.bufs, _HeteroLease(self, b), self._dims)
        for t, d in enumerate(self._dims):
            # a type that outgrew the rows reserved for it is gathered again, exactly
            if d and b.counts.nodes[t] > b.bufs.cap_x[t]:
                sg._x_override[t] = self._stores[t].gather(sg.nodes_t(self._graph._node_types[t][0]))
        return int(b.batch_idx), sg

    def next(self):
        r = self.next_batch()
        return None if r is None else r[1]

    @property
    def prefetch_depth(self) -> int:
        return self._depth

    def stats(self) -> PrefetchStats:
        s = _lib.LoaderStats()
        _lib.check(_lib.lib().ag_hetero_loader_stats_get(self._h, C.byref(s)))
        return PrefetchStats(s)

    def shutdown(self) -> None:
        if self._h:
            _lib.lib().ag_hetero_loader_shutdown(self._h)
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
                _lib.lib().ag_hetero_loader_free(h)
            except Exception:
                pass
            self._h = None

    def __repr__(self) -> str:
        return f"HeteroNeighborLoader(prefetch_depth={self._depth})"

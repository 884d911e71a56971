"""ctypes binding of the CPU oracle (liboracle.so) — TEST INFRASTRUCTURE.

The oracle restates the reference's CPU minibatch path in plain C (see
oracle.h).  Only tests, the smoke check and the bench's CPU-baseline legs may
import this module; the shipped package never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

F32, F16, BF16 = 0, 1, 2
DTYPE_TAG = {"f32": F32, "f16": F16, "bf16": BF16}


def build(force: bool = False) -> str:
    """Compile liboracle.so with the Makefile beside this file."""
    src = os.path.join(_HERE, "oracle.c")
    stale = (not os.path.exists(_LIB_PATH)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
             or os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "oracle.h")))
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


REF_WARP_SAMPLER = os.path.join(_HERE, "_ref", "libref_warp_sampler.so")
# A checkout of the reference: $AETHERGRAPH_REFERENCE, else a directory named
# `reference` beside this repository.
_REF_ROOT = os.environ.get("AETHERGRAPH_REFERENCE") or os.path.normpath(os.path.join(_HERE, "..", "..", "reference"))


def build_ref() -> str | None:
    """Compile the reference's own CUDA sampler kernel (from the reference checkout,
    where one is present) into oracle/_ref/.  Returns the library path, or None
    when neither a checkout nor a previously built library exists."""
    src = os.path.join(_REF_ROOT, "crates", "aether-stream", "src", "gpu", "kernels", "sampler", "sampler.cu")
    if os.path.exists(src):
        subprocess.run(["make", "-C", _HERE, "ref", f"REF={_REF_ROOT}"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return REF_WARP_SAMPLER if os.path.exists(REF_WARP_SAMPLER) else None


_ref_lib = None


def ref_warp_sample(offsets_ptr: int, neighbors_ptr: int, num_nodes: int, nodes_ptr: int, output_ptr: int,
                    counts_ptr: int, node_count: int, fanout: int, seed: int, layer: int, stream: int = 0) -> None:
    """Launch the reference's `warp_sample_neighbors` on device arrays (raw pointers)."""
    global _ref_lib
    if _ref_lib is None:
        if not os.path.exists(REF_WARP_SAMPLER):
            raise FileNotFoundError(REF_WARP_SAMPLER)
        _ref_lib = C.CDLL(REF_WARP_SAMPLER)
        _ref_lib.ref_warp_sample_launch.restype = C.c_int
        _ref_lib.ref_warp_sample_launch.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p,
                                                    C.c_void_p, C.c_int, C.c_int, C.c_uint64, C.c_uint32, C.c_void_p]
    rc = _ref_lib.ref_warp_sample_launch(offsets_ptr, neighbors_ptr, num_nodes, nodes_ptr, output_ptr, counts_ptr,
                                         node_count, fanout, seed & (2**64 - 1), layer, stream or None)
    if rc != 0:
        raise RuntimeError(f"reference warp_sample_neighbors launch failed: cudaError {rc}")


class _Csr(C.Structure):
    _fields_ = [("offsets", C.c_void_p), ("edges", C.c_void_p), ("weights", C.c_void_p),
                ("num_nodes", C.c_uint64), ("num_edges", C.c_uint64)]


class _Config(C.Structure):
    _fields_ = [("fanout", C.c_void_p), ("num_hops", C.c_uint32), ("replace", C.c_int),
                ("weighted", C.c_int), ("track_edge_ids", C.c_int), ("seed", C.c_uint64),
                ("dense_dedup_max_nodes", C.c_uint64)]


class _Subgraph(C.Structure):
    _fields_ = [("nodes", C.POINTER(C.c_uint32)), ("num_nodes", C.c_size_t),
                ("edge_src", C.POINTER(C.c_uint32)), ("edge_dst", C.POINTER(C.c_uint32)),
                ("edge_ids", C.POINTER(C.c_uint64)),
                ("src_local", C.POINTER(C.c_uint32)), ("dst_local", C.POINTER(C.c_uint32)),
                ("num_edges", C.c_size_t),
                ("seed_locals", C.POINTER(C.c_uint32)), ("num_seeds", C.c_size_t),
                ("num_sampled_nodes", C.POINTER(C.c_uint64)),
                ("num_sampled_edges", C.POINTER(C.c_uint64)),
                ("num_hops", C.c_uint32), ("draws", C.c_uint64)]


class _Relation(C.Structure):
    _fields_ = [("src_type", C.c_uint32), ("dst_type", C.c_uint32), ("csr", _Csr)]


class _InAdj(C.Structure):
    _fields_ = [("offsets", C.POINTER(C.c_uint64)), ("sources", C.POINTER(C.c_uint32)),
                ("num_dst", C.c_uint64)]


class _HeteroConfig(C.Structure):
    _fields_ = [("num_node_types", C.c_uint32), ("num_nodes", C.c_void_p),
                ("num_edge_types", C.c_uint32), ("relations", C.POINTER(_Relation)),
                ("fanout", C.c_void_p), ("num_hops", C.c_uint32), ("replace", C.c_int),
                ("seed", C.c_uint64), ("dense_dedup_max_nodes", C.c_uint64)]


class _HeteroSubgraph(C.Structure):
    _fields_ = [("num_node_types", C.c_uint32), ("num_edge_types", C.c_uint32),
                ("nodes", C.POINTER(C.POINTER(C.c_uint32))), ("num_nodes", C.POINTER(C.c_size_t)),
                ("edge_src_local", C.POINTER(C.POINTER(C.c_uint32))),
                ("edge_dst_local", C.POINTER(C.POINTER(C.c_uint32))),
                ("num_edges", C.POINTER(C.c_size_t)),
                ("seed_indices", C.POINTER(C.c_uint32)), ("num_seeds", C.c_size_t),
                ("draws", C.c_uint64)]


class _BenchResult(C.Structure):
    _fields_ = [("batches", C.c_uint64), ("edges", C.c_uint64), ("nodes", C.c_uint64),
                ("seconds", C.c_double), ("threads", C.c_int), ("checksum", C.c_uint64)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.ago_batch_seed.restype = C.c_uint64
        L.ago_batch_seed.argtypes = [C.c_uint64, C.c_uint64]
        L.ago_wyrand_at.restype = C.c_uint64
        L.ago_wyrand_at.argtypes = [C.c_uint64, C.c_uint64]
        L.ago_wyrand_next_u64.restype = C.c_uint64
        L.ago_wyrand_next_u64.argtypes = [C.POINTER(C.c_uint64)]
        L.ago_philox4x32_10.restype = None
        L.ago_philox4x32_10.argtypes = [C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint32,
                                        C.POINTER(C.c_uint32)]
        L.ago_philox_u32.restype = C.c_uint32
        L.ago_philox_u32.argtypes = [C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint32]
        L.ago_reservoir_sample.restype = C.c_size_t
        L.ago_reservoir_sample.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_uint64,
                                           C.c_uint32, C.c_uint64, C.c_void_p]
        L.ago_neg_ln_u64.restype = C.c_double
        L.ago_neg_ln_u64.argtypes = [C.c_uint64]
        L.ago_f32_to_bf16.restype = C.c_uint16
        L.ago_f32_to_bf16.argtypes = [C.c_float]
        L.ago_f32_to_f16.restype = C.c_uint16
        L.ago_f32_to_f16.argtypes = [C.c_float]
        L.ago_bf16_to_f32.restype = C.c_float
        L.ago_bf16_to_f32.argtypes = [C.c_uint16]
        L.ago_f16_to_f32.restype = C.c_float
        L.ago_f16_to_f32.argtypes = [C.c_uint16]
        L.ago_encode_rows.restype = None
        L.ago_encode_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        L.ago_decode_rows.restype = None
        L.ago_decode_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
        L.ago_encode_i8.restype = C.c_int
        L.ago_encode_i8.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p]
        L.ago_gather_i8.restype = C.c_int64
        L.ago_gather_i8.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p, C.c_size_t, C.c_void_p]
        L.ago_gather.restype = C.c_int64
        L.ago_gather.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_void_p,
                                 C.c_size_t, C.c_void_p]
        L.ago_crc32.restype = C.c_uint32
        L.ago_crc32.argtypes = [C.c_uint32, C.c_void_p, C.c_size_t]
        L.ago_sampler_new.restype = C.c_void_p
        L.ago_sampler_new.argtypes = [C.POINTER(_Csr), C.POINTER(_Config)]
        L.ago_sampler_free.restype = None
        L.ago_sampler_free.argtypes = [C.c_void_p]
        L.ago_sampler_reseed.restype = None
        L.ago_sampler_reseed.argtypes = [C.c_void_p, C.c_uint64]
        L.ago_sample.restype = C.c_int64
        L.ago_sample.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(_Subgraph)]
        L.ago_subgraph_free.restype = None
        L.ago_subgraph_free.argtypes = [C.POINTER(_Subgraph)]
        L.ago_transpose.restype = None
        L.ago_transpose.argtypes = [C.POINTER(_Csr), C.c_uint64, C.c_uint64, C.POINTER(_InAdj)]
        L.ago_in_adjacency_free.restype = None
        L.ago_in_adjacency_free.argtypes = [C.POINTER(_InAdj)]
        L.ago_hetero_sampler_new.restype = C.c_void_p
        L.ago_hetero_sampler_new.argtypes = [C.POINTER(_HeteroConfig)]
        L.ago_hetero_sampler_free.restype = None
        L.ago_hetero_sampler_free.argtypes = [C.c_void_p]
        L.ago_hetero_sampler_reseed.restype = None
        L.ago_hetero_sampler_reseed.argtypes = [C.c_void_p, C.c_uint64]
        L.ago_hetero_sample.restype = C.c_int64
        L.ago_hetero_sample.argtypes = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_size_t,
                                        C.POINTER(_HeteroSubgraph)]
        L.ago_hetero_subgraph_free.restype = None
        L.ago_hetero_subgraph_free.argtypes = [C.POINTER(_HeteroSubgraph)]
        L.ago_hetero_in_adjacency.restype = C.POINTER(_InAdj)
        L.ago_hetero_in_adjacency.argtypes = [C.c_void_p, C.c_uint32]
        L.ago_bench_run.restype = C.c_int
        L.ago_bench_run.argtypes = [C.POINTER(_Csr), C.POINTER(_Config), C.c_void_p, C.c_uint64,
                                    C.c_int, C.c_void_p, C.c_size_t, C.c_size_t, C.c_uint64,
                                    C.c_int, C.POINTER(_BenchResult)]
        L.ago_synth_rmat_csr.restype = C.c_int
        L.ago_synth_rmat_csr.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_float, C.c_float,
                                         C.c_uint64, C.c_int, C.c_void_p, C.c_void_p]
        L.ago_synth_features.restype = C.c_int
        L.ago_synth_features.argtypes = [C.c_uint64, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int,
                                         C.c_void_p]
        _lib = L
    return _lib


def synth_rmat_csr(num_src: int, num_dst: int, num_edges: int, seed: int, abc=(0.57, 0.19, 0.19),
                   threads: int = 1):
    """CPU twin of the library's R-MAT generator: (offsets u64, dst u32), rows sorted."""
    offsets = np.empty(num_src + 1, dtype=np.uint64)
    dst = np.empty(max(num_edges, 1), dtype=np.uint32)
    rc = lib().ago_synth_rmat_csr(num_src, num_dst, num_edges, abc[0], abc[1], abc[2], seed & (2**64 - 1),
                                  threads, offsets.ctypes.data, dst.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"ago_synth_rmat_csr failed ({rc})")
    return offsets, dst[:num_edges]


def synth_features(num_nodes: int, dim: int, dtype: str, seed: int, row_range=None, threads: int = 1):
    """CPU twin of the library's feature generator: encoded payload as a flat array."""
    lo, hi = row_range if row_range is not None else (0, num_nodes)
    tag = DTYPE_TAG[dtype]
    out = np.empty((hi - lo) * dim, dtype=np.float32 if tag == F32 else np.uint16)
    lib().ago_synth_features(dim, tag, seed & (2**64 - 1), lo, hi, threads, out.ctypes.data)
    return out


# ---------------------------------------------------------------- scalars --
def batch_seed(base: int, idx: int) -> int:
    return lib().ago_batch_seed(base & (2**64 - 1), idx)


def wyrand_at(seed: int, d: int) -> int:
    return lib().ago_wyrand_at(seed & (2**64 - 1), d)


def wyrand_stream(seed: int, n: int) -> np.ndarray:
    """The first n next_u64() values of a generator created with `seed`."""
    st = C.c_uint64(seed & (2**64 - 1))
    return np.array([lib().ago_wyrand_next_u64(C.byref(st)) for _ in range(n)], dtype=np.uint64)


def philox4x32_10(seed: int, layer: int, node: int, draw_group: int = 0):
    out = (C.c_uint32 * 4)()
    lib().ago_philox4x32_10(seed, layer, node, draw_group, out)
    return [int(x) for x in out]


def philox_u32(seed: int, layer: int, node: int, draw_index: int) -> int:
    return lib().ago_philox_u32(seed, layer, node, draw_index)


def reservoir_sample(neighbors, fanout: int, seed: int, layer: int, node: int) -> np.ndarray:
    nb = np.ascontiguousarray(neighbors, dtype=np.uint32)
    out = np.empty(max(len(nb), fanout, 1), dtype=np.uint32)
    n = lib().ago_reservoir_sample(nb.ctypes.data, len(nb), fanout, seed, layer, node,
                                   out.ctypes.data)
    return out[:n].copy()


def neg_ln_u64(bits: int) -> float:
    return lib().ago_neg_ln_u64(bits)


def crc32(data: bytes | np.ndarray, crc: int = 0) -> int:
    a = np.frombuffer(data, dtype=np.uint8) if isinstance(data, (bytes, bytearray)) else \
        np.ascontiguousarray(data).view(np.uint8).reshape(-1)
    return lib().ago_crc32(crc, a.ctypes.data, a.size)


# ----------------------------------------------------------------- codecs --
def encode(features: np.ndarray, dtype: str) -> np.ndarray:
    """f32 array -> stored payload (uint8 view of f32 / f16 bits / bf16 bits)."""
    f = np.ascontiguousarray(features, dtype=np.float32)
    tag = DTYPE_TAG[dtype]
    out = np.empty(f.size * (4 if tag == F32 else 2), dtype=np.uint8)
    lib().ago_encode_rows(f.ctypes.data, f.size, tag, out.ctypes.data)
    return out


def decode(payload: np.ndarray, dtype: str) -> np.ndarray:
    """Stored payload (any integer/float array viewed as bytes) -> f32, bit-preserving."""
    raw = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
    tag = DTYPE_TAG[dtype]
    n = raw.size // (4 if tag == F32 else 2)
    out = np.empty(n, dtype=np.float32)
    lib().ago_decode_rows(raw.ctypes.data, n, tag, out.ctypes.data)
    return out


def gather(payload: np.ndarray, num_nodes: int, dim: int, dtype: str, ids) -> np.ndarray:
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    payload = np.ascontiguousarray(payload)
    out = np.empty((len(ids), dim), dtype=np.float32)
    rc = lib().ago_gather(payload.ctypes.data, num_nodes, dim, DTYPE_TAG[dtype],
                          ids.ctypes.data, len(ids), out.ctypes.data)
    if rc != 0:
        raise ValueError(f"node {int(ids[-1 - rc])} out of bounds")
    return out


def encode_i8(features) -> tuple[np.ndarray, np.ndarray]:
    """Block-scaled int8 (internal/feature_codec.rs:73-112): (codes int8 [n, dim], scales f32 [n, ceil(dim / 32)])."""
    f = np.ascontiguousarray(features, dtype=np.float32)
    n, dim = f.shape
    if dim == 0:
        raise ValueError("feature_dim must be non-zero")
    codes = np.zeros((n, dim), dtype=np.int8)
    scales = np.zeros((n, (dim + 31) // 32), dtype=np.float32)
    if lib().ago_encode_i8(f.ctypes.data, n, dim, codes.ctypes.data, scales.ctypes.data) != 0:
        raise ValueError("feature values must be finite")
    return codes, scales


def gather_i8(codes: np.ndarray, scales: np.ndarray, ids) -> np.ndarray:
    """Decoded rows `ids` of a block-scaled int8 table (feature_codec.rs:121-133)."""
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    n, dim = codes.shape
    out = np.empty((len(ids), dim), dtype=np.float32)
    rc = lib().ago_gather_i8(np.ascontiguousarray(codes).ctypes.data, np.ascontiguousarray(scales).ctypes.data, n, dim,
                             ids.ctypes.data, len(ids), out.ctypes.data)
    if rc != 0:
        raise ValueError(f"node {int(ids[-1 - rc])} out of bounds")
    return out


# ---------------------------------------------------------------- sampler --
def _csr_struct(offsets, edges, weights, keep):
    offsets = np.ascontiguousarray(offsets, dtype=np.uint64)
    edges = np.ascontiguousarray(edges, dtype=np.uint32)
    keep += [offsets, edges]
    w = None
    if weights is not None:
        w = np.ascontiguousarray(weights, dtype=np.float32)
        keep.append(w)
    return _Csr(offsets.ctypes.data, edges.ctypes.data if edges.size else None,
                w.ctypes.data if w is not None else None, len(offsets) - 1, len(edges))


def _np(ptr, n, dtype):
    if n == 0:
        return np.empty(0, dtype=dtype)
    return np.ctypeslib.as_array(ptr, shape=(n,)).astype(dtype, copy=True)


class Sampler:
    """Oracle NeighborSampler (loader/sampler.rs)."""

    def __init__(self, offsets, edges, fanout, *, weights=None, replace=False, weighted=False,
                 track_edge_ids=True, seed=0, dense_dedup_max_nodes=0):
        self._keep = []
        self._csr = _csr_struct(offsets, edges, weights, self._keep)
        fan = np.ascontiguousarray(fanout, dtype=np.uint32)
        self._keep.append(fan)
        self._cfg = _Config(fan.ctypes.data, len(fan), int(replace), int(weighted),
                            int(track_edge_ids), seed & (2**64 - 1), dense_dedup_max_nodes)
        self.seed = seed & (2**64 - 1)
        self.num_hops = len(fan)
        self._h = lib().ago_sampler_new(C.byref(self._csr), C.byref(self._cfg))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ago_sampler_free(self._h)
            self._h = None

    def reseed(self, seed: int):
        lib().ago_sampler_reseed(self._h, seed & (2**64 - 1))

    def sample(self, seeds) -> dict:
        seeds = np.ascontiguousarray(seeds, dtype=np.uint32)
        sg = _Subgraph()
        rc = lib().ago_sample(self._h, seeds.ctypes.data, len(seeds), C.byref(sg))
        if rc != 0:
            pos = -1 - rc
            raise IndexError(f"seed node {int(seeds[pos])} (position {pos}) is out of range "
                             f"for {self._csr.num_nodes} nodes")
        try:
            e = sg.num_edges
            out = {
                "nodes": _np(sg.nodes, sg.num_nodes, np.uint32),
                "edge_src": _np(sg.edge_src, e, np.uint32),
                "edge_dst": _np(sg.edge_dst, e, np.uint32),
                "edge_ids": _np(sg.edge_ids, e, np.uint64) if sg.edge_ids else None,
                "src_local": _np(sg.src_local, e, np.uint32),
                "dst_local": _np(sg.dst_local, e, np.uint32),
                "seed_locals": _np(sg.seed_locals, sg.num_seeds, np.uint32),
                "num_sampled_nodes": _np(sg.num_sampled_nodes, sg.num_hops + 1, np.uint64),
                "num_sampled_edges": _np(sg.num_sampled_edges, sg.num_hops, np.uint64),
                "draws": int(sg.draws),
            }
        finally:
            lib().ago_subgraph_free(C.byref(sg))
        return out

    def bench(self, payload, dim, dtype, seeds, batch_size, first_position=0, threads=1) -> dict:
        seeds = np.ascontiguousarray(seeds, dtype=np.uint32)
        nb = len(seeds) // batch_size
        res = _BenchResult()
        ptr = None
        if payload is not None:
            payload = np.ascontiguousarray(payload)
            ptr = payload.ctypes.data
        rc = lib().ago_bench_run(C.byref(self._csr), C.byref(self._cfg), ptr, dim,
                                 DTYPE_TAG[dtype] if dtype else 0, seeds.ctypes.data,
                                 batch_size, nb, first_position, threads, C.byref(res))
        if rc != 0:
            raise RuntimeError("oracle bench run failed (bad seed or node id)")
        return {"batches": res.batches, "edges": res.edges, "nodes": res.nodes,
                "seconds": res.seconds, "threads": res.threads, "checksum": res.checksum}


def mirror(sub: dict) -> dict:
    """Bidirectional rewrite of one sampled subgraph
    (crates/aethergraph-core/src/loader/sampler.rs:1015-1040 `mirror`): the sampled
    edges stay as they are, then, walking them in order, the reverse of edge i is
    appended unless its (src_local, dst_local) pair is already present among the
    sampled edges or the reverses appended so far; a reverse carries its forward
    edge's id.  Per-hop counts are those of the sampling pass."""
    sl, dl = sub["src_local"], sub["dst_local"]
    pairs = {(int(a), int(b)) for a, b in zip(sl, dl)}
    keep = []
    for i, (a, b) in enumerate(zip(sl, dl)):
        r = (int(b), int(a))
        if r in pairs:
            continue
        pairs.add(r)
        keep.append(i)
    k = np.array(keep, dtype=np.int64)
    out = dict(sub)
    out["edge_src"] = np.concatenate([sub["edge_src"], sub["edge_dst"][k]])
    out["edge_dst"] = np.concatenate([sub["edge_dst"], sub["edge_src"][k]])
    out["src_local"] = np.concatenate([sl, dl[k]])
    out["dst_local"] = np.concatenate([dl, sl[k]])
    if sub.get("edge_ids") is not None:
        out["edge_ids"] = np.concatenate([sub["edge_ids"], sub["edge_ids"][k]])
    return out


def induce(offsets, edges, sub: dict) -> dict:
    """Induced rewrite (sampler.rs:972-1013 `induce`, no timestamps): the sampled edges
    are replaced by every stored edge u -> w with both ends among the sampled nodes,
    in the order of u's local index, then of the position in u's row; the edge id is
    the CSR position."""
    nodes = sub["nodes"]
    local = {int(v): i for i, v in enumerate(nodes)}
    es, ed, sl, dl, ids = [], [], [], [], []
    for u_local, u in enumerate(nodes):
        lo, hi = int(offsets[int(u)]), int(offsets[int(u) + 1])
        for pos in range(lo, hi):
            w = int(edges[pos])
            w_local = local.get(w)
            if w_local is not None:
                es.append(int(u)); ed.append(w); sl.append(u_local); dl.append(w_local); ids.append(pos)
    out = dict(sub)
    out["edge_src"], out["edge_dst"] = np.array(es, dtype=np.uint32), np.array(ed, dtype=np.uint32)
    out["src_local"], out["dst_local"] = np.array(sl, dtype=np.uint32), np.array(dl, dtype=np.uint32)
    out["edge_ids"] = np.array(ids, dtype=np.uint64) if sub.get("edge_ids") is not None else None
    return out


def transpose(offsets, edges, num_src: int, num_dst: int):
    keep = []
    csr = _csr_struct(offsets, edges, None, keep)
    adj = _InAdj()
    lib().ago_transpose(C.byref(csr), num_src, num_dst, C.byref(adj))
    off = _np(adj.offsets, num_dst + 1, np.uint64)
    src = _np(adj.sources, int(off[-1]), np.uint32)
    lib().ago_in_adjacency_free(C.byref(adj))
    return off, src


class HeteroSampler:
    """Oracle HeteroNeighborSampler (loader/hetero_sampler.rs).

    num_nodes: list per node type; relations: list of (src_type, dst_type,
    offsets, edges); fanout: [edge_type][hop].
    """

    def __init__(self, num_nodes, relations, fanout, *, replace=False, seed=0,
                 dense_dedup_max_nodes=0):
        self._keep = []
        nn = np.ascontiguousarray(num_nodes, dtype=np.uint64)
        fan = np.ascontiguousarray(fanout, dtype=np.uint32).reshape(len(relations), -1)
        rel = (_Relation * max(len(relations), 1))()
        for i, (st, dt, off, edg) in enumerate(relations):
            rel[i] = _Relation(st, dt, _csr_struct(off, edg, None, self._keep))
        self._keep += [nn, fan, rel]
        self.num_node_types, self.num_edge_types = len(nn), len(relations)
        self._num_nodes = nn
        cfg = _HeteroConfig(len(nn), nn.ctypes.data, len(relations), rel, fan.ctypes.data,
                            fan.shape[1], int(replace), seed & (2**64 - 1), dense_dedup_max_nodes)
        self._h = lib().ago_hetero_sampler_new(C.byref(cfg))

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ago_hetero_sampler_free(self._h)
            self._h = None

    def reseed(self, seed: int):
        lib().ago_hetero_sampler_reseed(self._h, seed & (2**64 - 1))

    def in_adjacency(self, edge_type: int):
        a = lib().ago_hetero_in_adjacency(self._h, edge_type).contents
        off = _np(a.offsets, a.num_dst + 1, np.uint64)
        return off, _np(a.sources, int(off[-1]), np.uint32)

    def sample(self, seed_type: int, seeds) -> dict:
        seeds = np.ascontiguousarray(seeds, dtype=np.uint32)
        sg = _HeteroSubgraph()
        rc = lib().ago_hetero_sample(self._h, seed_type, seeds.ctypes.data, len(seeds), C.byref(sg))
        if rc != 0:
            pos = -1 - rc
            raise IndexError(f"seed node {int(seeds[pos])} (position {pos}) is out of range "
                             f"for {int(self._num_nodes[seed_type])} nodes")
        try:
            out = {
                "nodes": [_np(sg.nodes[t], sg.num_nodes[t], np.uint32)
                          for t in range(sg.num_node_types)],
                "edge_src_local": [_np(sg.edge_src_local[e], sg.num_edges[e], np.uint32)
                                   for e in range(sg.num_edge_types)],
                "edge_dst_local": [_np(sg.edge_dst_local[e], sg.num_edges[e], np.uint32)
                                   for e in range(sg.num_edge_types)],
                "seed_indices": _np(sg.seed_indices, sg.num_seeds, np.uint32),
                "draws": int(sg.draws),
            }
        finally:
            lib().ago_hetero_subgraph_free(C.byref(sg))
        return out


# ---------------------------------------------------------------------------
# AETHHETG v1 (crates/aethergraph-core/src/internal/mmap_hetero.rs:1-45), in numpy:
# the oracle-side writer and reader the GPU loader / saver are checked against.
# ---------------------------------------------------------------------------
def _name64(text: str) -> bytes:
    b = text.encode()
    assert len(b) < 64, f"type name too long: {text}"
    return b + b"\0" * (64 - len(b))


def write_hetero_file(path, node_types, relations) -> None:
    """node_types: [(name, count)]; relations: [(src, rel, dst, offsets u64[num_src + 1], edges u32[E], weights f32[E] | None)]
    (mmap_hetero.rs:98-157: header, node type table, edge type table, then per relation
    offsets, edges and optional weights, the u32 sections zero-padded to 8 bytes)."""
    out = bytearray(64)
    out[:8] = b"AETHHETG"
    out[8:12] = np.uint32(1).tobytes()
    out[12:16] = np.uint32(len(node_types)).tobytes()
    out[16:20] = np.uint32(len(relations)).tobytes()
    for name, count in node_types:
        out += _name64(name) + np.uint64(count).tobytes()
    for (s, rel, d, offsets, edges, weights) in relations:
        out += _name64(s) + _name64(rel) + _name64(d)
        out += np.uint64(len(offsets) - 1).tobytes() + np.uint64(len(edges)).tobytes()
        out += np.uint32(1 if weights is not None else 0).tobytes() + np.uint32(0).tobytes()
    for (_, _, _, offsets, edges, weights) in relations:
        out += np.ascontiguousarray(offsets, dtype=np.uint64).tobytes()
        eb = np.ascontiguousarray(edges, dtype=np.uint32).tobytes()
        out += eb + b"\0" * (-len(eb) % 8)
        if weights is not None:
            wb = np.ascontiguousarray(weights, dtype=np.float32).tobytes()
            out += wb + b"\0" * (-len(wb) % 8)
    with open(path, "wb") as f:
        f.write(bytes(out))


def read_hetero_file(path):
    """Inverse of write_hetero_file (no validation beyond the layout): returns
    (node_types, relations)."""
    raw = open(path, "rb").read()
    assert raw[:8] == b"AETHHETG" and int(np.frombuffer(raw[8:12], np.uint32)[0]) == 1
    nt_n, et_n = (int(v) for v in np.frombuffer(raw[12:20], np.uint32))
    at = 64
    name = lambda b: b[:b.index(b"\0")].decode()
    node_types = []
    for _ in range(nt_n):
        node_types.append((name(raw[at:at + 64]), int(np.frombuffer(raw[at + 64:at + 72], np.uint64)[0])))
        at += 72
    heads = []
    for _ in range(et_n):
        ns, ne = (int(v) for v in np.frombuffer(raw[at + 192:at + 208], np.uint64))
        heads.append((name(raw[at:at + 64]), name(raw[at + 64:at + 128]), name(raw[at + 128:at + 192]), ns, ne,
                      int(np.frombuffer(raw[at + 208:at + 212], np.uint32)[0]) != 0))
        at += 216
    relations = []
    for (s, rel, d, ns, ne, has_w) in heads:
        offsets = np.frombuffer(raw[at:at + 8 * (ns + 1)], np.uint64).copy(); at += 8 * (ns + 1)
        edges = np.frombuffer(raw[at:at + 4 * ne], np.uint32).copy(); at += 4 * ne + (-4 * ne % 8)
        weights = None
        if has_w:
            weights = np.frombuffer(raw[at:at + 4 * ne], np.float32).copy(); at += 4 * ne + (-4 * ne % 8)
        relations.append((s, rel, d, offsets, edges, weights))
    assert at == len(raw), "trailing bytes"
    return node_types, relations


# ------------------------------------------------ AETH version 2 (compressed) --
# Succinct-coded CSR at rest (crates/aethergraph-core/src/internal/compressed_graph.rs:1-19,
# 39-88, 99-175) through the two codecs of internal/succinct.rs, restated in numpy.
def ef_encode(values):
    """Elias-Fano of a non-decreasing u64 sequence (succinct.rs:52-92):
    -> (len, universe, low_bits, low words, high words)."""
    v = np.ascontiguousarray(values, dtype=np.uint64)
    n = int(v.size)
    assert n < 2 or bool(np.all(v[:-1] <= v[1:])), "EliasFano requires a sorted sequence"
    universe = int(v[-1]) if n else 0
    low_bits = 0 if n == 0 or universe < n else (universe // n).bit_length() - 1
    high = np.zeros((n + (universe >> low_bits) + 1 + 63) // 64, dtype=np.uint64)
    idx = np.arange(n, dtype=np.uint64)
    pos = (v >> np.uint64(low_bits)) + idx
    np.bitwise_or.at(high, (pos // np.uint64(64)).astype(np.int64), np.uint64(1) << (pos % np.uint64(64)))
    low = np.zeros((n * low_bits + 63) // 64, dtype=np.uint64)
    if low_bits:
        part = v & np.uint64((1 << low_bits) - 1)
        bit = idx * np.uint64(low_bits)
        word, off = (bit // np.uint64(64)).astype(np.int64), bit % np.uint64(64)
        np.bitwise_or.at(low, word, part << off)                      # the bits that fit the word
        spill = (off + np.uint64(low_bits)) > np.uint64(64)           # the rest starts the next word
        np.bitwise_or.at(low, word[spill] + 1, part[spill] >> (np.uint64(64) - off[spill]))
    return n, universe, low_bits, low, high


def ef_decode(n: int, universe: int, low_bits: int, low: np.ndarray, high: np.ndarray) -> np.ndarray:
    """The sequence back (succinct.rs:162-192): element i sits at the (i+1)-th set bit."""
    bits = np.unpackbits(np.ascontiguousarray(high, dtype="<u8").view(np.uint8), bitorder="little")
    pos = np.flatnonzero(bits).astype(np.uint64)
    assert pos.size == n, f"EF high array has {pos.size} set bits for {n} elements"
    idx = np.arange(n, dtype=np.uint64)
    out = (pos - idx) << np.uint64(low_bits)
    if low_bits and n:
        lw = np.concatenate([np.ascontiguousarray(low, dtype=np.uint64), np.zeros(1, dtype=np.uint64)])
        bit = idx * np.uint64(low_bits)
        word, off = (bit // np.uint64(64)).astype(np.int64), bit % np.uint64(64)
        part = lw[word] >> off
        spill = (off + np.uint64(low_bits)) > np.uint64(64)
        part[spill] |= lw[word[spill] + 1] << (np.uint64(64) - off[spill])
        out |= part & np.uint64((1 << low_bits) - 1)
    return out


def svb_encode(values):
    """StreamVByte of the wrapping deltas of a u32 sequence (succinct.rs:397-420, 586-600):
    -> (len, first, control bytes, data bytes)."""
    v = np.ascontiguousarray(values, dtype=np.uint32)
    n = int(v.size)
    if n == 0:
        return 0, 0, np.zeros(0, np.uint8), np.zeros(0, np.uint8)
    d = (v[1:] - v[:-1]).astype(np.uint32)  # wraps modulo 2^32
    nbytes = 1 + (d >= (1 << 8)).astype(np.int64) + (d >= (1 << 16)) + (d >= (1 << 24))
    control = np.zeros((d.size + 3) // 4, dtype=np.uint8)
    i = np.arange(d.size)
    np.bitwise_or.at(control, i // 4, ((nbytes - 1) << ((i % 4) * 2)).astype(np.uint8))
    le = d.astype("<u4").view(np.uint8).reshape(-1, 4)
    data = le[np.arange(4)[None, :] < nbytes[:, None]]
    return n, int(v[0]), control, np.ascontiguousarray(data)


def svb_decode(n: int, first: int, control: np.ndarray, data: np.ndarray) -> np.ndarray:
    """Running wrapping sum of the deltas (succinct.rs:468-484)."""
    if n == 0:
        return np.zeros(0, np.uint32)
    nd = n - 1
    i = np.arange(nd)
    nbytes = ((control[i // 4].astype(np.int64) >> ((i % 4) * 2)) & 3) + 1
    start = np.concatenate([[0], np.cumsum(nbytes)[:-1]]) if nd else np.zeros(0, np.int64)
    assert int(nbytes.sum()) == data.size, f"SVB data stream is {data.size} bytes, control tags call for {int(nbytes.sum())}"
    padded = np.concatenate([data, np.zeros(4, np.uint8)])
    d = np.zeros(nd, dtype=np.uint64)
    for b in range(4):
        d |= np.where(b < nbytes, padded[start + b].astype(np.uint64) << np.uint64(8 * b), np.uint64(0))
    acc = (np.uint64(first) + np.concatenate([[np.uint64(0)], np.cumsum(d, dtype=np.uint64)])) & np.uint64(0xFFFFFFFF)
    return acc.astype(np.uint32)


def compressed_graph_bytes(offsets, dst, weights=None, checksum: bool = True) -> bytes:
    """The whole version-2 file (compressed_graph.rs:39-88; wire formats succinct.rs:198-214, 486-500)."""
    import struct

    off = np.ascontiguousarray(offsets, dtype=np.uint64)
    n, universe, low_bits, low, high = ef_encode(off)
    m, first, control, data = svb_encode(dst)
    payload = struct.pack("<QQIQ", n, universe, low_bits, low.size) + low.astype("<u8").tobytes()
    payload += struct.pack("<Q", high.size) + high.astype("<u8").tobytes()
    payload += struct.pack("<QIQ", m, first, control.size) + control.tobytes() + struct.pack("<Q", data.size) + data.tobytes()
    if weights is not None:
        payload += np.ascontiguousarray(weights, dtype="<f4").tobytes()
    head = struct.pack("<IIQQII", 0x41455448, 2, off.size - 1, m, 1 if weights is not None else 0,
                       crc32(payload) if checksum else 0)
    return head + payload


def read_compressed_graph(raw: bytes):
    """-> (num_nodes, offsets u64, dst u32, weights f32 | None), with the loader's checks
    (compressed_graph.rs:99-175)."""
    import struct

    magic, version, n, e, has_w, crc = struct.unpack_from("<IIQQII", raw, 0)
    assert magic == 0x41455448 and version == 2
    payload = raw[32:]
    if crc:
        assert crc32(payload) == crc, "compressed graph checksum mismatch"
    ef_len, universe, low_bits, lw = struct.unpack_from("<QQIQ", payload, 0)
    at = 28
    low = np.frombuffer(payload, "<u8", lw, at); at += lw * 8
    (hw,) = struct.unpack_from("<Q", payload, at); at += 8
    high = np.frombuffer(payload, "<u8", hw, at); at += hw * 8
    assert ef_len == n + 1
    m, first, nc = struct.unpack_from("<QIQ", payload, at); at += 20
    control = np.frombuffer(payload, np.uint8, nc, at); at += nc
    (nd,) = struct.unpack_from("<Q", payload, at); at += 8
    data = np.frombuffer(payload, np.uint8, nd, at); at += nd
    assert m == e
    w = None
    if has_w:
        w = np.frombuffer(payload, "<f4", e, at).copy(); at += e * 4
    assert at == len(payload), "trailing bytes after edges section"
    off = ef_decode(ef_len, universe, low_bits, low, high)
    assert off.size == 0 or int(off[-1]) == universe
    return n, off, svb_decode(m, first, control, data), w


# ------------------------------------------------------- locality reordering --
# Rabbit Order (crates/aethergraph-core/src/graph/reorder.rs:142-262) and the walks of
# its dendrogram (:46-105), restated in plain Python for small graphs; permute (:297-383)
# in numpy.  Python integers are exact, like the reference's i128 gains.
def rabbit_order(offsets, dst):
    """-> (perm, partitions): perm[new_id] = old_id, partitions[v] = dense community id."""
    off = [int(x) for x in np.asarray(offsets)]
    d = [int(x) for x in np.asarray(dst)]
    n = len(off) - 1
    parent, first_child, next_sibling = list(range(n)), [None] * n, [None] * n

    def root(v):
        r = v
        while parent[r] != r:
            r = parent[r]
        while parent[v] != r:
            parent[v], v = r, parent[v]
        return r

    if n > 1 and d:
        ins = [[] for _ in range(n)]                       # sources ascending per destination
        for u in range(n):
            for e in range(off[u], off[u + 1]):
                ins[d[e]].append(u)
        degree = [sum(1 for e in range(off[v], off[v + 1]) if d[e] != v) + sum(1 for s in ins[v] if s != v)
                  for v in range(n)]
        two_m = sum(degree)
        if two_m:
            carried, visited = [None] * n, [False] * n
            for u in sorted(range(n), key=lambda v: (degree[v], v)):
                weight_to = {}

                def add(c, w):
                    c = root(c)
                    if c != u:
                        weight_to[c] = weight_to.get(c, 0) + w

                for e in range(off[u], off[u + 1]):
                    add(d[e], 1)
                for s in ins[u]:
                    add(s, 1)
                child = first_child[u]
                while child is not None:
                    if carried[child] is not None:
                        for c, w in carried[child]:
                            add(c, w)
                        carried[child] = None
                    child = next_sibling[child]
                best = None
                for c, w in weight_to.items():
                    gain = two_m * w - degree[u] * degree[c]
                    if (gain > 0) if best is None else (gain > best[0] or (gain == best[0] and c < best[1])):
                        best = (gain, c)
                if best is not None:
                    c = best[1]
                    parent[u] = c
                    degree[c] += degree[u]
                    next_sibling[u], first_child[c] = first_child[c], u
                    if not visited[c]:
                        carried[u] = list(weight_to.items())
                visited[u] = True
    perm = []
    for r in range(n):
        if parent[r] != r:
            continue
        perm.append(r)
        stack = [first_child[r]]
        while stack:
            c = stack[-1]
            if c is None:
                stack.pop()
                continue
            stack[-1] = next_sibling[c]
            perm.append(c)
            stack.append(first_child[c])
    ids, parts = {}, []
    for v in range(n):
        parts.append(ids.setdefault(root(v), len(ids)))
    return np.array(perm, dtype=np.uint32), np.array(parts, dtype=np.uint32)


def permute_csr(offsets, dst, weights, perm):
    """Row new_id = row perm[new_id] of the old graph in its order, endpoints relabelled."""
    off = np.asarray(offsets, dtype=np.uint64)
    d = np.asarray(dst, dtype=np.uint32)
    p = np.asarray(perm, dtype=np.int64)
    inv = np.empty(p.size, dtype=np.uint32)
    inv[p] = np.arange(p.size, dtype=np.uint32)
    lens = (off[p + 1] - off[p]).astype(np.int64)
    new_off = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint64)
    src = np.concatenate([np.arange(int(off[o]), int(off[o + 1])) for o in p]).astype(np.int64) if d.size else np.zeros(0, np.int64)
    return new_off, inv[d[src]], (None if weights is None else np.asarray(weights, dtype=np.float32)[src])


def sample_disjoint(sampler: "Sampler", seeds, offsets=None, edges=None, subgraph_type: str = "directional") -> dict:
    """Disjoint sampling (crates/aethergraph-core/src/loader/sampler.rs:600-690): one pass per
    seed on the sampler's running stream, `subgraph_type` applied inside each block, the
    blocks concatenated with their local indices shifted by the nodes before them."""
    seeds = np.asarray(seeds, dtype=np.uint32)
    keys = ("nodes", "edge_src", "edge_dst", "src_local", "dst_local")
    parts = {k: [] for k in keys}
    seed_locals, batch = [], []
    nodes_per_hop = edges_per_hop = None
    at = 0
    for i, s in enumerate(seeds):
        sub = sampler.sample(seeds[i:i + 1])
        hop_nodes = np.asarray(sub["num_sampled_nodes"], dtype=np.uint64)
        hop_edges = np.asarray(sub["num_sampled_edges"], dtype=np.uint64)
        if subgraph_type == "bidirectional":
            sub = mirror(sub)
        elif subgraph_type == "induced":
            sub = induce(offsets, edges, sub)
        for k in ("nodes", "edge_src", "edge_dst"):
            parts[k].append(np.asarray(sub[k], dtype=np.uint32))
        parts["src_local"].append(np.asarray(sub["src_local"], dtype=np.uint32) + np.uint32(at))
        parts["dst_local"].append(np.asarray(sub["dst_local"], dtype=np.uint32) + np.uint32(at))
        seed_locals.append(int(sub["seed_locals"][0]) + at)
        batch.extend([i] * len(sub["nodes"]))
        if nodes_per_hop is None:
            nodes_per_hop, edges_per_hop = np.zeros_like(hop_nodes), np.zeros_like(hop_edges)
        nodes_per_hop[1:] += hop_nodes[1:]
        edges_per_hop += hop_edges
        at += len(sub["nodes"])
    out = {k: (np.concatenate(v) if v else np.zeros(0, np.uint32)) for k, v in parts.items()}
    if nodes_per_hop is not None:
        nodes_per_hop[0] = len(seeds)           # every block contributes its one seed node up front
    out.update(seed_locals=np.array(seed_locals, dtype=np.uint32), batch=np.array(batch, dtype=np.int64),
               num_sampled_nodes=nodes_per_hop, num_sampled_edges=edges_per_hop)
    return out


WYRAND_STEP = 0xA0761D6478BD642F  # the generator's additive constant (internal/genstamp.rs:181-202)


def sample_cumulative(offsets, edges, fanout, seeds, *, seed: int, weights=None, replace=False, weighted=False,
                      start_draw: int = 0) -> dict:
    """Cumulative sampling (crates/aethergraph-core/src/loader/sampler.rs:776-840 run_hops with
    `cumulative`, :1250-1258 fresh_edge, :1277-1285 emit_edge): hop h expands every node seen so
    far, in local-id order, and refuses an edge an earlier hop emitted.  Restated hop by hop on
    the one-hop restatement: a sampler seeded `seed + d * WYRAND_STEP` starts at draw d of the
    batch's stream.  Returns the arrays and `draws`, the stream position after the batch."""
    seeds = np.asarray(seeds, dtype=np.uint32)
    frontier, d = seeds, start_draw
    emitted: set = set()
    parts = {k: [] for k in ("edge_src", "edge_dst", "src_local", "dst_local", "edge_ids")}
    nodes = seed_locals = None
    nodes_per_hop, edges_per_hop = [], []
    for hop, k in enumerate(fanout):
        s = Sampler(offsets, edges, [k], weights=weights, replace=replace, weighted=weighted, track_edge_ids=True,
                    seed=(seed + d * WYRAND_STEP) & (2**64 - 1))
        one = s.sample(frontier)
        d += one["draws"]
        if hop == 0:
            nodes_per_hop.append(int(one["num_sampled_nodes"][0]))
            seed_locals = one["seed_locals"].copy()
        nodes_per_hop.append(int(one["num_sampled_nodes"][1]))
        eids = one["edge_ids"]
        keep = np.array([int(e) not in emitted for e in eids], dtype=bool)
        for name in parts:
            parts[name].append(one[name][keep])
        emitted.update(int(e) for e in eids[keep])
        edges_per_hop.append(int(keep.sum()))
        nodes = one["nodes"].copy()
        frontier = nodes
    out = {k: np.concatenate(v) for k, v in parts.items()}
    out.update(nodes=nodes, seed_locals=seed_locals, num_sampled_nodes=np.array(nodes_per_hop, dtype=np.uint64),
               num_sampled_edges=np.array(edges_per_hop, dtype=np.uint64), draws=d)
    return out

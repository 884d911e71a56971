"""Seeded synthetic inputs generated on the GPU (R-MAT graphs, feature tables, seed batches).

Stand-ins for datasets, with the shapes and value distributions of the benchmark
configurations.  Everything is a pure function of (seed, index); the recipe is
stated at the top of csrc/synth.cu.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from .features import FeatureStore
from .graph import CsrGraph

RMAT_ABC = (0.57, 0.19, 0.19)

_G1 = np.uint64(0x9E3779B97F4A7C15)


def _mix(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x.astype(np.uint64) + _G1
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _device(device):
    import torch

    if device is not None:
        return device
    if not torch.cuda.is_available():
        raise RuntimeError("aethergraph_b200 needs a CUDA device; there is no CPU path")
    return torch.cuda.current_device()


def rmat_graph(num_nodes: int, num_edges: int, seed: int, *, abc=RMAT_ABC, weight_sigma: float = 0.0,
               device: int | None = None) -> CsrGraph:
    """R-MAT graph with rows sorted by (source, destination); optional lognormal(0, sigma) weights."""
    out = C.c_void_p()
    _lib.check(_lib.lib().ag_synth_rmat_graph(num_nodes, num_edges, abc[0], abc[1], abc[2], seed & (2**64 - 1),
                                              weight_sigma, _device(device), C.byref(out)))
    return CsrGraph(out.value)


def features(num_nodes: int, dim: int, dtype: str, seed: int, *, device: int | None = None,
             row_range: tuple[int, int] | None = None) -> FeatureStore:
    """~N(0,1) feature table (or the vertex-range shard `row_range` of it) in `dtype`."""
    out = C.c_void_p()
    lo, hi = row_range if row_range is not None else (0, num_nodes)
    _lib.check(_lib.lib().ag_synth_features(num_nodes, dim, _lib.DTYPE_TAG[dtype], seed & (2**64 - 1),
                                            _device(device), lo, hi, C.byref(out)))
    return FeatureStore(out.value)


def seed_batch(num_nodes: int, batch_size: int, seed: int, batch_idx: int) -> np.ndarray:
    """Batch `batch_idx` of uniformly drawn seed ids: mix(mix(seed ^ mix(batch)) + i) % num_nodes."""
    base = _mix(np.array([seed & (2**64 - 1)], dtype=np.uint64) ^ _mix(np.array([batch_idx], dtype=np.uint64)))
    with np.errstate(over="ignore"):
        r = _mix(base + np.arange(batch_size, dtype=np.uint64))
    return (r % np.uint64(num_nodes)).astype(np.uint32)


def features_shard(num_nodes: int, dim: int, dtype: str, seed: int, rank: int, world: int, layout: str = "cyclic", *,
                   device: int | None = None) -> FeatureStore:
    """Shard `rank` of `world` of the same table as `features()`, generated in place."""
    out = C.c_void_p()
    _lib.check(_lib.lib().ag_synth_features_shard(num_nodes, dim, _lib.DTYPE_TAG[dtype], seed & (2**64 - 1),
                                                  _device(device), rank, world, _lib.SHARD_LAYOUT[layout], C.byref(out)))
    return FeatureStore(out.value)


def rmat_relation(num_src: int, num_dst: int, num_edges: int, seed: int, *, abc=RMAT_ABC, device: int | None = None):
    """One bipartite R-MAT relation generated on the device: returns
    `(offsets, dst)` as CUDA tensors (int64 offsets over the sources, int32 holding
    u32 destination ids), rows sorted by (source, destination)."""
    import torch

    dev = _device(device)
    po, pd, pw = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _lib.check(_lib.lib().ag_synth_rmat_csr(num_src, num_dst, num_edges, abc[0], abc[1], abc[2], seed & (2**64 - 1),
                                            0.0, dev, C.byref(po), C.byref(pd), C.byref(pw)))
    from .sampler import _DevArray

    tdev = torch.device("cuda", dev)
    try:
        offsets = torch.as_tensor(_DevArray(po.value, (num_src + 1,), "<i8", None), device=tdev).clone()
        dst = torch.as_tensor(_DevArray(pd.value, (max(num_edges, 1),), "<i4", None), device=tdev)[:num_edges].clone()
    finally:
        _lib.lib().ag_synth_free_device(po, dev)
        _lib.lib().ag_synth_free_device(pd, dev)
    return offsets, dst


def relation_sources(offsets):
    """Source id of every edge of a CSR relation (int32 CUDA tensor holding u32 ids)."""
    import torch

    deg = offsets[1:] - offsets[:-1]
    return torch.repeat_interleave(torch.arange(deg.numel(), dtype=torch.int32, device=offsets.device), deg)

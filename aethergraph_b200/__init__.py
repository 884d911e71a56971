"""aethergraph_b200 — the GNN minibatch hot path of aethergraph on B200 GPUs.

k-hop neighbor sampling over a static CSR graph, frontier dedup + relabel into a
local edge index, and the feature-row gather with fused f16/bf16 -> f32 upcast,
as hand-written CUDA kernels (sm_100a) behind a C ABI (include/aethergpu.h) and
the reference's Python sampler / feature-store / loader surface.
"""
from ._lib import GraphLoadError, SamplingError
from .features import FeatureStore, save_features
from .graph import CsrGraph, Graph, partition_aligned_batches
from .loader import NeighborLoader, PrefetchStats
from .hetero import (HeteroCsrGraph, HeteroNeighborLoader, HeteroNeighborSampler, HeteroSampledSubgraph,
                     HeteroSamplingConfig)
from .sampler import NeighborSampler, ParallelBatchSampler, SampledSubgraph, Sampler, SamplingConfig

__version__ = "0.1.0"

__all__ = [
    "CsrGraph", "FeatureStore", "Graph", "GraphLoadError", "HeteroCsrGraph", "HeteroNeighborLoader",
    "HeteroNeighborSampler", "HeteroSampledSubgraph", "HeteroSamplingConfig", "NeighborLoader", "NeighborSampler",
    "ParallelBatchSampler", "PrefetchStats",
    "SampledSubgraph", "Sampler", "SamplingConfig", "SamplingError", "__version__", "partition_aligned_batches",
    "save_features",
]

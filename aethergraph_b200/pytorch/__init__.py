"""Epoch-level loaders over the GPU minibatch path (the surface of the reference's
`aethergraph.pytorch` package: python/aethergraph/pytorch/__init__.py)."""
from .hetero_loader import HeteroBatch, HeteroLoaderMetrics, HeteroNeighborLoader
from .loader import Batch, LoaderMetrics, NeighborLoader

__all__ = ["Batch", "HeteroBatch", "HeteroLoaderMetrics", "HeteroNeighborLoader", "LoaderMetrics", "NeighborLoader"]

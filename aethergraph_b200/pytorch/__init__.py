"""Epoch-level loaders over the GPU minibatch path (the surface of the reference's
`aethergraph.pytorch` package: python/aethergraph/pytorch/__init__.py)."""
from .loader import Batch, LoaderMetrics, NeighborLoader

__all__ = ["Batch", "LoaderMetrics", "NeighborLoader"]

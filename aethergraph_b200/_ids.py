"""Validation and conversion of node-id arrays (the C ABI indexes nodes with u32).

Same rules as the reference's python/aethergraph/_ids.py: negative ids and ids
past 2**32 - 1 are errors, never silently wrapped.
"""
from __future__ import annotations

import numpy as np

_U32_MAX = int(np.iinfo(np.uint32).max)


def to_uint32_ids(arr, what: str) -> np.ndarray:
    a = np.asarray(arr)
    if a.dtype == np.uint32:
        return a
    if a.size:
        if a.dtype.kind not in "iu":
            if a.dtype.kind == "f" or a.dtype.kind == "b" or a.dtype.kind == "O":
                raise ValueError(f"{what} must be an integer array, got dtype {a.dtype}")
        lo, hi = int(a.min()), int(a.max())
        if lo < 0:
            raise ValueError(f"{what} contains negative node IDs (min {lo})")
        if hi > _U32_MAX:
            raise ValueError(f"{what} contains node IDs exceeding uint32 range (max {hi} > {_U32_MAX})")
    return a.astype(np.uint32, copy=False)

"""Seeded synthetic inputs shared by the tests (host side, numpy)."""
from __future__ import annotations

import numpy as np


def rmat_edges(scale: int, num_edges: int, seed: int, a=0.57, b=0.19, c=0.19, num_nodes=None):
    """R-MAT edge list over 2**scale vertices (endpoints >= num_nodes redrawn)."""
    rng = np.random.default_rng(seed)
    n = num_nodes or (1 << scale)
    src = np.zeros(num_edges, dtype=np.int64)
    dst = np.zeros(num_edges, dtype=np.int64)
    todo = np.arange(num_edges)
    while len(todo):
        s = np.zeros(len(todo), dtype=np.int64)
        d = np.zeros(len(todo), dtype=np.int64)
        for _ in range(scale):
            u = rng.random(len(todo))
            sb = (u >= a + b).astype(np.int64)
            db = (((u >= a) & (u < a + b)) | (u >= a + b + c)).astype(np.int64)
            s = (s << 1) | sb
            d = (d << 1) | db
        ok = (s < n) & (d < n)
        src[todo[ok]] = s[ok]
        dst[todo[ok]] = d[ok]
        todo = todo[~ok]
    return src.astype(np.uint32), dst.astype(np.uint32)


def csr_from_edges(num_nodes: int, src, dst, weights=None):
    """Stable counting sort by source: input order is kept within a row."""
    order = np.argsort(src, kind="stable")
    counts = np.bincount(src, minlength=num_nodes)
    offsets = np.zeros(num_nodes + 1, dtype=np.uint64)
    offsets[1:] = np.cumsum(counts)
    w = None if weights is None else np.asarray(weights, dtype=np.float32)[order]
    return offsets, np.asarray(dst, dtype=np.uint32)[order], w


def rmat_csr(scale: int, avg_degree: int, seed: int, weighted: bool = False, num_nodes=None):
    n = num_nodes or (1 << scale)
    src, dst = rmat_edges(scale, n * avg_degree, seed, num_nodes=n)
    w = None
    if weighted:
        w = np.random.default_rng(seed + 1).lognormal(0.0, 1.0, len(src)).astype(np.float32)
    off, d, w = csr_from_edges(n, src, dst, w)
    return n, off, d, w


ARRAYS = ("nodes", "edge_src", "edge_dst", "edge_ids", "src_local", "dst_local", "seed_locals",
          "num_sampled_nodes", "num_sampled_edges")


def assert_same_subgraph(got: dict, want: dict, ctx: str = ""):
    for k in ARRAYS:
        g, w = got[k], want[k]
        if w is None:
            assert g is None or len(g) == 0, f"{ctx}{k}: expected no array"
            continue
        assert g is not None, f"{ctx}{k}: missing"
        assert len(g) == len(w), f"{ctx}{k}: length {len(g)} != {len(w)}"
        if not np.array_equal(np.asarray(g), np.asarray(w)):
            bad = int(np.nonzero(np.asarray(g) != np.asarray(w))[0][0])
            raise AssertionError(f"{ctx}{k}: first mismatch at {bad}: got {g[bad]}, want {w[bad]}")
    assert got["draws"] == want["draws"], f"{ctx}draws {got['draws']} != {want['draws']}"

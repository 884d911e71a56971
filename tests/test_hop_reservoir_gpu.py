"""Fast-mode one-hop sampler (ag_sample_hop_reservoir) — bit-exact against

1. the CPU oracle's `reservoir_sample` (crates/aethergraph-core/src/internal/philox.rs:59-82),
2. the reference's own CUDA kernel `warp_sample_neighbors`, compiled from the
   reference checkout into oracle/_ref/ (skipped when that library was not built),

on the reference's two kernel tests (crates/aether-stream/tests/kernels/sampler.rs:6-82)
and on R-MAT rows with every fanout regime (copy, Algorithm R, > 32 with replacement).
"""
import os

import numpy as np
import pytest

from helpers import rmat_csr

pytestmark = pytest.mark.gpu
PAD = 0xFFFFFFFF


def _run(ag, g, nodes, fanout, seed, layer):
    from aethergraph_b200.sampler import reservoir_hop

    out, counts = reservoir_hop(g, nodes, fanout, seed, layer)
    return out.cpu().numpy().view(np.uint32), counts.cpu().numpy().view(np.uint32)


def _expect(ago, off, dst, nodes, fanout, seed, layer):
    n = len(off) - 1
    rows = np.full((len(nodes), fanout), PAD, dtype=np.uint32)
    counts = np.zeros(len(nodes), dtype=np.uint32)
    for i, v in enumerate(nodes):
        v = int(v)
        if v >= n:
            continue
        row = dst[int(off[v]):int(off[v + 1])]
        if len(row) == 0:
            continue
        if fanout > 32:  # with replacement: slot d = row[philox(d) % degree] (sampler.cu, fanout > 32 branch)
            rows[i] = [row[ago.philox_u32(seed, layer, v, d) % len(row)] for d in range(fanout)]
            counts[i] = fanout
        else:
            got = ago.reservoir_sample(row, fanout, seed, layer, v)
            rows[i, :len(got)] = got
            counts[i] = len(got)
    return rows, counts


def test_reference_kernel_test_cases():
    import aethergraph_b200 as ag
    from oracle import ago

    # one node of degree 10, fanout 4, seed 7, layer 1 (tests/kernels/sampler.rs:6-37)
    # (110 rows so that the destinations 100..109 are valid vertices of the graph)
    dst = np.arange(100, 110, dtype=np.uint32)
    g = ag.Graph.from_csr(np.array([0, 10] + [10] * 109, dtype=np.uint64), dst)
    rows, counts = _run(ag, g, [0], 4, 7, 1)
    assert rows[0].tolist() == ago.reservoir_sample(dst, 4, 7, 1, 0).tolist() and counts.tolist() == [4]
    # short rows are counted and padded (tests/kernels/sampler.rs:42-82)
    off = np.array([0, 2, 2, 8] + [8] * 13, dtype=np.uint64)
    dst = np.array([5, 6, 10, 11, 12, 13, 14, 15], dtype=np.uint32)
    g = ag.Graph.from_csr(off, dst)
    rows, counts = _run(ag, g, [0, 1, 2, 99], 4, 3, 0)
    assert counts.tolist() == [2, 0, 4, 0]
    assert rows[0].tolist() == [5, 6, PAD, PAD] and rows[1].tolist() == [PAD] * 4 and rows[3].tolist() == [PAD] * 4
    assert all(10 <= v < 16 for v in rows[2])


@pytest.mark.parametrize("fanout", [1, 4, 10, 25, 32, 40])
def test_rmat_rows_match_the_oracle(fanout):
    import aethergraph_b200 as ag
    from oracle import ago

    n, off, dst, _ = rmat_csr(12, 16, seed=9)
    g = ag.Graph.from_csr(off, dst)
    rng = np.random.default_rng(fanout)
    nodes = np.concatenate([rng.integers(0, n, 1500), np.argsort(np.diff(off.astype(np.int64)))[-20:], [n, n + 7]])
    rows, counts = _run(ag, g, nodes, fanout, 0xDEADBEEFCAFE, 3)
    want_rows, want_counts = _expect(ago, off, dst, nodes, fanout, 0xDEADBEEFCAFE, 3)
    assert np.array_equal(counts, want_counts)
    assert np.array_equal(rows, want_rows)


@pytest.mark.parametrize("fanout", [4, 25, 32, 48])
def test_matches_the_reference_cuda_kernel(fanout):
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import _lib
    from oracle import ago

    if not os.path.exists(ago.REF_WARP_SAMPLER):
        pytest.skip("oracle/_ref/libref_warp_sampler.so was not built (no reference checkout at build time)")
    n, off, dst, _ = rmat_csr(13, 16, seed=10)
    g = ag.Graph.from_csr(off, dst)
    rng = np.random.default_rng(1)
    nodes = np.concatenate([rng.integers(0, n, 5000), [n + 1]]).astype(np.uint64)
    rows, counts = _run(ag, g, nodes, fanout, 77, 2)
    # the reference kernel on the very same device arrays
    po, pd, pw = _lib.C.c_void_p(), _lib.C.c_void_p(), _lib.C.c_void_p()
    _lib.check(_lib.lib().ag_graph_device_ptrs(g._h, _lib.C.byref(po), _lib.C.byref(pd), _lib.C.byref(pw)))
    nodes_dev = torch.from_numpy(nodes.view(np.int64)).cuda()
    out = torch.full((len(nodes), fanout), -7, dtype=torch.int32, device="cuda")
    cnt = torch.full((len(nodes),), -7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ago.ref_warp_sample(po.value, pd.value, n, nodes_dev.data_ptr(), out.data_ptr(), cnt.data_ptr(), len(nodes), fanout,
                        77, 2, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert np.array_equal(counts, cnt.cpu().numpy().view(np.uint32))
    assert np.array_equal(rows, out.cpu().numpy().view(np.uint32))

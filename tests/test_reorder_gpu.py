"""GPU: Rabbit Order (host merge inside the library) and the permuted graph (built on
the GPU) against the oracle's restatement, through the C ABI."""
import numpy as np
import pytest

from helpers import assert_same_subgraph, csr_from_edges, rmat_csr

pytestmark = pytest.mark.gpu


def _graphs():
    from test_reorder_cpu import two_cliques

    off, dst = two_cliques()
    yield "two cliques", 8, off, dst, None
    for scale, deg, seed in ((7, 4, 1), (9, 8, 2), (10, 3, 3)):
        n, off, dst, _ = rmat_csr(scale, deg, seed=seed)
        yield f"rmat {scale}", n, off, dst, None
    rng = np.random.default_rng(4)
    src, d = rng.integers(0, 300, 2000), rng.integers(0, 300, 2000)
    d[:100] = src[:100]                                     # self-loops
    off, dd, w = csr_from_edges(300, src, d, rng.random(2000).astype(np.float32))
    yield "random with self-loops and weights", 300, off, dd, w
    yield "no edges", 6, np.zeros(7, np.uint64), np.zeros(0, np.uint32), None
    off, dd, _ = csr_from_edges(400, np.arange(1, 400), np.arange(0, 399))   # a path pointing backwards
    yield "backward path", 400, off, dd, None


def test_rabbit_order_and_permute_match_the_oracle():
    import aethergraph_b200 as ag
    from oracle import ago

    for name, n, off, dst, w in _graphs():
        g = ag.Graph.from_csr(off, dst, w)
        perm, parts = g.reorder_rabbit_with_partitions()
        want_perm, want_parts = ago.rabbit_order(off, dst)
        assert np.array_equal(perm, want_perm), name
        assert np.array_equal(parts, want_parts), name
        assert np.array_equal(g.reorder_rabbit(), perm) and np.array_equal(g.rabbit_partitions(), parts)
        p = g.permute(perm)
        no, nd, nw = ago.permute_csr(off, dst, w, perm)
        o2, d2, w2 = p.to_host()
        assert (p.num_nodes, p.num_edges) == (n, dst.size), name
        assert np.array_equal(o2, no) and np.array_equal(d2, nd), name
        if w is not None:
            assert np.array_equal(w2, nw), name
        # a random permutation too, and back again: the original graph
        rp = np.random.default_rng(7).permutation(n).astype(np.uint32)
        back = g.permute(rp).permute(np.argsort(rp).astype(np.uint32))
        o3, d3, _ = back.to_host()
        assert np.array_equal(o3, off) and np.array_equal(d3, dst), name


def test_permute_rejects_bad_permutations_and_the_result_samples():
    # reorder.rs test_permute_invalid
    import aethergraph_b200 as ag
    from oracle import ago

    n, off, dst, _ = rmat_csr(9, 8, seed=5)
    g = ag.Graph.from_csr(off, dst)
    with pytest.raises(ValueError, match="length mismatch"):
        g.permute(np.arange(n - 1))
    bad = np.arange(n); bad[3] = bad[4]
    with pytest.raises(ValueError, match="duplicate|twice"):
        g.permute(bad)
    bad = np.arange(n); bad[0] = n + 5
    with pytest.raises(ValueError, match="out-of-range"):
        g.permute(bad)
    perm = g.reorder_rabbit()
    p = g.permute(perm)
    no, nd, _ = ago.permute_csr(off, dst, None, perm)
    seeds = np.arange(0, 64, dtype=np.uint32)
    got = ag.NeighborSampler(p, ag.SamplingConfig(num_neighbors=[6, 3], seed=4)).sample(seeds)
    assert_same_subgraph(got.raw_u32(), ago.Sampler(no, nd, [6, 3], seed=4).sample(seeds))
    # batches that follow the communities: every seed once, communities together
    parts = g.rabbit_partitions()
    batches = ag.partition_aligned_batches(parts, np.arange(n), 64)
    assert sorted(np.concatenate(batches).tolist()) == list(range(n))

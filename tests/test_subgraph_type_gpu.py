"""`subgraph_type` "bidirectional" / "induced" on the GPU against the CPU restatements
of the reference's `mirror` / `induce`
(crates/aethergraph-core/src/loader/sampler.rs:972-1040), bit for bit, through the
sampler, the parallel batch sampler and the loader; plus the properties the
reference's own tests assert (python/tests/test_sampler_semantics.py:112-127)."""
import numpy as np
import pytest

from helpers import assert_same_subgraph, csr_from_edges

pytestmark = pytest.mark.gpu


def _ring():
    n = 200
    src = np.repeat(np.arange(n, dtype=np.int64), 6)
    dst = (src + np.tile(np.arange(1, 7, dtype=np.int64) * 7, n)) % n
    return n, csr_from_edges(n, src.astype(np.uint32), dst.astype(np.uint32))


def _want(ago, off, dst, kind, fwd):
    return ago.mirror(fwd) if kind == "bidirectional" else ago.induce(off, dst, fwd)


def test_reference_ring_properties():
    import aethergraph_b200 as ag

    n, (off, dst, _) = _ring()
    g = ag.Graph.from_csr(off, dst)
    sub = ag.Sampler(g, ag.SamplingConfig(num_neighbors=[4, 3], subgraph_type="bidirectional", seed=6)).sample([0, 1, 2])
    pairs = set(map(tuple, sub.edge_index_local.T.tolist()))
    assert len(pairs) == sub.num_edges
    assert all((v, u) in pairs for u, v in pairs)
    assert sum(sub.num_sampled_edges_per_hop) < sub.num_edges  # counts describe the sampling pass
    sub = ag.Sampler(g, ag.SamplingConfig(num_neighbors=[4, 3], subgraph_type="induced", seed=6)).sample([0, 1, 2])
    members = set(sub.nodes.tolist())
    expected = {(int(v), u) for u in members for v in dst[int(off[u]):int(off[u + 1])].tolist() if int(v) in members}
    assert set(map(tuple, sub.edge_index.T.tolist())) == expected
    np.testing.assert_array_equal(sub.edge_index, sub.nodes[sub.edge_index_local])


@pytest.mark.parametrize("kind", ["bidirectional", "induced"])
@pytest.mark.parametrize("replace,track", [(False, True), (True, True), (False, False)])
def test_rewrites_match_the_oracle(kind, replace, track):
    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(17)
    n = 3000
    e = 40_000
    src = rng.integers(0, n, e).astype(np.uint32)
    dst_e = (rng.zipf(1.4, e) % n).astype(np.uint32)
    # mutual pairs and self loops so that reverses already exist
    src = np.concatenate([src, dst_e[:5000], np.arange(50, dtype=np.uint32)])
    dst_e = np.concatenate([dst_e, src[:5000], np.arange(50, dtype=np.uint32)])
    off, dst, _ = csr_from_edges(n, src, dst_e)
    g = ag.Graph.from_csr(off, dst)
    cfg = ag.SamplingConfig(num_neighbors=[6, 4], replace=replace, track_edge_ids=track, subgraph_type=kind, seed=23)
    s = ag.NeighborSampler(g, cfg)
    o = ago.Sampler(off, dst, [6, 4], replace=replace, track_edge_ids=track, seed=23)
    for n_seeds in (1, 40, 700, 0):
        seeds = rng.integers(0, n, n_seeds).astype(np.uint32)
        sg = s.sample(seeds)
        want = _want(ago, off, dst, kind, o.sample(seeds))
        assert_same_subgraph(sg.raw_u32(), want)
        eil = sg.edge_index_local
        assert eil.shape == (2, len(want["src_local"]))
        assert np.array_equal(eil[0], want["dst_local"].astype(np.int64)) and np.array_equal(eil[1], want["src_local"].astype(np.int64))


@pytest.mark.parametrize("kind", ["bidirectional", "induced"])
def test_rewrites_through_the_parallel_sampler_and_the_loader(kind):
    import torch

    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(5)
    n, (off, dst, _) = _ring()
    g = ag.Graph.from_csr(off, dst)
    feats = rng.standard_normal((n, 8)).astype(np.float32)
    store = ag.FeatureStore.from_array(feats, dtype="f32")
    cfg = ag.SamplingConfig(num_neighbors=[3, 3], subgraph_type=kind, seed=9)
    batches = [rng.integers(0, n, 12).astype(np.uint32) for _ in range(10)]
    o = ago.Sampler(off, dst, [3, 3], seed=9)
    wants = []
    for i, b in enumerate(batches):
        o.reseed(ago.batch_seed(9, i))
        wants.append(_want(ago, off, dst, kind, o.sample(b)))
    for sg, want in zip(ag.ParallelBatchSampler(g, cfg).sample_batches(batches), wants):
        assert_same_subgraph(sg.raw_u32(), want)
    with ag.NeighborLoader(g, cfg, prefetch_depth=2, sampler_threads=2, features=store, group=4) as ld:
        for i, b in enumerate(batches):
            ld.submit(i, b)
        for i, want in enumerate(wants):
            idx, sg, x = ld.next_batch()
            assert idx == i
            assert_same_subgraph(sg.raw_u32(), want)
            assert torch.equal(x.cpu(), torch.from_numpy(feats[want["nodes"].astype(np.int64)]))

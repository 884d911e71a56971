"""Heterogeneous sampler on the GPU against the CPU oracle, through the C ABI.

Bit-exact: per-type node ids in discovery order, per-edge-type local indices in
emission order, seed indices and the number of RNG draws.  The cases follow the
reference's own hetero tests (crates/aethergraph-core/src/loader/hetero_sampler.rs
tests module; python/tests/test_hetero.py) on the same "reddit" toy schema, plus
R-MAT relations with reverse edge types for multi-hop, multi-type frontiers.
"""
import numpy as np
import pytest

from helpers import csr_from_edges, rmat_csr

pytestmark = pytest.mark.gpu

USER, POST, COMMENT, SUB = "user", "post", "comment", "subreddit"


def _reddit_edges():
    voted = [(post, user) for user in range(50) for post in range(4)]
    written = [(c, user) for user in range(30) for c in range(3)]
    contains = [(post % 20, post) for post in range(100)]
    return voted, written, contains


def _reddit_graph(ag):
    voted, written, contains = _reddit_edges()

    def arr(pairs):
        return (np.array([p[0] for p in pairs], dtype=np.uint32), np.array([p[1] for p in pairs], dtype=np.uint32))

    return ag.HeteroCsrGraph.from_edge_arrays(
        {USER: 100, POST: 100, COMMENT: 100, SUB: 20},
        [(POST, "voted_by", USER, *arr(voted)), (COMMENT, "written_by", USER, *arr(written)),
         (SUB, "contains", POST, *arr(contains))])


def _reddit_oracle_parts():
    voted, written, contains = _reddit_edges()

    def rel(pairs, n_src):
        pairs = sorted(pairs)
        s = np.array([p[0] for p in pairs], dtype=np.uint32)
        d = np.array([p[1] for p in pairs], dtype=np.uint32)
        off, dd, _ = csr_from_edges(n_src, s, d)
        return off, dd

    return [100, 100, 100, 20], [(1, 0, *rel(voted, 100)), (2, 0, *rel(written, 100)), (0 + 3, 1, *rel(contains, 20))]


ETS = [(POST, "voted_by", USER), (COMMENT, "written_by", USER), (SUB, "contains", POST)]


def _same(got: dict, want: dict):
    assert len(got["nodes"]) == len(want["nodes"])
    for t, (a, b) in enumerate(zip(got["nodes"], want["nodes"])):
        assert np.array_equal(a, b), f"nodes of type {t} differ"
    for e, (a, b) in enumerate(zip(got["edge_src_local"], want["edge_src_local"])):
        assert np.array_equal(a, b), f"edge_src_local of edge type {e} differ"
    for e, (a, b) in enumerate(zip(got["edge_dst_local"], want["edge_dst_local"])):
        assert np.array_equal(a, b), f"edge_dst_local of edge type {e} differ"
    assert np.array_equal(got["seed_indices"], want["seed_indices"])
    assert got["draws"] == want["draws"]


def test_graph_metadata_and_errors():
    import aethergraph_b200 as ag

    g = _reddit_graph(ag)
    assert g.node_types() == [USER, POST, COMMENT, SUB]
    assert g.edge_types() == ETS
    assert g.num_nodes(USER) == 100 and g.num_nodes(SUB) == 20
    assert g.total_nodes() == 320 and g.total_edges() == 200 + 90 + 100
    assert g.num_edges(POST, "voted_by", USER) == 200
    with pytest.raises(KeyError):
        g.num_nodes("nope")
    with pytest.raises(KeyError):
        g.num_edges(USER, "nope", POST)
    e = np.zeros(1, dtype=np.uint32)
    with pytest.raises(ValueError, match="duplicate edge type"):
        ag.HeteroCsrGraph.from_edge_arrays({"a": 2}, [("a", "r", "a", e, e), ("a", "r", "a", e, e)])
    with pytest.raises(ValueError, match="unknown source type"):
        ag.HeteroCsrGraph.from_edge_arrays({"a": 2}, [("b", "r", "a", e, e)])
    with pytest.raises(ValueError, match="same length"):
        ag.HeteroCsrGraph.from_edge_arrays({"a": 2}, [("a", "r", "a", e, np.zeros(2, dtype=np.uint32))])
    with pytest.raises(ValueError, match="failed to build CSR"):
        ag.HeteroCsrGraph.from_edge_arrays({"a": 2, "b": 3}, [("a", "r", "b", np.array([2], dtype=np.uint32), e)])
    with pytest.raises(ValueError, match="at most 16 edge types"):
        ag.HeteroCsrGraph.from_edge_arrays({"a": 2}, [("a", f"r{i}", "a", e, e) for i in range(17)])


def test_in_adjacency_matches_the_stable_transpose():
    import aethergraph_b200 as ag
    from oracle import ago

    g = _reddit_graph(ag)
    num_nodes, rels = _reddit_oracle_parts()
    o = ago.HeteroSampler(num_nodes, rels, [[1]] * 3, seed=1)
    for e, et in enumerate(ETS):
        off, src = g.in_adjacency(*et)
        want_off, want_src = o.in_adjacency(e)
        assert np.array_equal(off, want_off) and np.array_equal(src, want_src)


def test_reference_fixture_cases_match_the_oracle():
    import aethergraph_b200 as ag
    from oracle import ago

    g = _reddit_graph(ag)
    num_nodes, rels = _reddit_oracle_parts()
    # fanouts (2, 1, 0): user 0 voted on 4 posts and wrote 3 comments (hetero_sampler.rs:740-758)
    cfg = ag.HeteroSamplingConfig({ETS[0]: [2], ETS[1]: [1], ETS[2]: [0]}, seed=42)
    sg = ag.HeteroNeighborSampler(g, cfg).sample(USER, [0])
    raw = sg.raw_u32()
    assert [len(e) for e in raw["edge_src_local"]] == [2, 1, 0]
    _same(raw, ago.HeteroSampler(num_nodes, rels, [[2], [1], [0]], seed=42).sample(0, [0]))
    # a duplicate seed expands once (hetero_sampler.rs:898-909)
    cfg = ag.HeteroSamplingConfig({et: [10] for et in ETS}, seed=42)
    sg = ag.HeteroNeighborSampler(g, cfg).sample(USER, np.array([0, 0], dtype=np.int64))
    assert sg.seed_indices.tolist() == [0, 0] and sg.edge_index_local(*ETS[0]).shape == (2, 4)
    assert sg.seeds.tolist() == [0, 0] and sg.seed_type == USER
    _same(sg.raw_u32(), ago.HeteroSampler(num_nodes, rels, [[10]] * 3, seed=42).sample(0, [0, 0]))
    # an edge type left out of num_neighbors draws nothing (aethergraph-py/src/hetero.rs:309-328)
    cfg = ag.HeteroSamplingConfig({ETS[0]: [3, 3]}, seed=9)
    sg = ag.HeteroNeighborSampler(g, cfg).sample(USER, [5, 6, 7])
    _same(sg.raw_u32(), ago.HeteroSampler(num_nodes, rels, [[3, 3], [0, 0], [0, 0]], seed=9).sample(0, [5, 6, 7]))
    assert sg.node_types == [USER, POST] and sg.edge_types == [ETS[0]]


def test_two_hops_stream_continues_and_accessors():
    import aethergraph_b200 as ag
    from oracle import ago

    g = _reddit_graph(ag)
    num_nodes, rels = _reddit_oracle_parts()
    cfg = ag.HeteroSamplingConfig({et: [5, 5] for et in ETS}, seed=42)
    s = ag.HeteroNeighborSampler(g, cfg)
    o = ago.HeteroSampler(num_nodes, rels, [[5, 5]] * 3, seed=42)
    # three batches on one handle: the WyRand stream carries on between them
    for seeds in ([0, 1, 2], [10, 11, 3, 10], list(range(40, 60))):
        sg = s.sample(USER, seeds)
        want = o.sample(0, seeds)
        _same(sg.raw_u32(), want)
        for t, name in enumerate([USER, POST, COMMENT, SUB]):
            assert np.array_equal(sg.nodes(name), want["nodes"][t].astype(np.int64))
            assert np.array_equal(sg.nodes_u32(name), want["nodes"][t])
            assert sg.nodes_t(name).dtype.is_floating_point is False and sg.nodes_t(name).is_cuda
        for e, et in enumerate(ETS):
            ei = sg.edge_index_local(*et)
            assert ei.dtype == np.int64 and ei.shape == (2, len(want["edge_src_local"][e]))
            assert np.array_equal(ei[0], want["edge_src_local"][e]) and np.array_equal(ei[1], want["edge_dst_local"][e])
    # edges point at the expanded node (hetero_sampler.rs:519-545)
    sg = s.sample(USER, [0, 1, 2])
    users, posts = sg.nodes(USER), sg.nodes(POST)
    voted = set(_reddit_edges()[0])
    ei = sg.edge_index_local(*ETS[0])
    assert all((int(posts[a]), int(users[b])) in voted for a, b in zip(ei[0], ei[1]))
    with pytest.raises(KeyError):
        sg.nodes("nope")
    with pytest.raises(KeyError):
        sg.edge_index_local(USER, "x", POST)


def test_seed_errors_and_empty_batch():
    import aethergraph_b200 as ag

    g = _reddit_graph(ag)
    s = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig({et: [2] for et in ETS}, seed=42))
    s.sample(USER, [0, 99])
    with pytest.raises(ag.SamplingError, match="out of range for 20 nodes"):
        s.sample(SUB, [0, 99])  # hetero_sampler.rs:911-929: the bound is the seed type's
    with pytest.raises(ag.SamplingError, match="unknown seed type"):
        s.sample("nope", [0])
    sg = s.sample(USER, [])
    assert sg.node_types == [] and sg.edge_types == [] and sg.seed_indices.shape == (0,)
    with pytest.raises(ag.SamplingError, match="unknown edge type"):
        ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig({(USER, "x", POST): [2]}))
    with pytest.raises(ValueError, match="same number of hops"):
        ag.HeteroSamplingConfig({ETS[0]: [1], ETS[1]: [1, 2]})
    with pytest.raises(ValueError, match="must not be empty"):
        ag.HeteroSamplingConfig({})


def _rmat_hetero(scale_a=12, scale_b=11):
    """Two node types and four edge types (two relations and their reverses, as
    PyG's ToUndirected would add), with hub rows well past any fanout."""
    na, offa, dsta, _ = rmat_csr(scale_a, 12, seed=21)   # a -> a
    nb = 1 << scale_b
    rng = np.random.default_rng(33)
    e = 60_000
    src = (rng.zipf(1.3, e) % na).astype(np.uint32)       # a -> b, skewed
    dst = rng.integers(0, nb, e).astype(np.uint32)
    src_aa = np.repeat(np.arange(na, dtype=np.uint32), np.diff(offa).astype(np.int64))
    return na, nb, (src_aa, dsta.astype(np.uint32)), (src, dst)


@pytest.mark.parametrize("replace", [False, True])
def test_rmat_multi_type_multi_hop_matches_the_oracle(replace):
    import aethergraph_b200 as ag
    from oracle import ago

    na, nb, (s_aa, d_aa), (s_ab, d_ab) = _rmat_hetero()
    ets = [("a", "links", "a"), ("a", "owns", "b"), ("b", "rev_owns", "a"), ("a", "rev_links", "a")]
    edges = [(s_aa, d_aa), (s_ab, d_ab), (d_ab, s_ab), (d_aa, s_aa)]
    g = ag.HeteroCsrGraph.from_edge_arrays({"a": na, "b": nb}, [(*et, *e) for et, e in zip(ets, edges)])
    fan = [[10, 5, 3], [4, 4, 2], [6, 0, 3], [32, 2, 1]]
    cfg = ag.HeteroSamplingConfig({et: f for et, f in zip(ets, fan)}, replace=replace, seed=1234)
    s = ag.HeteroNeighborSampler(g, cfg)
    tid = {"a": 0, "b": 1}
    n_of = {"a": na, "b": nb}
    rels = []
    for (st, _, dt), (src, dst) in zip(ets, edges):
        off, dd, _ = csr_from_edges(n_of[st], src, dst)
        rels.append((tid[st], tid[dt], off, dd))
    o = ago.HeteroSampler([na, nb], rels, fan, replace=replace, seed=1234)
    for e, et in enumerate(ets):
        off, src = g.in_adjacency(*et)
        want_off, want_src = o.in_adjacency(e)
        assert np.array_equal(off, want_off) and np.array_equal(src, want_src)
    rng = np.random.default_rng(8)
    for seed_type, n in (("a", 256), ("b", 300), ("a", 1024), ("b", 1)):
        seeds = rng.integers(0, n_of[seed_type], n).astype(np.uint32)
        sg = s.sample(seed_type, seeds)
        want = o.sample(tid[seed_type], seeds)
        _same(sg.raw_u32(), want)
        assert sum(len(x) for x in want["edge_src_local"]) > n  # the case is not trivially empty
    # reseeding restarts the stream
    s2 = ag.HeteroNeighborSampler(g, cfg)
    o.reseed(1234)
    seeds = rng.integers(0, na, 100).astype(np.uint32)
    _same(s2.sample("a", seeds).raw_u32(), o.sample(0, seeds))


def test_loader_delivers_in_order_with_per_batch_seeds():
    import aethergraph_b200 as ag
    from oracle import ago

    g = _reddit_graph(ag)
    num_nodes, rels = _reddit_oracle_parts()
    cfg = ag.HeteroSamplingConfig({et: [3, 2] for et in ETS}, seed=77)
    rng = np.random.default_rng(2)
    batches = [rng.integers(0, 100, 16).astype(np.int64) for _ in range(24)]
    o = ago.HeteroSampler(num_nodes, rels, [[3, 2]] * 3, seed=77)
    with ag.HeteroNeighborLoader(g, cfg, USER, prefetch_depth=2, sampler_threads=3) as ld:
        assert ld.prefetch_depth == 2
        got = []
        for i, b in enumerate(batches):  # submit a window ahead, as the epoch driver does
            ld.submit(100 + i, b)
            if i >= 4:
                got.append(ld.next_batch())
        while len(got) < len(batches):
            got.append(ld.next_batch())
        for seq, (idx, sg) in enumerate(got):
            assert idx == 100 + seq  # submission order (prefetch.rs:486-491)
            o.reseed(ago.batch_seed(77, seq))
            _same(sg.raw_u32(), o.sample(0, batches[seq].astype(np.uint32)))
        assert ld.stats().total == len(batches)
        with pytest.raises(ag.SamplingError, match="out of range"):
            ld.submit(0, [100])  # test_hetero.py: a seed past its type fails at submit
    assert ld.next_batch() is None  # after shutdown


def test_c4_shaped_schema_down_scaled_matches_the_oracle():
    """The heterogeneous benchmark configuration at 1/1000 scale: user / post /
    comment / subreddit, three stored relations plus their reverses, fanouts
    votes [15,10], writes [10,5], belongs_to [3,2], user seeds."""
    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(44)
    nn = {"user": 50_000, "post": 20_000, "comment": 100_000, "subreddit": 100}

    def skewed(n_src, n_dst, e):
        # every source gets edges, destinations are skewed (hubs far past any fanout)
        return (rng.integers(0, n_src, e).astype(np.uint32), (rng.zipf(1.3, e) % n_dst).astype(np.uint32))

    votes = skewed(nn["user"], nn["post"], 30 * nn["user"])
    writes = skewed(nn["user"], nn["comment"], 8 * nn["user"])
    belongs = (np.arange(nn["post"], dtype=np.uint32), rng.integers(0, nn["subreddit"], nn["post"]).astype(np.uint32))
    ets = [("user", "votes", "post"), ("user", "writes", "comment"), ("post", "belongs_to", "subreddit"),
           ("post", "rev_votes", "user"), ("comment", "rev_writes", "user"), ("subreddit", "rev_belongs_to", "post")]
    edges = [votes, writes, belongs, votes[::-1], writes[::-1], belongs[::-1]]
    fan = [[15, 10], [10, 5], [3, 2], [15, 10], [10, 5], [3, 2]]
    g = ag.HeteroCsrGraph.from_edge_arrays(nn, [(*et, *e) for et, e in zip(ets, edges)])
    s = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig(dict(zip(ets, fan)), seed=42))
    names = list(nn)
    rels = []
    for (st, _, dt), (src, dst) in zip(ets, edges):
        off, dd, _ = csr_from_edges(nn[st], src, dst)
        rels.append((names.index(st), names.index(dt), off, dd))
    o = ago.HeteroSampler([nn[k] for k in names], rels, fan, seed=42)
    for i in range(3):
        seeds = rng.integers(0, nn["user"], 1024).astype(np.uint32)
        sg = s.sample("user", seeds)
        want = o.sample(0, seeds)
        _same(sg.raw_u32(), want)
        assert sum(len(x) for x in want["nodes"]) > 5000 and all(len(x) for x in want["nodes"])


def test_features_ride_the_chain_and_outgrown_reservations_are_regathered():
    """x of a node type == the type's stored rows at its node ids, both when the rows
    fit the space reserved from earlier batches and when a batch outgrows it."""
    import torch

    import aethergraph_b200 as ag

    rng = np.random.default_rng(12)
    nn = {"a": 6000, "b": 3000}
    e1 = (rng.integers(0, 6000, 60_000).astype(np.uint32), rng.integers(0, 3000, 60_000).astype(np.uint32))
    ets = [("a", "to", "b"), ("b", "back", "a")]
    g = ag.HeteroCsrGraph.from_edge_arrays(nn, [(*ets[0], *e1), (*ets[1], *e1[::-1])])
    feats = {"a": ag.FeatureStore.from_array(rng.standard_normal((6000, 32)).astype(np.float32), dtype="bf16"),
             "b": ag.FeatureStore.from_array(rng.standard_normal((3000, 5)).astype(np.float32), dtype="f32")}
    s = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig({ets[0]: [8, 8], ets[1]: [8, 8]}, seed=3), features=feats)
    for n_seeds in (2, 1500, 40, 3000):   # small, far larger (outgrows the reservation), small, larger again
        sg = s.sample("a", rng.integers(0, 6000, n_seeds))
        for nt in nn:
            ids = sg.nodes_t(nt)
            x = sg.x_t(nt)
            assert x.shape == (ids.shape[0], feats[nt].feature_dim)
            assert torch.equal(x, feats[nt].gather(ids))
    plain = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig({ets[0]: [2]}, seed=3)).sample("a", [1, 2])
    assert plain.x_t("a") is None


def test_stream_continues_when_the_handle_grows():
    """One RNG stream per handle across calls, also when a later batch needs more scratch."""
    import aethergraph_b200 as ag
    from oracle import ago

    g = _reddit_graph(ag)
    num_nodes, rels = _reddit_oracle_parts()
    cfg = ag.HeteroSamplingConfig({et: [3, 2] for et in ETS}, seed=5)
    s = ag.HeteroNeighborSampler(g, cfg)
    o = ago.HeteroSampler(num_nodes, rels, [[3, 2]] * 3, seed=5)
    rng = np.random.default_rng(1)
    for ns in (4, 2500, 10, 6000):
        seeds = rng.integers(0, 100, ns).astype(np.uint32)
        _same(s.sample(USER, seeds).raw_u32(), o.sample(0, seeds))


def test_native_loader_features_pool_reuse_and_outgrown_reservations():
    """The native hetero loader over many batches of changing size: x of every type ==
    the stored rows of its node ids (also for a batch that outgrows the rows reserved
    from earlier batches), sampled arrays == the oracle, pooled buffers recycled."""
    import torch

    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(91)
    nn = {"a": 6000, "b": 3000}
    e1 = (rng.integers(0, 6000, 60_000).astype(np.uint32), rng.integers(0, 3000, 60_000).astype(np.uint32))
    ets = [("a", "to", "b"), ("b", "back", "a")]
    g = ag.HeteroCsrGraph.from_edge_arrays(nn, [(*ets[0], *e1), (*ets[1], *e1[::-1])])
    feats = {"a": ag.FeatureStore.from_array(rng.standard_normal((6000, 32)).astype(np.float32), dtype="bf16"),
             "b": ag.FeatureStore.from_array(rng.standard_normal((3000, 5)).astype(np.float32), dtype="f32")}
    rels = []
    for (st, _, dt), (src, dst) in zip(ets, [e1, e1[::-1]]):
        off, dd, _ = csr_from_edges(nn[st], src, dst)
        rels.append((list(nn).index(st), list(nn).index(dt), off, dd))
    fan = [[6, 4], [6, 4]]
    o = ago.HeteroSampler([6000, 3000], rels, fan, seed=19)
    sizes = [4] * 12 + [900] + [4] * 6 + [64] * 20 + [2000] + [64] * 10
    batches = [rng.integers(0, 6000, n).astype(np.int64) for n in sizes]
    cfg = ag.HeteroSamplingConfig(dict(zip(ets, fan)), seed=19)
    with ag.HeteroNeighborLoader(g, cfg, "a", prefetch_depth=3, sampler_threads=2, features=feats, group=4) as ld:
        sub = got = 0
        while got < len(batches):
            while sub < len(batches) and sub - got < 9:
                ld.submit(sub, batches[sub])
                sub += 1
            idx, sg = ld.next_batch()
            assert idx == got
            o.reseed(ago.batch_seed(19, got))
            _same(sg.raw_u32(), o.sample(0, batches[got].astype(np.uint32)))
            for nt in nn:
                ids = sg.nodes_t(nt)
                x = sg.x_t(nt)
                assert x.shape == (ids.shape[0], feats[nt].feature_dim)
                assert torch.equal(x, feats[nt].gather(ids)), (got, nt)
            del sg
            got += 1
        st = ld.stats()
        assert st.total == len(batches) and st.submitted == len(batches)


def test_native_loader_unseeded_delivers_every_batch_once_and_shuts_down():
    import aethergraph_b200 as ag

    g = _reddit_graph(ag)
    cfg = ag.HeteroSamplingConfig({et: [3, 2] for et in ETS})  # no seed: arrival order, each worker its own stream
    rng = np.random.default_rng(5)
    ld = ag.HeteroNeighborLoader(g, cfg, USER, prefetch_depth=2, sampler_threads=3)
    seen = set()
    for i in range(12):
        ld.submit(i, rng.integers(0, 100, 8))
    for _ in range(12):
        idx, sg = ld.next_batch()
        assert idx not in seen
        seen.add(idx)
        assert len(sg.nodes(USER)) >= 1 and sg.seed_indices.shape == (8,)
    assert seen == set(range(12))
    ld.shutdown()
    assert ld.next_batch() is None
    with pytest.raises(ag.SamplingError, match="shut down"):
        ld.submit(99, [1])
    with pytest.raises(RuntimeError, match="prefetch_depth"):
        ag.HeteroNeighborLoader(g, cfg, USER, prefetch_depth=0)
    with pytest.raises(ag.SamplingError, match="unknown seed type"):
        ag.HeteroNeighborLoader(g, cfg, "nobody")

"""GPU parity: the CUDA sampler against the CPU oracle on the same inputs.
Bit-exact for every output array (ids, local ids, edge ids, per-hop counts)."""
import numpy as np
import pytest

from helpers import assert_same_subgraph, csr_from_edges, rmat_csr

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ag():
    import aethergraph_b200 as ag

    return ag


@pytest.fixture(scope="module")
def ago():
    from oracle import ago

    return ago


@pytest.fixture(scope="module")
def rmat12():
    return rmat_csr(12, 16, seed=1)


def _both(ag, ago, csr, fanout, seed, **kw):
    n, off, dst, w = csr
    g = ag.Graph.from_csr(off, dst, w)
    cfg = ag.SamplingConfig(num_neighbors=list(fanout), seed=seed, **kw)
    gpu = ag.NeighborSampler(g, cfg)
    cpu = ago.Sampler(off, dst, fanout, weights=w, replace=kw.get("replace", False),
                      weighted=kw.get("weighted", False), track_edge_ids=kw.get("track_edge_ids", True), seed=seed)
    return g, gpu, cpu


def test_simple_graph_take_all(ag, ago):
    # reference fixture test_data/simple_graph.txt: 0-1 0-2 1-2 1-3 2-3 3-4
    off = np.array([0, 2, 4, 5, 6, 6], dtype=np.uint64)
    dst = np.array([1, 2, 2, 3, 3, 4], dtype=np.uint32)
    _, gpu, cpu = _both(ag, ago, (5, off, dst, None), [2, 2], 42)
    sg = gpu.sample([0, 0, 1])
    assert_same_subgraph(sg.raw_u32(), cpu.sample([0, 0, 1]))
    assert sg.nodes.tolist() == [0, 1, 2, 3, 4]
    assert sg.seed_indices.tolist() == [0, 0, 1]
    assert sg.num_sampled_nodes_per_hop == [2, 2, 1]
    assert sg.num_sampled_edges_per_hop == [4, 2]
    # row 0 = sampled neighbor, row 1 = expanded node; edge_ids name the stored edge row1 -> row0
    ei = sg.edge_index
    assert ei[1].tolist() == [0, 0, 1, 1, 2, 3] and ei[0].tolist() == [1, 2, 2, 3, 3, 4]
    assert sg.edge_ids.tolist() == [0, 1, 2, 3, 4, 5]
    nodes = sg.nodes
    assert np.array_equal(nodes[sg.edge_index_local], ei)


@pytest.mark.parametrize("fanout", [[15, 10], [25, 10], [5, 5, 5], [3], [40, 3], [1, 1, 1, 1], [0, 4], [16, 33]])
def test_uniform_exact_parity(ag, ago, rmat12, fanout):
    n = rmat12[0]
    _, gpu, cpu = _both(ag, ago, rmat12, fanout, seed=42)
    rng = np.random.default_rng(7)
    for call in range(3):  # the RNG stream continues across calls
        seeds = rng.integers(0, n, size=128).astype(np.uint32)
        seeds[5] = seeds[3]  # duplicate seed
        assert_same_subgraph(gpu.sample(seeds).raw_u32(), cpu.sample(seeds), f"call {call} ")


def test_large_batch_parity(ag, ago):
    csr = rmat_csr(16, 16, seed=3)
    _, gpu, cpu = _both(ag, ago, csr, [25, 10], seed=5)
    seeds = np.random.default_rng(1).integers(0, csr[0], size=6000).astype(np.uint32)
    got = gpu.sample(seeds)
    assert_same_subgraph(got.raw_u32(), cpu.sample(seeds))
    assert got.num_edges > 100_000  # several hundred scan tiles: exercises the look-back chain


def test_replace_parity(ag, ago, rmat12):
    _, gpu, cpu = _both(ag, ago, rmat12, [10, 5], seed=9, replace=True)
    seeds = np.arange(100, 200, dtype=np.uint32)
    for _ in range(2):
        assert_same_subgraph(gpu.sample(seeds).raw_u32(), cpu.sample(seeds))


def test_no_edge_ids(ag, ago, rmat12):
    _, gpu, cpu = _both(ag, ago, rmat12, [10, 5], seed=9, track_edge_ids=False)
    seeds = np.arange(64, dtype=np.uint32)
    got = gpu.sample(seeds)
    assert_same_subgraph(got.raw_u32(), cpu.sample(seeds))
    assert len(got.edge_ids) == 0


def test_reseed_matches_batch_seed(ag, ago, rmat12):
    n, off, dst, _ = rmat12
    g = ag.Graph.from_csr(off, dst)
    cfg = ag.SamplingConfig(num_neighbors=[15, 10], seed=42)
    pbs = ag.ParallelBatchSampler(g, cfg, streams=3)
    cpu = ago.Sampler(off, dst, [15, 10], seed=42)
    rng = np.random.default_rng(11)
    pos = 0
    for call in range(2):  # successive calls continue the stream of positions
        batches = [rng.integers(0, n, size=64).astype(np.uint32) for _ in range(7)]
        out = pbs.sample_batches(batches)
        for b, sg in zip(batches, out):
            cpu.reseed(ago.batch_seed(42, pos))
            assert_same_subgraph(sg.raw_u32(), cpu.sample(b), f"position {pos} ")
            pos += 1


def test_weighted_parity(ag, ago):
    csr = rmat_csr(11, 24, seed=4, weighted=True)
    _, gpu, cpu = _both(ag, ago, csr, [15, 10, 5], seed=17, weighted=True)
    seeds = np.random.default_rng(2).integers(0, csr[0], size=64).astype(np.uint32)
    for _ in range(2):
        assert_same_subgraph(gpu.sample(seeds).raw_u32(), cpu.sample(seeds))


def test_weighted_bad_weights(ag, ago):
    # non-finite and non-positive weights get an infinite key (sampler.rs:1448-1455)
    off = np.array([0, 8, 8], dtype=np.uint64)
    dst = np.array([1, 1, 1, 1, 1, 1, 1, 1], dtype=np.uint32)
    w = np.array([1.0, np.nan, 0.0, -2.0, np.inf, 3.0, 0.5, 2.0], dtype=np.float32)
    _, gpu, cpu = _both(ag, ago, (2, off, dst, w), [6], seed=3, weighted=True)
    got, want = gpu.sample([0]).raw_u32(), cpu.sample([0])
    assert_same_subgraph(got, want)
    assert set(got["edge_ids"][:4].tolist()) == {0, 5, 6, 7}  # the four usable weights win first


def test_empty_and_isolated(ag, ago):
    off = np.array([0, 0, 1, 1], dtype=np.uint64)
    dst = np.array([0], dtype=np.uint32)
    _, gpu, cpu = _both(ag, ago, (3, off, dst, None), [2, 2], seed=1)
    for seeds in ([], [0], [2, 2], [1]):
        s = np.array(seeds, dtype=np.uint32)
        assert_same_subgraph(gpu.sample(s).raw_u32(), cpu.sample(s), f"seeds {seeds} ")


def test_seed_out_of_range(ag, rmat12):
    n, off, dst, _ = rmat12
    g = ag.Graph.from_csr(off, dst)
    s = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[2], seed=1))
    with pytest.raises(ag.SamplingError, match=r"seed node %d \(position 1\) is out of range for %d nodes" % (n, n)):
        s.sample(np.array([0, n], dtype=np.int64))
    with pytest.raises(ag.SamplingError, match="out of u32 range"):
        s.sample(np.array([-1], dtype=np.int64))
    assert s.sample([0]).num_seeds == 1  # the handle is still usable


def test_config_errors(ag, rmat12):
    n, off, dst, _ = rmat12
    g = ag.Graph.from_csr(off, dst)
    with pytest.raises(ValueError, match="non-empty"):
        ag.SamplingConfig(num_neighbors=[])
    with pytest.raises(ValueError, match="non-negative"):
        ag.SamplingConfig(num_neighbors=[3, -1])
    with pytest.raises(ValueError, match="no edge weights"):
        ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[3], weighted=True))
    for kw in ({"temporal_strategy": "last"}, {"cumulative": True, "disjoint": True}):
        with pytest.raises(ValueError, match="not supported"):
            ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[3], **kw))
    # disjoint (seed by seed) and cumulative (hop by hop) are compositions of launch chains: the plain
    # sampler and the loader run them, the parallel batch sampler (groups of batches per chain) does not
    with pytest.raises(ValueError, match="disjoint sampling in a parallel batch sampler"):
        ag.ParallelBatchSampler(g, ag.SamplingConfig(num_neighbors=[3], disjoint=True, seed=1))
    with pytest.raises(ValueError, match="cumulative sampling in a parallel batch sampler"):
        ag.ParallelBatchSampler(g, ag.SamplingConfig(num_neighbors=[3], cumulative=True, seed=1))


def test_loader_runs_disjoint_and_cumulative_batches_in_order(ag):
    """Behind the loader interface both modes are sampled on demand, batch `seq` from
    batch_seed(seed, seq) like every other batch (prefetch.rs:926-930)."""
    from oracle import ago

    n, off, dst, _ = rmat_csr(10, 8, seed=6)
    g = ag.Graph.from_csr(off, dst)
    feats = ag.FeatureStore.from_array(np.random.default_rng(0).standard_normal((n, 8)).astype(np.float32), "f32")
    rng = np.random.default_rng(2)
    batches = [rng.integers(0, n, 12).astype(np.uint32) for _ in range(4)]
    with ag.NeighborLoader(g, ag.SamplingConfig(num_neighbors=[4, 2], seed=3, cumulative=True), features=feats) as ld:
        ld.submit_epoch(batches, [10, 11, 12, 13])
        for i, b in enumerate(batches):
            idx, sg, x = ld.next_batch()
            want = ago.sample_cumulative(off, dst, [4, 2], b, seed=ago.batch_seed(3, i))
            assert idx == 10 + i and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
            assert np.array_equal(sg.raw_u32()["edge_ids"], want["edge_ids"])
            assert np.array_equal(x.cpu().numpy(), feats.get_batch(want["nodes"].astype(np.int64)))
        assert ld.stats().total == 4 and ld.try_next() is None
    with ag.NeighborLoader(g, ag.SamplingConfig(num_neighbors=[4, 2], seed=3, disjoint=True)) as ld:
        for i, b in enumerate(batches):
            ld.submit(i, b)
        for i, b in enumerate(batches):
            idx, sg, x = ld.next_batch()
            oracle = ago.Sampler(off, dst, [4, 2], seed=ago.batch_seed(3, i))
            want = ago.sample_disjoint(oracle, b)
            assert idx == i and x is None and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
            assert np.array_equal(sg.batch, want["batch"])


@pytest.mark.parametrize("kw", [{}, {"replace": True}, {"weighted": True}])
def test_cumulative_sampling_matches_the_oracle(ag, kw):
    """Every hop expands all nodes seen so far and an edge of an earlier hop is refused
    (sampler.rs:834-837, 1250-1258, 1277-1285; test cumulative_mode_emits_each_edge_once
    :3362-3390); the stream runs on from call to call."""
    from oracle import ago

    n, off, dst, w = rmat_csr(10, 8, seed=6, weighted=True)
    g = ag.Graph.from_csr(off, dst, w)
    feats = ag.FeatureStore.from_array(np.random.default_rng(0).standard_normal((n, 16)).astype(np.float32), "f32")
    fan = [5, 3, 2]
    sampler = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=fan, seed=6, cumulative=True, **kw), features=feats)
    okw = dict(kw, weights=w) if kw.get("weighted") else kw
    draw = 0
    for seeds in (np.array([0, 1, 2, 1], dtype=np.uint32), np.arange(40, 90, dtype=np.uint32), np.zeros(0, np.uint32)):
        sg = sampler.sample(seeds)
        want = ago.sample_cumulative(off, dst, fan, seeds, seed=6, start_draw=draw, **okw)
        draw = want["draws"]
        got = sg.raw_u32()
        for k in ("nodes", "edge_src", "edge_dst", "src_local", "dst_local", "seed_locals", "edge_ids",
                  "num_sampled_nodes", "num_sampled_edges"):
            assert np.array_equal(got[k], want[k]), (k, len(seeds))
        e, at, seen = got["edge_ids"], 0, set()
        for c in got["num_sampled_edges"]:
            hop = set(e[at:at + int(c)].tolist())
            assert not (seen & hop), "a later hop re-emitted an edge"
            seen |= hop
            at += int(c)
        if not kw.get("replace"):
            assert len(set(e.tolist())) == len(e), "cumulative mode repeated an edge"
        if len(seeds):
            assert np.array_equal(sg.x.cpu().numpy(), feats.get_batch(want["nodes"].astype(np.int64)))
            assert np.array_equal(sg.edge_index_local, np.stack([want["dst_local"], want["src_local"]]).astype(np.int64))


@pytest.mark.parametrize("kw", [{}, {"replace": True}, {"weighted": True}, {"subgraph_type": "bidirectional"}])
def test_disjoint_sampling_matches_the_oracle(ag, kw):
    """Every seed its own block, the RNG stream running on from block to block, local indices
    shifted per block, `batch` naming each node's seed (sampler.rs:600-690); repeated and
    isolated seeds included."""
    from oracle import ago

    n, off, dst, w = rmat_csr(10, 8, seed=6, weighted=True)
    g = ag.Graph.from_csr(off, dst, w)
    feats = ag.FeatureStore.from_array(np.random.default_rng(0).standard_normal((n, 16)).astype(np.float32), "f32")
    cfg = ag.SamplingConfig(num_neighbors=[4, 3], seed=12, disjoint=True, **kw)
    okw = {k: v for k, v in kw.items() if k != "subgraph_type"}
    oracle = ago.Sampler(off, dst, [4, 3], seed=12, weights=w if kw.get("weighted") else None, **okw)
    deg = np.diff(off.astype(np.int64))
    isolated = int(np.flatnonzero(deg == 0)[0]) if (deg == 0).any() else 0
    seeds = np.array([5, 9, 5, isolated, 700, 1, 2, 3], dtype=np.uint32)
    sampler = ag.NeighborSampler(g, cfg, features=feats)
    for _ in range(2):                                     # the stream also runs on from call to call
        sg = sampler.sample(seeds)
        want = ago.sample_disjoint(oracle, seeds, off, dst, kw.get("subgraph_type", "directional"))
        got = sg.raw_u32()
        for k in ("nodes", "edge_src", "edge_dst", "src_local", "dst_local", "seed_locals", "num_sampled_nodes",
                  "num_sampled_edges"):
            assert np.array_equal(got[k], want[k]), k
        assert np.array_equal(sg.batch, want["batch"])
        assert np.array_equal(sg.edge_index_local, np.stack([want["dst_local"], want["src_local"]]).astype(np.int64))
        assert np.array_equal(sg.seed_indices, want["seed_locals"].astype(np.int64))
        assert np.array_equal(sg.x.cpu().numpy(), feats.get_batch(want["nodes"].astype(np.int64)))
        assert got["nodes"][got["seed_locals"]].tolist() == seeds.tolist()


def test_philox_mode_invariants_and_uniformity(ag, rmat12):
    from scipy import stats

    n, off, dst, _ = rmat12
    g = ag.Graph.from_csr(off, dst)
    s = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[10, 5], seed=3, rng_mode="philox"))
    seeds = np.arange(256, dtype=np.uint32)
    raw = s.sample(seeds).raw_u32()
    # structural invariants (sampler.rs:2299-2369, 3423-3444)
    assert np.array_equal(raw["nodes"][raw["src_local"]], raw["edge_src"])
    assert np.array_equal(raw["nodes"][raw["dst_local"]], raw["edge_dst"])
    assert len(np.unique(raw["edge_ids"])) == len(raw["edge_ids"])
    assert np.array_equal(dst[raw["edge_ids"]], raw["edge_dst"])
    assert len(np.unique(raw["nodes"])) == len(raw["nodes"])
    # chi-square: picks of a hub row are uniform over its positions
    hub = int(np.argmax(np.diff(off.astype(np.int64))))
    deg = int(off[hub + 1] - off[hub])
    k = 8
    counts = np.zeros(deg)
    trials = 3000
    for t in range(trials):
        s1 = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[k], seed=1000 + t, rng_mode="philox"))
        r = s1.sample([hub]).raw_u32()
        counts[(r["edge_ids"] - off[hub]).astype(np.int64)] += 1
    # fold positions into 16 bins so every expected count is large
    bins = np.add.reduceat(counts, np.linspace(0, deg, 17)[:-1].astype(int))
    widths = np.diff(np.append(np.linspace(0, deg, 17)[:-1].astype(int), deg))
    expected = trials * k * widths / deg
    p = stats.chisquare(bins, expected).pvalue
    assert p > 0.01, p


def test_weighted_hub_rows_match_the_oracle():
    """Rows far longer than the fanout (block-per-row path, with the single-precision
    pre-filter in front of the f64 keys), next to ordinary rows, zero weights included."""
    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(77)
    n = 60_000
    hubs = {0: 50_000, 7: 9000, 11: 4097, 13: 4096}
    src = [np.full(d, v, dtype=np.uint32) for v, d in hubs.items()]
    dst = [rng.integers(0, n, d).astype(np.uint32) for d in hubs.values()]
    rest = rng.integers(0, n, 300_000).astype(np.uint32)
    src.append(rest)
    dst.append(rng.integers(0, n, 300_000).astype(np.uint32))
    dst.append(np.array([0, 7, 11, 13] * 50, dtype=np.uint32))   # edges INTO the hubs, so later hops expand them
    src.append(rng.integers(100, n, 200).astype(np.uint32))
    src, dst = np.concatenate(src), np.concatenate(dst)
    w = rng.lognormal(0.0, 1.0, len(src)).astype(np.float32)
    w[rng.integers(0, len(w), 2000)] = 0.0
    off, d2, w2 = csr_from_edges(n, src, dst, w)
    g = ag.Graph.from_csr(off, d2, w2)
    for fan, seeds in (([15, 10, 5], [0, 7, 11, 13, 5, 9]), ([32], [0, 0, 7]),
                       ([8, 8], rng.integers(0, n, 700).tolist() + [0, 11])):
        cfg = ag.SamplingConfig(num_neighbors=fan, weighted=True, seed=21)
        got = ag.NeighborSampler(g, cfg).sample(seeds).raw_u32()
        want = ago.Sampler(off, d2, fan, weights=w2, weighted=True, seed=21).sample(np.array(seeds, dtype=np.uint32))
        assert_same_subgraph(got, want)
        assert len(want["edge_dst"]) > len(seeds)


def test_stream_continues_across_calls_of_any_size():
    """Consecutive calls on one handle consume ONE RNG stream (the reference's sampler is
    `&mut self` with a persistent generator): also when a later call is larger than any
    before it and the handle has to grow its scratch memory in between."""
    import aethergraph_b200 as ag
    from oracle import ago

    n, off, dst, w = rmat_csr(13, 10, seed=31, weighted=True)
    g = ag.Graph.from_csr(off, dst, w)
    rng = np.random.default_rng(4)
    for kw in (dict(), dict(replace=True), dict(weighted=True)):
        cfg = ag.SamplingConfig(num_neighbors=[6, 3], seed=99, **kw)
        s = ag.NeighborSampler(g, cfg)
        o = ago.Sampler(off, dst, [6, 3], weights=w if kw.get("weighted") else None, seed=99, **kw)
        for ns in (5, 3000, 40, 7000, 1):   # 3000 and 7000 exceed the scratch sized for the call before
            seeds = rng.integers(0, n, ns).astype(np.uint32)
            assert_same_subgraph(s.sample(seeds).raw_u32(), o.sample(seeds))

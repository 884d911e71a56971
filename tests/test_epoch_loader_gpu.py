"""Epoch driver (`aethergraph_b200.pytorch.NeighborLoader`) against the CPU oracle.

Every batch of an epoch must be what the reference produces for the same
arguments: seeds from the same batch getter, sampled from
batch_seed(epoch seed, batch number) (python/aethergraph/pytorch/loader.py:195-205,
crates/aethergraph-core/src/loader/prefetch.rs:926-930), delivered in order, with
the feature rows of `n_id`.  Bit-exact.
"""
import numpy as np
import pytest

from helpers import rmat_csr

pytestmark = pytest.mark.gpu


def _graph_and_features(ag, scale=12, dim=24):
    n, off, dst, _ = rmat_csr(scale, 10, seed=17)
    g = ag.Graph.from_csr(off, dst)
    feats = np.random.default_rng(5).standard_normal((n, dim)).astype(np.float32)
    return n, off, dst, g, feats


def _expect(ago, off, dst, fanout, epoch_seed, b, seeds, **kw):
    s = ago.Sampler(off, dst, fanout, seed=ago.batch_seed(epoch_seed, b), **kw)
    return s.sample(np.asarray(seeds, dtype=np.uint32))


def _check_batch(data, want, feats, seeds, input_id):
    n_id = data.n_id.cpu().numpy()
    assert np.array_equal(n_id, want["nodes"].astype(np.int64))
    ei = data.edge_index.cpu().numpy()
    assert ei.shape == (2, len(want["dst_local"]))
    assert np.array_equal(ei[0], want["dst_local"]) and np.array_equal(ei[1], want["src_local"])
    assert np.array_equal(data.e_id.cpu().numpy(), want["edge_ids"].astype(np.int64))
    assert np.array_equal(data.seed_index.cpu().numpy(), want["seed_locals"].astype(np.int64))
    assert np.array_equal(data.input_id.cpu().numpy(), input_id)
    assert data.batch_size == len(seeds) and data.num_nodes == len(n_id)
    assert np.array_equal(n_id[data.seed_index.cpu().numpy()], seeds)
    assert list(data.num_sampled_nodes) == want["num_sampled_nodes"].tolist()
    assert list(data.num_sampled_edges) == want["num_sampled_edges"].tolist()
    if feats is not None:
        assert data.x.is_cuda and np.array_equal(data.x.cpu().numpy().view(np.uint32), feats[n_id].view(np.uint32))


def test_all_nodes_in_order_matches_the_oracle_and_epochs_resample():
    import aethergraph_b200 as ag
    from aethergraph_b200.pytorch import NeighborLoader
    from aethergraph_b200.pytorch.loader import epoch_sampling_seed
    from oracle import ago

    n, off, dst, g, feats = _graph_and_features(ag)
    fanout, bs = [6, 4], 500
    loader = NeighborLoader(g, fanout, batch_size=bs, shuffle=False, seed=7, features=feats, num_workers=2,
                            prefetch_factor=3)
    assert len(loader) == (n + bs - 1) // bs
    ss = np.random.SeedSequence(7)
    first_epoch = None
    for epoch in range(2):
        es = epoch_sampling_seed(ss)
        count = 0
        for b, data in enumerate(loader):
            seeds = np.arange(b * bs, min((b + 1) * bs, n), dtype=np.int64)
            _check_batch(data, _expect(ago, off, dst, fanout, es, b, seeds), feats, seeds, seeds)
            if b == 0:
                if epoch == 0:
                    first_epoch = data.edge_index.cpu().numpy()
                else:  # a new epoch draws new neighborhoods for the same seeds
                    assert not np.array_equal(first_epoch, data.edge_index.cpu().numpy())
            count += 1
        assert count == len(loader)
        m = loader.metrics
        assert m.batches_processed == count and m.total_time_ms > 0 and 0.0 <= m.prefetch_hit_rate <= 1.0
        assert m.prefetch_hits + m.prefetch_misses == count
    # a loader built with the same seed replays the same epochs
    again = NeighborLoader(g, fanout, batch_size=bs, shuffle=False, seed=7, features=feats)
    assert np.array_equal(next(iter(again)).edge_index.cpu().numpy(), first_epoch)


def test_shuffled_input_nodes_mask_and_strided_permutation():
    import aethergraph_b200 as ag
    from aethergraph_b200.pytorch import NeighborLoader
    from aethergraph_b200.pytorch.loader import epoch_sampling_seed
    from oracle import ago

    n, off, dst, g, feats = _graph_and_features(ag, scale=11)
    fanout, bs = [5, 3], 128
    mask = np.zeros(n, dtype=bool)
    mask[::3] = True
    nodes = np.nonzero(mask)[0].astype(np.int64)
    loader = NeighborLoader(g, fanout, input_nodes=mask, batch_size=bs, shuffle=True, seed=11, features=feats,
                            transform=lambda d: d)
    order = np.random.default_rng(11).spawn(1)[0].permutation(len(nodes))   # loader.py:155-156
    es = epoch_sampling_seed(np.random.SeedSequence(11))
    seen = []
    for b, data in enumerate(loader):
        pos = order[b * bs:(b + 1) * bs]
        _check_batch(data, _expect(ago, off, dst, fanout, es, b, nodes[pos]), feats, nodes[pos], pos)
        seen.append(nodes[pos])
    assert np.array_equal(np.sort(np.concatenate(seen)), nodes)
    # all nodes + shuffle: the coprime-stride walk visits every node exactly once (loader.py:169-184)
    loader = NeighborLoader(g, [2], batch_size=200, shuffle=True, seed=3, track_edge_ids=False)
    got = [d for d in loader]
    assert all(d.e_id is None and d.x is None for d in got)
    ids = np.concatenate([d.n_id.cpu().numpy()[d.seed_index.cpu().numpy()] for d in got])
    assert np.array_equal(np.sort(ids), np.arange(n))
    assert not np.array_equal(ids, np.arange(n))


def test_early_break_custom_sampler_and_argument_errors():
    import aethergraph_b200 as ag
    from aethergraph_b200.pytorch import NeighborLoader

    n, off, dst, g, feats = _graph_and_features(ag, scale=10)
    loader = NeighborLoader(g, [3, 2], batch_size=64, seed=1)
    for i, data in enumerate(loader):
        if i == 2:
            break  # the generator's cleanup shuts the native loader down
    assert loader.metrics.batches_processed == 3
    calls = []
    custom = NeighborLoader(g, [3], batch_size=256, shuffle=False,
                            neighbor_sampler=lambda graph, seeds: calls.append(len(seeds)) or len(seeds))
    assert list(custom) == calls and sum(calls) == n
    with pytest.raises(ValueError, match="float32"):
        NeighborLoader(g, [3], features=feats.astype(np.float64))
    with pytest.raises(ValueError, match="does not match graph num_nodes"):
        NeighborLoader(g, [3], features=feats[:-1])
    with pytest.raises(ValueError, match="out-of-range node IDs"):
        NeighborLoader(g, [3], input_nodes=[0, n])
    with pytest.raises(ValueError, match="unrecognized feature_source"):
        NeighborLoader(g, [3], feature_source="http://x")
    with pytest.raises(NotImplementedError):
        NeighborLoader(g, [3], input_time=np.zeros(4))
    with pytest.raises(ValueError, match="not both"):
        NeighborLoader(g, [3], features=feats, feature_path="x.bin")


def test_hetero_epoch_loader_matches_the_oracle():
    """python/aethergraph/pytorch/hetero_loader.py:289-404: per-type n_id / x, per-edge-type
    edge_index, seed_index / input_id / batch_size on the seed type, batches in order."""
    import aethergraph_b200 as ag
    from aethergraph_b200.pytorch import HeteroNeighborLoader
    from aethergraph_b200.pytorch.loader import epoch_sampling_seed
    from helpers import csr_from_edges
    from oracle import ago

    rng = np.random.default_rng(6)
    nn = {"user": 3000, "item": 1500}
    buys = (rng.integers(0, 3000, 20_000).astype(np.uint32), (rng.zipf(1.5, 20_000) % 1500).astype(np.uint32))
    ets = [("user", "buys", "item"), ("item", "rev_buys", "user")]
    edges = [buys, buys[::-1]]
    g = ag.HeteroCsrGraph.from_edge_arrays(nn, [(*et, *e) for et, e in zip(ets, edges)])
    fan = {ets[0]: [4, 3], ets[1]: [6, 2]}
    feats = {"user": rng.standard_normal((3000, 16)).astype(np.float32),
             "item": rng.standard_normal((1500, 8)).astype(np.float32)}
    ids = np.arange(0, 3000, 2)
    loader = HeteroNeighborLoader(g, fan, input_nodes=("user", ids), batch_size=256, shuffle=True, seed=5,
                                  num_workers=2, prefetch_factor=3, features=feats)
    assert len(loader) == (len(ids) + 255) // 256
    order = np.random.default_rng(5).spawn(1)[0].permutation(len(ids))
    es = epoch_sampling_seed(np.random.SeedSequence(5))
    rels = []
    for (st, _, dt), (src, dst) in zip(ets, edges):
        off, dd, _ = csr_from_edges(nn[st], src, dst)
        rels.append((["user", "item"].index(st), ["user", "item"].index(dt), off, dd))
    o = ago.HeteroSampler([3000, 1500], rels, [fan[ets[0]], fan[ets[1]]], seed=0)
    count = 0
    for b, data in enumerate(loader):
        pos = order[b * 256:(b + 1) * 256]
        o.reseed(ago.batch_seed(es, b))
        want = o.sample(0, ids[pos].astype(np.uint32))
        for t, nt in enumerate(["user", "item"]):
            n_id = data[nt].n_id.cpu().numpy()
            assert np.array_equal(n_id, want["nodes"][t].astype(np.int64)) and data[nt].num_nodes == len(n_id)
            assert np.array_equal(data[nt].x.cpu().numpy().view(np.uint32), feats[nt][n_id].view(np.uint32))
        for e, et in enumerate(ets):
            ei = data[et].edge_index.cpu().numpy()
            assert np.array_equal(ei[0], want["edge_src_local"][e]) and np.array_equal(ei[1], want["edge_dst_local"][e])
        u = data["user"]
        assert u.batch_size == len(pos) and np.array_equal(u.input_id.cpu().numpy(), pos)
        assert np.array_equal(u.seed_index.cpu().numpy(), want["seed_indices"].astype(np.int64))
        count += 1
    assert count == len(loader) and loader.metrics.batches_processed == count
    with pytest.raises(ValueError, match="input_nodes is required"):
        HeteroNeighborLoader(g, fan)
    with pytest.raises(ValueError, match="same number of hops"):
        HeteroNeighborLoader(g, {ets[0]: [1], ets[1]: [1, 2]}, input_nodes=("user", None))


def test_disjoint_epoch_batches_carry_the_batch_vector():
    """`disjoint=True`: every seed its own block, `data.batch` names each node's seed
    (python/aethergraph/pytorch/loader.py:985-991); sampled from batch_seed(epoch seed, b)."""
    import aethergraph_b200 as ag
    from aethergraph_b200.pytorch import NeighborLoader
    from aethergraph_b200.pytorch.loader import epoch_sampling_seed
    from oracle import ago

    n, off, dst, g, feats = _graph_and_features(ag, scale=9, dim=8)
    ids = np.arange(0, 40)
    loader = NeighborLoader(g, [3, 2], batch_size=16, shuffle=False, seed=5, features=feats, input_nodes=ids,
                            disjoint=True)
    es = epoch_sampling_seed(np.random.SeedSequence(5))
    seen = 0
    for b, data in enumerate(loader):
        seeds = ids[b * 16:(b + 1) * 16]
        want = ago.sample_disjoint(ago.Sampler(off, dst, [3, 2], seed=ago.batch_seed(es, b)), seeds)
        n_id = data.n_id.cpu().numpy()
        assert np.array_equal(n_id, want["nodes"].astype(np.int64))
        assert np.array_equal(data.batch.cpu().numpy(), want["batch"])
        assert np.array_equal(data.seed_index.cpu().numpy(), want["seed_locals"].astype(np.int64))
        assert np.array_equal(data.x.cpu().numpy().view(np.uint32), feats[n_id].view(np.uint32))
        assert np.array_equal(n_id[data.seed_index.cpu().numpy()], seeds)
        seen += 1
    assert seen == 3

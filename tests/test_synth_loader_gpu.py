"""GPU: the synthetic generators against their CPU twin, and the prefetching loader
against the oracle (ordering, reseeding, errors, shutdown)."""
import threading
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ag():
    import aethergraph_b200 as ag

    return ag


@pytest.fixture(scope="module")
def ago():
    from oracle import ago

    return ago


@pytest.mark.parametrize("n,e", [(1 << 12, 1 << 16), (5000, 60000), (1, 10), (300, 0)])
def test_rmat_matches_cpu_twin(ag, ago, n, e):
    from aethergraph_b200 import synth

    g = synth.rmat_graph(n, e, seed=11)
    off, dst, w = g.to_host()
    off2, dst2 = ago.synth_rmat_csr(n, n, e, 11, threads=4)
    assert np.array_equal(off, off2) and np.array_equal(dst, dst2)
    assert w is None and g.num_edges == e
    # rows are sorted by destination
    if e:
        row = np.repeat(np.arange(n), np.diff(off.astype(np.int64)))
        key = row.astype(np.int64) << 32 | dst
        assert np.all(np.diff(key) >= 0)


@pytest.mark.parametrize("n,e,budget", [(1 << 12, 1 << 16, 5000), (5000, 60000, 1), (70_001, 400_000, 150_000)])
def test_rmat_built_in_source_ranges_is_the_same_graph(ag, ago, n, e, budget, monkeypatch):
    """Graphs whose sort keys exceed the free device memory are built a range of source
    ids at a time; forced here with a small budget of edges per range (weights included)."""
    from aethergraph_b200 import synth

    monkeypatch.setenv("AG_SYNTH_PARTITION_EDGES", str(budget))
    g = synth.rmat_graph(n, e, seed=11, weight_sigma=1.0)
    monkeypatch.delenv("AG_SYNTH_PARTITION_EDGES")
    whole = synth.rmat_graph(n, e, seed=11, weight_sigma=1.0)
    off, dst, w = g.to_host()
    off2, dst2, w2 = whole.to_host()
    assert np.array_equal(off, off2) and np.array_equal(dst, dst2) and np.array_equal(w, w2)
    off3, dst3 = ago.synth_rmat_csr(n, n, e, 11, threads=4)
    assert np.array_equal(off, off3) and np.array_equal(dst, dst3)


def test_rmat_is_skewed_and_weighted(ag):
    from aethergraph_b200 import synth

    g = synth.rmat_graph(1 << 14, 1 << 18, seed=5, weight_sigma=1.0)
    off, dst, w = g.to_host()
    deg = np.diff(off.astype(np.int64))
    assert deg.max() > 20 * deg.mean()          # power-law-ish hubs
    assert (deg == 0).mean() > 0.1              # and many isolated rows
    assert w is not None and np.all(w > 0)
    assert abs(np.log(w).mean()) < 0.02 and abs(np.log(w).std() - 1.0) < 0.02


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_features_match_cpu_twin(ag, ago, dtype):
    from aethergraph_b200 import synth

    n, dim = 3000, 96
    f = synth.features(n, dim, dtype, seed=9)
    assert np.array_equal(f.payload_to_host(), ago.synth_features(n, dim, dtype, 9, threads=3))
    shard = synth.features(n, dim, dtype, seed=9, row_range=(1000, 1800))
    assert np.array_equal(shard.payload_to_host(), ago.synth_features(n, dim, dtype, 9, (1000, 1800)))
    x = f.features()
    assert abs(x.mean()) < 0.01 and abs(x.std() - 1.0) < 0.01
    # a shard answers for its own rows only
    ids = np.array([1000, 1799], dtype=np.int64)
    assert np.array_equal(shard.get_batch(ids), f.get_batch(ids))
    with pytest.raises(ValueError, match="not held by this shard"):
        shard.get_batch(np.array([5], dtype=np.int64))


@pytest.fixture(scope="module")
def world(ag):
    from aethergraph_b200 import synth

    n = 1 << 13
    g = synth.rmat_graph(n, n * 16, seed=1)
    feats = synth.features(n, 32, "f16", seed=2)
    off, dst, _ = g.to_host()
    return n, g, feats, off, dst, feats.payload_to_host()


@pytest.mark.parametrize("threads", [1, 4])
def test_loader_order_reseed_and_features(ag, ago, world, threads):
    from aethergraph_b200 import synth

    n, g, feats, off, dst, payload = world
    cfg = ag.SamplingConfig(num_neighbors=[15, 10], seed=42)
    cpu = ago.Sampler(off, dst, [15, 10], seed=42)
    with ag.NeighborLoader(g, cfg, prefetch_depth=2, sampler_threads=threads, features=feats) as loader:
        assert loader.has_features and loader.feature_dim == 32 and loader.num_nodes == n
        batches = [synth.seed_batch(n, 64, 3, b) for b in range(12)]
        got = []

        def consume():
            for _ in batches:
                got.append(loader.next_batch())

        t = threading.Thread(target=consume)
        t.start()
        for i, b in enumerate(batches):
            loader.submit(100 + i, b)  # batch_idx is only echoed back
        t.join(60)
        assert not t.is_alive()
        for i, (idx, sg, x) in enumerate(got):
            assert idx == 100 + i  # submission order, whatever the pool size
            cpu.reseed(ago.batch_seed(42, i))
            want = cpu.sample(batches[i])
            raw = sg.raw_u32()
            for k in ("nodes", "edge_dst", "edge_ids", "src_local", "dst_local", "seed_locals"):
                assert np.array_equal(raw[k], want[k]), (i, k)
            xw = ago.gather(payload, n, 32, "f16", want["nodes"])
            assert np.array_equal(x.cpu().numpy().view(np.uint32), xw.view(np.uint32))
        st = loader.stats()
        assert st.total == 12 and st.hits + st.misses == 12 and 0.0 <= st.hit_rate <= 1.0
        assert st.edges == sum(s.num_edges for _, s, _ in got)


def test_loader_unseeded_and_errors(ag, world):
    n, g, feats, off, dst, _ = world
    cfg = ag.SamplingConfig(num_neighbors=[5], seed=None)
    loader = ag.NeighborLoader(g, cfg, prefetch_depth=1, sampler_threads=2)
    assert not loader.has_features and loader.feature_dim is None
    for i in range(6):
        loader.submit(i, np.arange(10, dtype=np.uint32))
    seen = sorted(loader.next_batch()[0] for _ in range(6))
    assert seen == list(range(6))  # completion order, every batch_idx echoed once
    with pytest.raises(ag.SamplingError, match="out of range"):
        loader.submit(7, np.array([n], dtype=np.int64))
    assert loader.try_next() is None
    # a consumer blocked in next_batch() is released by shutdown() and sees None
    out = []
    t = threading.Thread(target=lambda: out.append(loader.next_batch()))
    t.start()
    time.sleep(0.2)
    loader.shutdown()
    t.join(10)
    assert not t.is_alive() and out == [None]
    assert loader.next_batch() is None
    with pytest.raises(RuntimeError, match="shut down"):
        loader.submit(8, [1])


def test_loader_backpressure_does_not_deadlock(ag, world):
    n, g, feats, _, _, _ = world
    cfg = ag.SamplingConfig(num_neighbors=[10, 5], seed=7)
    with ag.NeighborLoader(g, cfg, prefetch_depth=1, sampler_threads=3, features=feats) as loader:
        total = 40  # far more than the 8 x depth work queue and the depth-1 result channel
        done = []

        def consume():
            for _ in range(total):
                done.append(loader.next_batch()[0])

        t = threading.Thread(target=consume)
        t.start()
        for i in range(total):
            loader.submit(i, np.arange(i, i + 32, dtype=np.uint32))
        t.join(60)
        assert done == list(range(total))


def test_seed_sequence_makes_batches_independent_of_the_rank_count(ag, ago, world):
    """Rank r of W ranks takes global batches r, r + W, ... and sets the loader's seed
    sequence to (r, W): every global batch is then sampled from batch_seed(seed, b),
    whatever W is (the property the reference tests for its thread pool,
    crates/aethergraph-core/src/loader/sampler.rs:3116-3148)."""
    n, g, feats, off, dst, payload = world
    cfg = ag.SamplingConfig(num_neighbors=[5, 3], seed=77)
    s = ago.Sampler(off, dst, [5, 3], seed=77)
    rng = np.random.default_rng(1)
    batches = [rng.integers(0, n, 64).astype(np.uint32) for _ in range(12)]
    for W in (1, 2, 3):
        for r in range(W):
            mine = list(range(r, len(batches), W))
            with ag.NeighborLoader(g, cfg, prefetch_depth=4, sampler_threads=2, group=4, seed_sequence=(r, W)) as ld:
                ld.submit_epoch([batches[b] for b in mine], mine)
                for b in mine:
                    idx, sg, _ = ld.next_batch()
                    s.reseed(ago.batch_seed(77, b))
                    want = s.sample(batches[b])
                    assert idx == b
                    got = sg.raw_u32()
                    for k in ("nodes", "edge_dst", "src_local", "dst_local"):
                        assert np.array_equal(got[k], want[k]), (W, r, b, k)
    with ag.NeighborLoader(g, cfg, prefetch_depth=2, sampler_threads=1) as ld:
        ld.submit(0, batches[0])
        from aethergraph_b200 import _lib
        assert _lib.lib().ag_loader_set_seed_sequence(ld._h, 1, 2) == _lib.AG_ERR_VALUE  # only before the first submit
        ld.next_batch()


def test_pooled_x_is_reserved_from_observed_counts_and_outgrown_batches_are_gathered_again(ag, ago, world):
    """The loader's own batch buffers reserve feature rows for 1.5 x the largest batch seen
    so far, not for the worst-case bound; a batch that outgrows the reservation gets every
    row all the same (exact second gather), and later buffers are sized for it."""
    n, g, feats, off, dst, payload = world
    cfg = ag.SamplingConfig(num_neighbors=[10, 5], seed=21)
    s = ago.Sampler(off, dst, [10, 5], seed=21)
    rng = np.random.default_rng(3)
    small = [rng.integers(0, n, 300)[:2].astype(np.uint32) for _ in range(6)]
    big = [rng.integers(0, n, 300).astype(np.uint32) for _ in range(6)]
    with ag.NeighborLoader(g, cfg, prefetch_depth=4, sampler_threads=1, features=feats, group=2) as ld:
        seq = 0
        for phase in (small, big, small):
            ld.submit_epoch(phase, list(range(seq, seq + len(phase))))
            for b in phase:
                idx, sg, x = ld.next_batch()
                s.reseed(ago.batch_seed(21, seq))
                want = s.sample(b)
                assert idx == seq and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
                xw = ago.gather(payload, n, 32, "f16", want["nodes"])
                assert x.shape[0] == len(want["nodes"])
                assert np.array_equal(x.cpu().numpy().view(np.uint32), xw.view(np.uint32)), seq
                seq += 1
                del sg, x   # hand the pooled buffers back


def test_batches_given_back_early_or_read_on_a_side_stream(ag, ago, world):
    """`release(stream)` hands a pooled batch back before the object dies (a second release and
    the later destructor do nothing), `record_stream` names the stream that still reads it:
    the loader keeps delivering exact batches out of the few buffers it has."""
    import torch

    n, g, feats, off, dst, payload = world
    cfg = ag.SamplingConfig(num_neighbors=[8, 4], seed=9)
    s = ago.Sampler(off, dst, [8, 4], seed=9)
    rng = np.random.default_rng(11)
    batches = [rng.integers(0, n, 200).astype(np.uint32) for _ in range(40)]
    side = torch.cuda.Stream()
    kept = []
    with ag.NeighborLoader(g, cfg, prefetch_depth=2, sampler_threads=1, features=feats, group=2) as ld:
        ld.submit_epoch(batches[:8], list(range(8)))
        for i, b in enumerate(batches):
            idx, sg, x = ld.next_batch()
            if i + 8 < len(batches):
                ld.submit(i + 8, batches[i + 8])
            s.reseed(ago.batch_seed(9, i))
            want = s.sample(b)
            assert idx == i and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
            if i % 3 == 0:
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    total = x.sum()                       # read on the side stream ...
                sg.record_stream(side)                    # ... which the loader must wait for
                xw = ago.gather(payload, n, 32, "f16", want["nodes"])
                side.synchronize()
                assert np.isclose(float(total), float(xw.astype(np.float64).sum()), rtol=1e-3)
            elif i % 3 == 1:
                assert np.array_equal(x.cpu().numpy().view(np.uint32),
                                      ago.gather(payload, n, 32, "f16", want["nodes"]).view(np.uint32))
                sg.release(torch.cuda.current_stream())
                sg.release()                              # harmless
                kept.append(sg)                           # the destructor must not give it back twice
            del x

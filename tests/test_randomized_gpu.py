"""Randomized parity sweeps (fixed seeds, bounded): random graphs x sampling configs x
call sequences on the GPU against the CPU oracle, bit for bit.  They cover the
combinations the hand-written cases do not enumerate — skewed and hub-heavy rows,
every sampling mode at 1-4 hops, consecutive calls of changing size on one handle
(one RNG stream, scratch regrown in between), random heterogeneous schemas with
features, and the loader at random thread / group / depth settings.
"""
import numpy as np
import pytest

from helpers import assert_same_subgraph, csr_from_edges

pytestmark = pytest.mark.gpu


def _random_graph(rng, weighted):
    n = int(rng.choice([50, 700, 5000, 40000]))
    e = int(n * rng.choice([1, 4, 20]))
    src = (rng.zipf(1.5, e) % n if rng.random() < 0.5 else rng.integers(0, n, e)).astype(np.uint32)
    dst = (rng.zipf(1.3, e) % n if rng.random() < 0.5 else rng.integers(0, n, e)).astype(np.uint32)
    if rng.random() < 0.3:  # a few giant rows (block-per-row path of the weighted picks, long Floyd rows)
        hub = rng.integers(0, n, 2)
        extra = int(rng.choice([3000, 9000, 20000]))
        src = np.concatenate([src, np.repeat(hub, extra).astype(np.uint32)])
        dst = np.concatenate([dst, rng.integers(0, n, 2 * extra).astype(np.uint32)])
    w = rng.lognormal(0, 1, len(src)).astype(np.float32) if weighted else None
    if weighted and rng.random() < 0.5:
        w[rng.integers(0, len(w), len(w) // 10)] = 0.0
    return (n, *csr_from_edges(n, src, dst, w))


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_sampler_call_sequences(seed):
    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(seed)
    for _ in range(40):
        weighted = rng.random() < 0.4
        n, off, dst, w = _random_graph(rng, weighted)
        g = ag.Graph.from_csr(off, dst, w)
        fan = [int(rng.choice([1, 2, 5, 10, 25, 32] + ([] if weighted else [40, 100]))) for _ in range(int(rng.integers(1, 5)))]
        replace = (not weighted) and rng.random() < 0.3
        s_seed = int(rng.integers(0, 2**63))
        s = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=fan, weighted=weighted, replace=replace, seed=s_seed))
        o = ago.Sampler(off, dst, fan, weights=w, weighted=weighted, replace=replace, seed=s_seed)
        for _call in range(3):
            seeds = rng.integers(0, n, int(rng.choice([1, 7, 128, 1024, 3000]))).astype(np.uint32)
            try:
                got = s.sample(seeds).raw_u32()
            except ValueError as ex:  # a worst-case bound past the per-batch limits is refused up front
                assert "batch too large" in str(ex)
                break
            assert_same_subgraph(got, o.sample(seeds))


@pytest.mark.parametrize("seed", [21, 22])
def test_hetero_schemas_with_features(seed):
    import torch

    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(seed)
    for _ in range(30):
        nt, et = int(rng.integers(1, 6)), int(rng.integers(1, 9))
        names = [f"t{i}" for i in range(nt)]
        nn = {nm: int(rng.choice([1, 30, 800, 20000])) for nm in names}
        ets, edges, rels = [], [], []
        for e in range(et):
            s_t, d_t = names[int(rng.integers(0, nt))], names[int(rng.integers(0, nt))]
            m = int(rng.choice([0, 10, 2000, 60000]))
            a = (rng.zipf(1.5, m) % nn[s_t] if rng.random() < 0.5 else rng.integers(0, nn[s_t], m)).astype(np.uint32)
            b = (rng.zipf(1.3, m) % nn[d_t] if rng.random() < 0.5 else rng.integers(0, nn[d_t], m)).astype(np.uint32)
            ets.append((s_t, f"r{e}", d_t))
            edges.append((a, b))
            off, dd, _ = csr_from_edges(nn[s_t], a, b)
            rels.append((names.index(s_t), names.index(d_t), off, dd))
        hops = int(rng.integers(1, 4))
        fan = [[int(rng.choice([0, 1, 3, 8, 32])) for _ in range(hops)] for _ in range(et)]
        replace = bool(rng.random() < 0.3)
        s_seed = int(rng.integers(0, 2**63))
        g = ag.HeteroCsrGraph.from_edge_arrays(nn, [(*t, *ed) for t, ed in zip(ets, edges)])
        feats = {nm: ag.FeatureStore.from_array(rng.standard_normal((nn[nm], int(rng.choice([3, 8, 64])))).astype(np.float32),
                                                dtype=str(rng.choice(["f32", "f16", "bf16"])))
                 for nm in names if rng.random() < 0.6}
        s = ag.HeteroNeighborSampler(g, ag.HeteroSamplingConfig(dict(zip(ets, fan)), replace=replace, seed=s_seed),
                                     features=feats or None)
        o = ago.HeteroSampler([nn[k] for k in names], rels, fan, replace=replace, seed=s_seed)
        for _call in range(3):
            st = names[int(rng.integers(0, nt))]
            seeds = rng.integers(0, nn[st], int(rng.choice([0, 1, 9, 300, 2000]))).astype(np.uint32)
            sg = s.sample(st, seeds)
            want = o.sample(names.index(st), seeds)
            got = sg.raw_u32()
            for k in ("nodes", "edge_src_local", "edge_dst_local"):
                for a, b in zip(got[k], want[k]):
                    assert np.array_equal(a, b), k
            assert np.array_equal(got["seed_indices"], want["seed_indices"]) and got["draws"] == want["draws"]
            for nm, f in feats.items():
                ids = sg.nodes_t(nm)
                if ids.shape[0]:
                    assert torch.equal(sg.x_t(nm), f.gather(ids)), nm


@pytest.mark.parametrize("seed", [31, 32])
def test_loader_settings_and_feature_layouts(seed):
    import aethergraph_b200 as ag
    from oracle import ago

    rng = np.random.default_rng(seed)
    for _ in range(25):
        weighted = rng.random() < 0.3
        n, off, dst, w = _random_graph(rng, weighted)
        g = ag.Graph.from_csr(off, dst, w)
        fan = [int(rng.choice([1, 3, 10, 25])) for _ in range(int(rng.integers(1, 4)))]
        replace = (not weighted) and rng.random() < 0.3
        s_seed = int(rng.integers(0, 2**63))
        dim, dtype = int(rng.choice([1, 7, 16, 64, 100, 256])), str(rng.choice(["f32", "f16", "bf16"]))
        feats_np = rng.standard_normal((n, dim)).astype(np.float32)
        store = ag.FeatureStore.from_array(feats_np, dtype=dtype) if rng.random() < 0.7 else None
        payload = ago.encode(feats_np, dtype) if store is not None else None
        cfg = ag.SamplingConfig(num_neighbors=fan, weighted=weighted, replace=replace, seed=s_seed)
        threads, group, depth = int(rng.integers(1, 5)), int(rng.choice([1, 2, 8, 16])), int(rng.integers(1, 6))
        o = ago.Sampler(off, dst, fan, weights=w, weighted=weighted, replace=replace, seed=s_seed)
        batches = [rng.integers(0, n, int(rng.choice([0, 1, 33, 500, 1500]))).astype(np.uint32)
                   for _ in range(int(rng.integers(1, 30)))]
        with ag.NeighborLoader(g, cfg, prefetch_depth=depth, sampler_threads=threads, features=store, group=group) as ld:
            sub = got = 0
            window = max(1, min(8 * depth - 1, threads * group + 2))
            while got < len(batches):
                while sub < len(batches) and sub - got < window:
                    ld.submit(1000 + sub, batches[sub])
                    sub += 1
                idx, sg, x = ld.next_batch()
                o.reseed(ago.batch_seed(s_seed, got))
                want = o.sample(batches[got])
                assert idx == 1000 + got
                assert_same_subgraph(sg.raw_u32(), want)
                if store is not None:
                    xw = ago.gather(payload, n, dim, dtype, want["nodes"])
                    assert np.array_equal(x.cpu().numpy().view(np.uint32).reshape(-1), xw.view(np.uint32).reshape(-1))
                got += 1

"""Weighted sampling on the GPU, pinned as far as the reference's algorithm pins it.

The reference selects the k winners of a row by Efraimidis-Spirakis keys
(crates/aethergraph-core/src/loader/sampler.rs:1418-1469): one 64-bit WyRand draw
per row position in row order, u = ((bits >> 11) + 1) * 2^-53, key = -ln(u) / w, the
k smallest keys win.  The SET of winners is therefore a function of the algorithm
alone and is checked here against an independent numpy restatement (not through the
CPU oracle).  The ORDER in which the winners are emitted comes from Rust libcore's
select_nth_unstable_by and cannot be pinned; frequencies are checked against exact
inclusion probabilities instead (chi-square, p > 0.01), and the reference's own
statistical case (the heavy edge wins more than half of 1000 trials,
sampler.rs:2574-2618) is replayed on the GPU.
"""
import itertools

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

M64 = (1 << 64) - 1


def wyrand_draws(seed: int, n: int) -> list[int]:
    """The first n outputs of WyRand seeded `seed` (internal/genstamp.rs:181-202)."""
    out, state = [], seed & M64
    for _ in range(n):
        state = (state + 0xA0761D6478BD642F) & M64
        t = state * (state ^ 0xE7037ED1A0B428DB)
        out.append(((t >> 64) ^ t) & M64)
    return out


def es_keys(bits: list[int], w: np.ndarray) -> np.ndarray:
    u = (np.array([b >> 11 for b in bits], dtype=np.float64) + 1.0) * (1.0 / 9007199254740992.0)
    w = w.astype(np.float64)
    keys = np.full(len(w), np.inf)
    ok = np.isfinite(w) & (w > 0)
    keys[ok] = -np.log(u[ok]) / w[ok]
    return keys


@pytest.mark.parametrize("k", [3, 10, 32, 40, 100])
def test_one_hop_winner_sets_follow_the_reference_algorithm(k):
    import aethergraph_b200 as ag
    from helpers import rmat_csr

    n, off, dst, w = rmat_csr(11, 24, seed=21, weighted=True)
    g = ag.Graph.from_csr(off, dst, w)
    seeds = np.random.default_rng(k).permutation(n)[:300].astype(np.uint32)   # distinct, so each row is expanded once
    seed = 1000 + k
    sg = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[k], weighted=True, seed=seed)).sample(seeds)
    raw = sg.raw_u32()
    deg = np.diff(off.astype(np.int64))
    total_draws = int(sum(deg[s] for s in seeds if deg[s] > k))
    draws = wyrand_draws(seed, total_draws)
    at, sampled_rows = 0, 0
    for s in seeds:
        d, o = int(deg[s]), int(off[s])
        got = np.sort(raw["edge_ids"][raw["edge_src"] == s].astype(np.int64) - o)
        if d <= k:
            assert np.array_equal(got, np.arange(d)), "take-all row"
            continue
        keys = es_keys(draws[at:at + d], w[o:o + d])
        at += d
        order = np.lexsort((np.arange(d), keys))          # by key, ties by row position
        assert np.array_equal(got, np.sort(order[:k])), f"row {s}: winners differ from the k smallest keys"
        sampled_rows += 1
    assert sampled_rows > 5 and raw["draws"] == total_draws


def test_inclusion_frequencies_match_exact_efraimidis_spirakis():
    """20 000 independent copies of one 5-neighbour row, k = 2: the ten possible winner
    sets must occur with their exact probabilities (sum over both orders of
    w_a / W * w_b / (W - w_a))."""
    from scipy import stats

    import aethergraph_b200 as ag

    copies, weights, k = 20_000, np.array([1.0, 2.0, 3.0, 4.0, 5.0], dtype=np.float32), 2
    deg = len(weights)
    n = copies + deg
    off = np.concatenate([np.arange(copies + 1) * deg, np.full(deg, copies * deg)]).astype(np.uint64)
    dst = np.tile(np.arange(copies, copies + deg, dtype=np.uint32), copies)
    g = ag.Graph.from_csr(off, dst, np.tile(weights, copies))
    counts = {c: 0 for c in itertools.combinations(range(deg), k)}
    for part in range(4):   # several batches: the picks of a batch restart from its own seed
        seeds = np.arange(part * copies // 4, (part + 1) * copies // 4, dtype=np.uint32)
        raw = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[k], weighted=True, seed=77 + part)).sample(seeds).raw_u32()
        pos = (raw["edge_ids"].astype(np.int64) - raw["edge_src"].astype(np.int64) * deg).reshape(-1, k)
        assert len(pos) == len(seeds)
        for a, b in np.sort(pos, axis=1):
            counts[(int(a), int(b))] += 1
    W = float(weights.sum())
    expect = []
    for a, b in counts:
        wa, wb = float(weights[a]), float(weights[b])
        expect.append(copies * (wa / W * wb / (W - wa) + wb / W * wa / (W - wb)))
    chi2, p = stats.chisquare(list(counts.values()), expect)
    assert p > 0.01, f"chi-square {chi2:.1f}, p = {p:.4f}"


def test_heavy_edge_wins_most_trials():
    """sampler.rs:2574-2618: one neighbour of weight 100 among three of weight 1, one pick
    per trial, 1000 trials with seeds 123, 124, ...: the heavy edge must win more than half
    (expected 100 / 103)."""
    import aethergraph_b200 as ag

    off = np.array([0, 4, 4, 4, 4, 4], dtype=np.uint64)
    g = ag.Graph.from_csr(off, np.array([1, 2, 3, 4], dtype=np.uint32), np.array([100.0, 1.0, 1.0, 1.0], dtype=np.float32))
    heavy = 0
    for trial in range(1000):
        s = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[1], weighted=True, seed=123 + trial))
        sg = s.sample(np.array([0], dtype=np.uint32)).raw_u32()
        assert len(sg["edge_dst"]) == 1
        heavy += int(sg["edge_dst"][0] == 1)
    assert heavy > 500, f"the heavy edge won {heavy} of 1000 trials"


@pytest.mark.parametrize("fanout", [[40], [64, 3], [5, 100]])
def test_large_weighted_fanout_matches_the_oracle(fanout):
    """Fanouts above 32 (a block per row, buffered top-k): every array bit for bit."""
    import aethergraph_b200 as ag
    from helpers import assert_same_subgraph, rmat_csr
    from oracle import ago

    n, off, dst, w = rmat_csr(11, 40, seed=5, weighted=True)
    g = ag.Graph.from_csr(off, dst, w)
    seeds = np.random.default_rng(1).integers(0, n, 150).astype(np.uint32)
    got = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=fanout, weighted=True, seed=9)).sample(seeds).raw_u32()
    want = ago.Sampler(off, dst, fanout, weights=w, weighted=True, seed=9).sample(seeds)
    assert_same_subgraph(got, want)
    assert want["num_sampled_edges"][0] > 0


@pytest.mark.parametrize("fanout", [[4], [10, 5], [40, 3]])
def test_weighted_with_replacement_matches_the_oracle(fanout):
    """sampler.rs:1383-1412: k draws over the row's cumulative weights (f64 sums in row
    order), repeats allowed.  Every array bit for bit, loader included."""
    import aethergraph_b200 as ag
    from helpers import assert_same_subgraph, rmat_csr
    from oracle import ago

    n, off, dst, w = rmat_csr(11, 20, seed=8, weighted=True)
    g = ag.Graph.from_csr(off, dst, w)
    seeds = np.random.default_rng(2).integers(0, n, 200).astype(np.uint32)
    cfg = ag.SamplingConfig(num_neighbors=fanout, weighted=True, replace=True, seed=13)
    s = ag.NeighborSampler(g, cfg)
    o = ago.Sampler(off, dst, fanout, weights=w, weighted=True, replace=True, seed=13)
    for _ in range(2):   # the handle's stream continues across calls
        assert_same_subgraph(s.sample(seeds).raw_u32(), o.sample(seeds))
    with ag.NeighborLoader(g, cfg, prefetch_depth=2, sampler_threads=2, group=4) as ld:
        ld.submit_epoch([seeds[:50], seeds[50:120], seeds[120:]])
        for i, part in enumerate((seeds[:50], seeds[50:120], seeds[120:])):
            _, sg, _ = ld.next_batch()
            o.reseed(ago.batch_seed(13, i))
            assert_same_subgraph(sg.raw_u32(), o.sample(part))


def test_heavy_edge_with_replacement_as_the_reference_tests_it():
    """sampler.rs:2574-2618 verbatim: weights [100, 1, 1, 1], fanout [1], replace = true,
    seeds 123 + trial; the heavy edge must win more than 500 of 1000 trials."""
    import aethergraph_b200 as ag

    off = np.array([0, 4, 4, 4, 4, 4], dtype=np.uint64)
    g = ag.Graph.from_csr(off, np.array([1, 2, 3, 4], dtype=np.uint32), np.array([100.0, 1.0, 1.0, 1.0], dtype=np.float32))
    heavy = 0
    for trial in range(1000):
        s = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[1], weighted=True, replace=True, seed=123 + trial))
        sg = s.sample(np.array([0], dtype=np.uint32)).raw_u32()
        assert len(sg["edge_dst"]) == 1
        heavy += int(sg["edge_dst"][0] == 1)
    assert heavy > 500, f"the heavy edge won {heavy} of 1000 trials"

"""CPU tests: the oracle against every known answer and invariant the reference's
own tests hold for the minibatch path (file:line cites are the reference's).
No GPU needed."""
import os
import zlib

import numpy as np
import pytest

from helpers import csr_from_edges, rmat_csr
from oracle import ago

MASK = (1 << 64) - 1


# ------------------------------------------------------------------- RNGs --
def test_philox_random123_zero_vector():
    # crates/aethergraph-core/src/internal/philox.rs:88-94
    assert ago.philox4x32_10(0, 0, 0) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def test_philox_counter_dimensions_and_lane_packing():
    # philox.rs:96-103, 116-122
    s = ago.philox4x32_10(42, 3, 99)
    assert s == ago.philox4x32_10(42, 3, 99)
    assert s != ago.philox4x32_10(42, 4, 99) and s != ago.philox4x32_10(43, 3, 99) and s != ago.philox4x32_10(42, 3, 100)
    full = ago.philox4x32_10(1, 2, 3, 0)
    assert [ago.philox_u32(1, 2, 3, i) for i in range(4)] == full
    assert ago.philox_u32(1, 2, 3, 5) == ago.philox4x32_10(1, 2, 3, 1)[1]


def test_reservoir_is_deterministic_sized_and_matches_algorithm_r():
    # philox.rs:105-114 and the GPU test crates/aethergraph-stream/tests/kernels/sampler.rs:6-37
    nb = np.arange(20, dtype=np.uint32)
    a = ago.reservoir_sample(nb, 5, 7, 1, 3)
    assert len(a) == 5 and np.array_equal(a, ago.reservoir_sample(nb, 5, 7, 1, 3)) and set(a) <= set(nb)
    # independent restatement of Algorithm R with the same draws
    res = list(nb[:5])
    for t in range(5, 20):
        j = ago.philox_u32(7, 1, 3, t) % (t + 1)
        if j < 5:
            res[j] = int(nb[t])
    assert list(a) == res
    assert list(ago.reservoir_sample(nb[:3], 5, 7, 1, 3)) == [0, 1, 2]  # fanout >= degree: the whole row
    assert len(ago.reservoir_sample(nb[:0], 5, 7, 1, 3)) == 0


def _splitmix_batch_seed(base, idx):
    # crates/aethergraph-core/src/loader/sampler.rs:69-75
    z = (base ^ (idx * 0x9E3779B97F4A7C15)) & MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def test_batch_seed_is_the_splitmix_finalizer():
    for base, idx in [(0, 0), (42, 0), (42, 1), (2**64 - 1, 12345), (7, 2**40)]:
        assert ago.batch_seed(base, idx) == _splitmix_batch_seed(base, idx)
    assert len({ago.batch_seed(42, i) for i in range(1000)}) == 1000


def test_wyrand_stream_and_random_access_agree():
    # crates/aethergraph-core/src/internal/genstamp.rs:181-202, 268-276
    def wy(seed, n):
        out, st = [], seed
        for _ in range(n):
            st = (st + 0xA0761D6478BD642F) & MASK
            t = st * (st ^ 0xE7037ED1A0B428DB)
            out.append(((t >> 64) ^ t) & MASK)
        return out
    for seed in (0, 42, 2**64 - 5):
        want = wy(seed, 64)
        assert list(ago.wyrand_stream(seed, 64)) == want            # same seed, same stream
        assert [ago.wyrand_at(seed, d) for d in range(64)] == want  # draw d is a function of (seed, d)


def test_neg_ln_is_finite_and_monotone():
    # sampler.rs:43-55
    assert ago.neg_ln_u64(2**64 - 1) == 0.0
    assert np.isfinite(ago.neg_ln_u64(0)) and ago.neg_ln_u64(0) > 36.0
    assert ago.neg_ln_u64(1 << 63) == pytest.approx(-np.log(0.5 + 2.0**-53), rel=1e-15)


# ---------------------------------------------------------------- codecs --
def test_f16_decode_every_pattern_matches_ieee():
    bits = np.arange(65536, dtype=np.uint16)
    got = ago.decode(bits, "f16").view(np.uint32)
    want = bits.view(np.float16).astype(np.float32).view(np.uint32)
    nan = np.isnan(bits.view(np.float16))
    assert np.array_equal(got[~nan], want[~nan])
    # NaN: payload kept, quiet bit set (what half 2.x and the F16C converts produce)
    assert np.array_equal(got[nan], want[nan] | 0x00400000)


def test_bf16_decode_every_pattern_is_a_shift():
    # internal/simd.rs:233-238
    bits = np.arange(65536, dtype=np.uint16)
    assert np.array_equal(ago.decode(bits, "bf16").view(np.uint32), bits.astype(np.uint32) << 16)


def test_encoders_round_to_nearest_even():
    import torch

    rng = np.random.default_rng(0)
    x = np.concatenate([
        (rng.standard_normal(200_000) * 10.0 ** rng.integers(-8, 6, 200_000)).astype(np.float32),
        np.array([0, -0.0, np.inf, -np.inf, 65504, 65520, 65519.99, 1e-8, 6e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                  2.99e-8, 1e38, -3e38, 1e-40], dtype=np.float32)])
    with np.errstate(over="ignore"):
        want16 = x.astype(np.float16).view(np.uint16)
    assert np.array_equal(ago.encode(x, "f16").view(np.uint16), want16)
    want_bf = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(ago.encode(x, "bf16").view(np.uint16), want_bf)
    # NaN rules: bf16 keeps the top bits and sets 0x40 (features/store.rs:1094-1104)
    nan = np.array([np.nan], dtype=np.float32)
    assert ago.encode(nan, "bf16").view(np.uint16)[0] == (nan.view(np.uint32)[0] >> 16) | 0x40
    assert ago.encode(nan, "f16").view(np.uint16)[0] & 0x7E00 == 0x7E00
    assert np.array_equal(ago.encode(x, "f32").view(np.float32), x)


def test_half_round_trips_keep_reference_tolerances():
    # python/tests/test_dtypes_and_gather.py:16-63: bf16 keeps 1e+-30, f16 within tolerance
    x = np.array([1e30, -1e-30, 3.14159, 0.001], dtype=np.float32)
    back = ago.decode(ago.encode(x, "bf16"), "bf16")
    assert np.allclose(back, x, rtol=1e-2) and np.all(np.isfinite(back)) and back[1] != 0
    y = np.linspace(-4, 4, 1001, dtype=np.float32)
    assert np.allclose(ago.decode(ago.encode(y, "f16"), "f16"), y, atol=2e-3)


def test_gather_orders_rows_by_ids_and_checks_bounds():
    # features/store.rs:777-838, 1194-1226
    feats = np.arange(40, dtype=np.float32).reshape(10, 4)
    for dtype in ("f32", "f16", "bf16"):
        payload = ago.encode(feats, dtype)
        got = ago.gather(payload, 10, 4, dtype, [9, 0, 0, 3])
        assert np.array_equal(got, feats[[9, 0, 0, 3]])  # small integers are exact in every dtype
    with pytest.raises(ValueError, match="out of bounds"):
        ago.gather(ago.encode(feats, "f32"), 10, 4, "f32", [1, 10])


def test_crc32_is_ieee():
    data = np.random.default_rng(1).integers(0, 256, 10_000, dtype=np.uint8).tobytes()
    assert ago.crc32(data) == zlib.crc32(data)
    assert ago.crc32(data[5000:], ago.crc32(data[:5000])) == zlib.crc32(data)


# --------------------------------------------------------------- sampler --
def _test_graph():
    # loader/sampler.rs:1781-1799: 0->1,2,3  1->2,3  2->3,4  3->4  4->()
    src = np.array([0, 0, 0, 1, 1, 2, 2, 3], dtype=np.uint32)
    dst = np.array([1, 2, 3, 2, 3, 3, 4, 4], dtype=np.uint32)
    return csr_from_edges(5, src, dst)


def test_dedup_first_sighting_indices_dense_equals_map():
    # internal/genstamp.rs:208-236 (GenSlots / GenDedup cases) through seed registration
    off, dst, _ = _test_graph()
    for dense_max in (0, 1):  # 0: the reference bound (dense table); 1: forces the map
        s = ago.Sampler(off, dst, [0], seed=1, dense_dedup_max_nodes=dense_max)
        sg = s.sample([3, 4, 3])
        assert sg["nodes"].tolist() == [3, 4] and sg["seed_locals"].tolist() == [0, 1, 0]
        sg = s.sample([3])  # a new pass forgets everything
        assert sg["nodes"].tolist() == [3] and sg["seed_locals"].tolist() == [0]
    n, off, dst, _ = rmat_csr(10, 12, seed=3)
    seeds = np.random.default_rng(0).integers(0, n, 64).astype(np.uint32)
    a = ago.Sampler(off, dst, [7, 5], seed=9).sample(seeds)
    b = ago.Sampler(off, dst, [7, 5], seed=9, dense_dedup_max_nodes=1).sample(seeds)
    for k in ("nodes", "edge_dst", "edge_ids", "src_local", "dst_local"):
        assert np.array_equal(a[k], b[k])


def test_take_all_when_fanout_covers_the_row():
    # sampler.rs:1855-1881: node 0 has two neighbors, fanout 5 -> exactly {1, 2}, no RNG draws
    off, dst, _ = csr_from_edges(3, np.array([0, 0], dtype=np.uint32), np.array([1, 2], dtype=np.uint32))
    sg = ago.Sampler(off, dst, [5], seed=42).sample([0])
    assert sg["edge_dst"].tolist() == [1, 2] and sg["edge_ids"].tolist() == [0, 1] and sg["draws"] == 0
    # sampler.rs:3342-3357: seeds [0, 0, 1] at fanout 10 -> 5 distinct edges, the duplicate expands once
    off, dst, _ = _test_graph()
    sg = ago.Sampler(off, dst, [10], seed=1).sample([0, 0, 1])
    assert len(sg["edge_ids"]) == 5 and len(set(sg["edge_ids"].tolist())) == 5
    assert sg["seed_locals"].tolist() == [0, 0, 1]          # sampler.rs:3330-3338
    assert sg["num_sampled_nodes"].tolist()[0] == 2


def test_simple_graph_two_hops_exact():
    # the reference fixture test_data/simple_graph.txt, fanout >= degree everywhere: fully determined
    off = np.array([0, 2, 4, 5, 6, 6], dtype=np.uint64)
    dst = np.array([1, 2, 2, 3, 3, 4], dtype=np.uint32)
    sg = ago.Sampler(off, dst, [2, 2], seed=42).sample([0, 0, 1])
    assert sg["nodes"].tolist() == [0, 1, 2, 3, 4]
    assert sg["edge_src"].tolist() == [0, 0, 1, 1, 2, 3] and sg["edge_dst"].tolist() == [1, 2, 2, 3, 3, 4]
    assert sg["src_local"].tolist() == [0, 0, 1, 1, 2, 3] and sg["dst_local"].tolist() == [1, 2, 2, 3, 3, 4]
    assert sg["num_sampled_nodes"].tolist() == [2, 2, 1] and sg["num_sampled_edges"].tolist() == [4, 2]


@pytest.mark.parametrize("replace", [False, True])
def test_structural_invariants(replace):
    n, off, dst, _ = rmat_csr(12, 16, seed=1)
    s = ago.Sampler(off, dst, [15, 10], seed=42, replace=replace)
    seeds = np.random.default_rng(5).integers(0, n, 128).astype(np.uint32)
    sg = s.sample(seeds)
    # sampler.rs:2299-2369: local indices name the endpoints; seeds come first
    assert np.array_equal(sg["nodes"][sg["src_local"]], sg["edge_src"])
    assert np.array_equal(sg["nodes"][sg["dst_local"]], sg["edge_dst"])
    assert np.array_equal(sg["nodes"][sg["seed_locals"]], seeds)
    assert len(np.unique(sg["nodes"])) == len(sg["nodes"])
    # python/tests/test_sampler_semantics.py:25-42: edge_ids name the stored edge src -> dst
    assert np.array_equal(dst[sg["edge_ids"]], sg["edge_dst"])
    row = np.searchsorted(off, sg["edge_ids"], side="right") - 1
    assert np.array_equal(row.astype(np.uint32), sg["edge_src"])
    # sampler.rs:3397-3421: per-hop counts sum to the totals
    assert sg["num_sampled_nodes"].sum() == len(sg["nodes"]) and sg["num_sampled_edges"].sum() == len(sg["edge_ids"])
    if not replace:
        # sampler.rs:3423-3444: unique edge ids; every expanded node emits min(deg, k) edges, once
        assert len(np.unique(sg["edge_ids"])) == len(sg["edge_ids"])
        deg = np.diff(off.astype(np.int64))
        e0 = int(sg["num_sampled_edges"][0])
        srcs, counts = np.unique(sg["edge_src"][:e0], return_counts=True)
        assert np.array_equal(counts, np.minimum(deg[srcs], 15))


def test_determinism_and_stream_continuation():
    # sampler.rs:3116-3164; prefetch.rs:2297-2315
    n, off, dst, _ = rmat_csr(11, 16, seed=2)
    seeds = np.arange(50, dtype=np.uint32)
    a, b = ago.Sampler(off, dst, [5, 5], seed=7), ago.Sampler(off, dst, [5, 5], seed=7)
    first = a.sample(seeds)
    assert np.array_equal(first["edge_ids"], b.sample(seeds)["edge_ids"])
    second = a.sample(seeds)  # the stream continues: a second call differs
    assert not np.array_equal(first["edge_ids"], second["edge_ids"])
    assert np.array_equal(second["edge_ids"], b.sample(seeds)["edge_ids"])
    a.reseed(ago.batch_seed(7, 3)); b.reseed(ago.batch_seed(7, 3))
    assert np.array_equal(a.sample(seeds)["edge_ids"], b.sample(seeds)["edge_ids"])
    a.reseed(ago.batch_seed(7, 4))
    assert not np.array_equal(a.sample(seeds)["edge_ids"], b.sample(seeds)["edge_ids"])  # equal batches differ


def test_corrupt_destination_is_skipped():
    # sampler.rs:2149-2183
    off = np.array([0, 3, 3], dtype=np.uint64)
    dst = np.array([1, 77, 1], dtype=np.uint32)
    sg = ago.Sampler(off, dst, [5], seed=1).sample([0])
    assert sg["edge_dst"].tolist() == [1, 1] and sg["nodes"].tolist() == [0, 1]


def test_seed_out_of_range_names_the_position():
    off, dst, _ = _test_graph()
    with pytest.raises(IndexError, match=r"seed node 5 \(position 1\) is out of range for 5 nodes"):
        ago.Sampler(off, dst, [1], seed=1).sample([0, 5])


def test_uniform_coverage_of_a_hub_row():
    # sampler.rs:2242-2265: both halves of a 100-neighbor row within +-10 % over 4000 draws
    off = np.array([0, 100] + [100] * 100, dtype=np.uint64)
    dst = np.arange(1, 101, dtype=np.uint32)
    low = 0
    s = ago.Sampler(off, dst, [1], seed=3)
    for _ in range(4000):
        low += int(s.sample([0])["edge_dst"][0] <= 50)
    assert 1800 <= low <= 2200


def test_weighted_picks_distinct_neighbors_and_prefers_heavy_edges():
    # sampler.rs:2537-2618
    off = np.array([0, 10] + [10] * 10, dtype=np.uint64)
    dst = np.arange(1, 11, dtype=np.uint32)
    w = np.ones(10, dtype=np.float32); w[4] = 100.0
    s = ago.Sampler(off, dst, [3], weights=w, weighted=True, seed=5)
    wins = 0
    for _ in range(1000):
        sg = s.sample([0])
        assert len(set(sg["edge_dst"].tolist())) == 3 and sg["draws"] == 10
        wins += int(5 in sg["edge_dst"])
    assert wins > 900  # the reference asks for > 50 %
    # all weights unusable: keys are all +inf, ties break by row position
    s = ago.Sampler(off, dst, [3], weights=np.zeros(10, dtype=np.float32), weighted=True, seed=5)
    assert s.sample([0])["edge_ids"].tolist() == [0, 1, 2]


# ---------------------------------------------------------------- hetero --
def _reddit():
    # loader/hetero_sampler.rs:439-490.  types: user 100, post 100, comment 100, subreddit 20
    def rel(pairs, n_src):
        pairs = sorted(pairs)
        s = np.array([p[0] for p in pairs], dtype=np.uint32)
        d = np.array([p[1] for p in pairs], dtype=np.uint32)
        off, dd, _ = csr_from_edges(n_src, s, d)
        return off, dd
    voted = rel([(post, user) for user in range(50) for post in range(4)], 100)
    written = rel([(c, user) for user in range(30) for c in range(3)], 100)
    contains = rel([(post % 20, post) for post in range(100)], 100)
    USER, POST, COMMENT, SUB = 0, 1, 2, 3
    return [100, 100, 100, 20], [(POST, USER, *voted), (COMMENT, USER, *written), (SUB, POST, *contains)]


def test_hetero_fanout_per_edge_type_and_duplicates():
    num_nodes, rels = _reddit()
    # hetero_sampler.rs:740-758: fanouts (2, 1, 0): user 0 voted on 4 posts and wrote 3 comments
    sg = ago.HeteroSampler(num_nodes, rels, [[2], [1], [0]], seed=42).sample(0, [0])
    assert [len(e) for e in sg["edge_src_local"]] == [2, 1, 0]
    # hetero_sampler.rs:898-909: a duplicate seed expands once (4 edges), both entries share slot 0
    sg = ago.HeteroSampler(num_nodes, rels, [[10], [10], [10]], seed=42).sample(0, [0, 0])
    assert sg["seed_indices"].tolist() == [0, 0] and len(sg["edge_src_local"][0]) == 4


def test_hetero_edges_point_at_the_expanded_node_and_use_local_indices():
    num_nodes, rels = _reddit()
    # hetero_sampler.rs:519-545 and 547-570
    sg = ago.HeteroSampler(num_nodes, rels, [[5, 5]] * 3, seed=42).sample(0, [0, 1, 2])
    users, posts = sg["nodes"][0], sg["nodes"][1]
    assert users[:3].tolist() == [0, 1, 2] and len(posts) > 0 and len(sg["nodes"][3]) > 0
    off, dst = rels[0][2], rels[0][3]
    for s, d in zip(sg["edge_src_local"][0], sg["edge_dst_local"][0]):
        post, user = int(posts[s]), int(users[d])
        assert user in dst[int(off[post]):int(off[post + 1])]
    for et, (st, dt, _, _) in enumerate(rels):
        assert np.all(sg["edge_src_local"][et] < len(sg["nodes"][st]))
        assert np.all(sg["edge_dst_local"][et] < len(sg["nodes"][dt]))


def test_hetero_seed_bound_is_the_seed_types():
    num_nodes, rels = _reddit()
    s = ago.HeteroSampler(num_nodes, rels, [[2]] * 3, seed=42)
    s.sample(0, [0, 99])
    with pytest.raises(IndexError, match="out of range for 20 nodes"):
        s.sample(3, [0, 99])  # hetero_sampler.rs:911-929


def test_in_adjacency_is_the_stable_transpose():
    # graph/hetero.rs:70-97; hetero_sampler.rs:931-956
    n, off, dst, _ = rmat_csr(9, 8, seed=4)
    t_off, t_src = ago.transpose(off, dst, n, n)
    fwd = sorted((int(s), int(d)) for s in range(n) for d in dst[int(off[s]):int(off[s + 1])])
    back = sorted((int(s), int(d)) for d in range(n) for s in t_src[int(t_off[d]):int(t_off[d + 1])])
    assert fwd == back
    for d in range(n):  # sources in stored edge order: ascending source row
        row = t_src[int(t_off[d]):int(t_off[d + 1])]
        assert np.all(np.diff(row.astype(np.int64)) >= 0)
    # rows past num_src and destinations past num_dst are dropped
    t_off2, t_src2 = ago.transpose(off, dst, n // 2, n // 2)
    keep = [(s, d) for (s, d) in fwd if s < n // 2 and d < n // 2]
    assert int(t_off2[-1]) == len(keep) == len(t_src2)


# ------------------------------------------------------------ generators --
def test_cpu_generators_are_deterministic_and_shaped():
    off, dst = ago.synth_rmat_csr(1 << 12, 1 << 12, 1 << 16, 11, threads=4)
    off2, dst2 = ago.synth_rmat_csr(1 << 12, 1 << 12, 1 << 16, 11, threads=1)
    assert np.array_equal(off, off2) and np.array_equal(dst, dst2)  # thread count does not matter
    assert int(off[-1]) == 1 << 16 and dst.max() < (1 << 12)
    deg = np.diff(off.astype(np.int64))
    assert deg.max() > 20 * deg.mean()
    x = ago.decode(ago.synth_features(2000, 64, "f32", 9), "f32")
    assert abs(x.mean()) < 0.02 and abs(x.std() - 1.0) < 0.02
    assert np.array_equal(ago.synth_features(2000, 64, "bf16", 9, (500, 700)),
                          ago.synth_features(2000, 64, "bf16", 9).reshape(2000, 64)[500:700].reshape(-1))


def test_hetero_file_layout_follows_the_reference(tmp_path):
    """AETHHETG v1 field offsets and sizes as documented at
    crates/aethergraph-core/src/internal/mmap_hetero.rs:1-45 (64-byte header, 72-byte
    node entries, 216-byte edge entries, u32 sections padded to 8 bytes)."""
    from oracle import ago

    nt = [("user", 3), ("post", 2)]
    rels = [("user", "votes", "post", np.array([0, 2, 2, 3], np.uint64), np.array([0, 1, 1], np.uint32), None),
            ("post", "by", "user", np.array([0, 1, 2], np.uint64), np.array([2, 0], np.uint32), np.array([1.0, 2.0], np.float32))]
    p = tmp_path / "h.hetg"
    ago.write_hetero_file(p, nt, rels)
    raw = p.read_bytes()
    assert raw[:8] == b"AETHHETG" and raw[20:64] == bytes(44)
    assert np.frombuffer(raw[8:20], np.uint32).tolist() == [1, 2, 2]
    assert raw[64:68] == b"user" and raw[68:128] == bytes(60) and np.frombuffer(raw[128:136], np.uint64)[0] == 3
    e0 = 64 + 2 * 72
    assert raw[e0:e0 + 4] == b"user" and raw[e0 + 64:e0 + 69] == b"votes" and raw[e0 + 128:e0 + 132] == b"post"
    assert np.frombuffer(raw[e0 + 192:e0 + 208], np.uint64).tolist() == [3, 3]
    assert np.frombuffer(raw[e0 + 208:e0 + 216], np.uint32).tolist() == [0, 0]
    body = e0 + 2 * 216
    # relation 0: 4 offsets (32 B), 3 edges (12 B + 4 B pad); relation 1: 3 offsets, 2 edges (8 B), 2 weights (8 B)
    assert len(raw) == body + 32 + 16 + 24 + 8 + 8
    assert np.frombuffer(raw[body + 32:body + 44], np.uint32).tolist() == [0, 1, 1] and raw[body + 44:body + 48] == bytes(4)
    nt2, rels2 = ago.read_hetero_file(p)
    assert nt2 == nt and rels2[1][5].tolist() == [1.0, 2.0] and rels2[0][4].tolist() == [0, 1, 1]


def test_block_scaled_int8_codec_follows_the_reference_tests():
    """crates/aethergraph-core/src/internal/feature_codec.rs tests (:182-262): values come
    back within half a quantisation step of their block; the scale is per block, not per
    row; an all-zero block round-trips exactly with scale 0; a partial trailing block is
    encoded; NaN / infinite values and dim 0 are refused; 1.125 bytes per feature."""
    from oracle import ago

    ramp = lambda rows, dim: (np.arange(rows * dim, dtype=np.float32) * np.float32(0.25) - np.float32(3.0)).reshape(rows, dim)
    src = ramp(4, 96)
    codes, scales = ago.encode_i8(src)
    out = ago.gather_i8(codes, scales, np.arange(4))
    for b in range(3):
        blk = slice(32 * b, 32 * b + 32)
        step = np.abs(src[:, blk]).max(axis=1, keepdims=True) / 127.0
        assert np.all(np.abs(src[:, blk] - out[:, blk]) <= step * 0.5 + 1e-6)
    row = np.zeros((1, 64), dtype=np.float32)
    row[0, 0], row[0, 32], row[0, 33] = 1000.0, 0.5, -0.25
    codes, scales = ago.encode_i8(row)
    out = ago.gather_i8(codes, scales, [0])
    assert scales.shape == (1, 2) and abs(out[0, 32] - 0.5) < 0.01 and abs(out[0, 33] + 0.25) < 0.01
    codes, scales = ago.encode_i8(np.zeros((2, 32), dtype=np.float32))
    assert np.all(scales == 0) and np.all(ago.gather_i8(codes, scales, [0, 1]) == 0)
    codes, scales = ago.encode_i8(ramp(2, 40))
    assert scales.shape == (2, 2) and codes.shape == (2, 40)
    for bad in ([[1.0, np.nan]], [[np.inf, 1.0]]):
        with pytest.raises(ValueError, match="finite"):
            ago.encode_i8(np.array(bad, dtype=np.float32))
    with pytest.raises(ValueError, match="non-zero"):
        ago.encode_i8(np.zeros((3, 0), dtype=np.float32))
    codes, scales = ago.encode_i8(ramp(8, 128))
    assert abs((codes.size + scales.size * 4) / (codes.size * 4) - 1.125 / 4.0) < 1e-9
    # codes are symmetric, clamped to +-127, the peak of a block is +-127
    assert codes.min() >= -127 and np.all(np.abs(codes.reshape(8, 4, 32)).max(axis=2) == 127)


# ---- AETH version 2: the succinct codecs (crates/aethergraph-core/src/internal/succinct.rs) ----
def test_elias_fano_cases_of_the_reference_round_trip():
    # succinct.rs:607-640 (round trips, large universe), :704-722 (serialisation cases)
    from oracle import ago

    cases = [[], [0], [5], [0, 0, 0, 0], [1, 2, 3, 4, 5], [0, 10, 20, 30, 1000], [i * 7 for i in range(1000)],
             [0, 1, 1, 2, 3, 5, 8, 13, 21, 34, 55], [0, 1_000, 1_000_000, 4_000_000_000], [0, 0, 7, 7, 1_000_000],
             [i * 13 for i in range(2048)]]
    for c in cases:
        n, universe, low_bits, low, high = ago.ef_encode(np.array(c, dtype=np.uint64))
        assert n == len(c) and universe == (c[-1] if c else 0)
        assert int(sum(bin(int(w)).count("1") for w in high)) == len(c)           # one set bit per element
        assert low.size == (len(c) * low_bits + 63) // 64
        assert ago.ef_decode(n, universe, low_bits, low, high).tolist() == c
    # 4096 ids in a 65536 universe stay well under 16 bits per element (succinct.rs:642-650)
    n, _, _, low, high = ago.ef_encode(np.arange(4096, dtype=np.uint64) * 16)
    assert (low.size + high.size) * 64 / n < 16.0


def test_elias_fano_bit_layout_matches_the_reference_hand_built_records():
    # succinct.rs:772-781: two elements in high bucket 0 with low parts 3 then 1 -> low = 3 | 1 << 2, high = 0b11
    from oracle import ago

    assert ago.ef_decode(2, 3, 2, np.array([3 | (1 << 2)], np.uint64), np.array([0b11], np.uint64)).tolist() == [3, 1]
    # the encoder's own record for [1, 5, 9, 200] (succinct.rs:739-741) decodes to itself and follows
    # low_bits = floor(log2(universe / len)) (succinct.rs:60-66)
    n, universe, low_bits, low, high = ago.ef_encode(np.array([1, 5, 9, 200], np.uint64))
    assert (n, universe, low_bits) == (4, 200, 5)
    assert int(low[0]) == 1 | (5 << 5) | (9 << 10) | ((200 & 31) << 15)
    assert [i for i in range(64) if int(high[0]) >> i & 1] == [0, 1, 2, (200 >> 5) + 3]
    # succinct.rs:785-789: one element with bit 2 set, low_bits 0 -> value 2 (the reader rejects it for universe 5)
    assert ago.ef_decode(1, 5, 0, np.zeros(0, np.uint64), np.array([1 << 2], np.uint64)).tolist() == [2]


def test_streamvbyte_cases_of_the_reference_round_trip():
    # succinct.rs:659-673, :688-702 (non-monotone, wrapping), :797-806 (length boundaries)
    from oracle import ago

    cases = [[], [42], [0, 1, 2, 3, 4], [0, 255, 256, 65535, 65536, 16_777_215, 16_777_216], [i * 3 for i in range(1000)],
             [100] * 4, [0, 2**32 - 1], [5, 3], [10, 0, 2**32 - 1, 1, 2, 1], [2**32 - 1, 0, 2**32 - 1],
             [(i * 2_654_435_761) % 4_294_967_291 for i in range(500)]]
    for c in cases:
        n, first, control, data = ago.svb_encode(np.array(c, dtype=np.uint32))
        assert n == len(c) and control.size == (max(len(c) - 1, 0) + 3) // 4
        assert ago.svb_decode(n, first, control, data).tolist() == c
    # deltas 0, 255 | 256, 65535 | 65536, 16777215 | 16777216, 2^32-1 take 1, 1, 2, 2, 3, 3, 4, 4 bytes
    seq = np.cumsum([0, 0, 255, 256, 65_535, 65_536, 16_777_215, 16_777_216, 2**32 - 1], dtype=np.uint64).astype(np.uint32)
    _, _, control, data = ago.svb_encode(seq)
    assert control.tolist() == [0b01_01_00_00, 0b11_11_10_10] and data.size == 20
    # consecutive ids: about one byte per value (succinct.rs:675-686)
    _, _, control, data = ago.svb_encode(np.arange(10_000, dtype=np.uint32))
    assert control.size + data.size < 20_000


def test_compressed_graph_file_layout_and_round_trip():
    # compressed_graph.rs:39-88 (writer), :99-175 (reader), tests :205-235
    import struct

    from oracle import ago

    n, off, dst, _ = rmat_csr(10, 8, seed=2)
    order = np.concatenate([np.sort(dst[off[v]:off[v + 1]]) for v in range(n)]).astype(np.uint32)  # sorted rows compress
    w = np.random.default_rng(1).random(order.size).astype(np.float32)
    raw = ago.compressed_graph_bytes(off, order, w)
    magic, version, nn, ee, has_w, crc = struct.unpack_from("<IIQQII", raw, 0)
    assert (magic, version, nn, ee, has_w) == (0x41455448, 2, n, order.size, 1) and crc == ago.crc32(raw[32:])
    back = ago.read_compressed_graph(raw)
    assert back[0] == n and np.array_equal(back[1], off) and np.array_equal(back[2], order) and np.array_equal(back[3], w)
    flat = (n + 1) * 8 + order.size * 4
    assert len(ago.compressed_graph_bytes(off, order)) < flat          # "compresses below flat"


def test_compressed_golden_file_of_the_reference_fixture_graph():
    """tests/golden/simple_graph_aeth_v2.bin: header fields, section layout byte by byte, and the
    decoded CSR of the reference's fixture graph (test_data/simple_graph.txt)."""
    import struct

    from oracle import ago

    raw = open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "simple_graph_aeth_v2.bin"), "rb").read()
    magic, version, n, e, has_w, crc = struct.unpack_from("<IIQQII", raw, 0)
    assert (magic, version, n, e, has_w) == (0x41455448, 2, 5, 6, 0) and crc == zlib.crc32(raw[32:])
    # offsets [0,2,4,5,6,6]: len 6, universe 6, low_bits floor(log2(6/6)) = 0, no low words, one high word
    # with a set bit at value + index: 0, 3, 6, 8, 10, 11
    assert struct.unpack_from("<QQIQ", raw, 32) == (6, 6, 0, 0)
    assert struct.unpack_from("<QQ", raw, 32 + 28) == (1, sum(1 << b for b in (0, 3, 6, 8, 10, 11)))
    # edges [1,2,2,3,3,4]: first 1, deltas 1,0,1,0,1 of one byte each -> two control bytes of zeros
    at = 32 + 28 + 16
    assert struct.unpack_from("<QIQ", raw, at) == (6, 1, 2)
    assert raw[at + 20:at + 22] == bytes(2) and struct.unpack_from("<Q", raw, at + 22) == (5,)
    assert raw[at + 30:] == bytes([1, 0, 1, 0, 1])
    back = ago.read_compressed_graph(raw)
    assert back[0] == 5 and back[1].tolist() == [0, 2, 4, 5, 6, 6] and back[2].tolist() == [1, 2, 2, 3, 3, 4]
    assert ago.compressed_graph_bytes(back[1], back[2]) == raw

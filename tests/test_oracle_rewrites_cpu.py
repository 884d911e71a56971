"""The CPU restatements of the bidirectional and induced subgraph rewrites, checked
with the fixtures and properties of the reference's own tests
(crates/aethergraph-core/src/loader/sampler.rs:1908-2060
`induced_returns_every_edge_between_sampled_nodes`, `bidirectional_mirrors_and_coalesces`;
python/tests/test_sampler_semantics.py:112-127)."""
import numpy as np

from helpers import csr_from_edges
from oracle import ago


def _ring():
    n = 200
    src = np.repeat(np.arange(n, dtype=np.int64), 6)
    dst = (src + np.tile(np.arange(1, 7, dtype=np.int64) * 7, n)) % n
    return n, csr_from_edges(n, src.astype(np.uint32), dst.astype(np.uint32))


def test_bidirectional_mirrors_and_coalesces():
    edges = [(s, (s * 11 + st * 7) % 120) for s in range(120) for st in range(1, 6)]
    edges += [((s * 11 + 7) % 120, s) for s in range(60)]  # mutual pairs
    edges = sorted(set(edges))
    src, dst = (np.array(c, dtype=np.uint32) for c in zip(*edges))
    off, d, _ = csr_from_edges(120, src, dst)
    fwd = ago.Sampler(off, d, [6, 6], seed=11).sample(np.arange(40, dtype=np.uint32))
    bidi = ago.mirror(fwd)
    n = len(fwd["edge_src"])
    assert n > 0
    for k in ("edge_src", "edge_dst", "edge_ids", "src_local", "dst_local"):
        assert np.array_equal(bidi[k][:n], fwd[k])
    fwd_pairs = set(zip(fwd["edge_src"].tolist(), fwd["edge_dst"].tolist()))
    expected = [(int(fwd["edge_dst"][i]), int(fwd["edge_src"][i]), int(fwd["edge_ids"][i])) for i in range(n)
                if (int(fwd["edge_dst"][i]), int(fwd["edge_src"][i])) not in fwd_pairs]
    assert len(expected) < n  # the fixture has mutual pairs to coalesce
    got = list(zip(bidi["edge_src"][n:].tolist(), bidi["edge_dst"][n:].tolist(), bidi["edge_ids"][n:].tolist()))
    assert got == expected
    pairs = set(zip(bidi["edge_src"].tolist(), bidi["edge_dst"].tolist()))
    assert len(pairs) == len(bidi["edge_src"]) and all((b, a) in pairs for a, b in pairs)
    nodes = bidi["nodes"]
    assert np.array_equal(nodes[bidi["src_local"]], bidi["edge_src"]) and np.array_equal(nodes[bidi["dst_local"]], bidi["edge_dst"])


def test_bidirectional_with_replacement_keeps_one_reverse_per_pair():
    n, (off, d, _) = _ring()
    fwd = ago.Sampler(off, d, [4, 3], replace=True, seed=6).sample(np.array([0, 1, 2], dtype=np.uint32))
    bidi = ago.mirror(fwd)
    m = len(fwd["edge_src"])
    rev = list(zip(bidi["src_local"][m:].tolist(), bidi["dst_local"][m:].tolist()))
    assert len(set(rev)) == len(rev)
    assert set(rev) == {(b, a) for a, b in zip(fwd["src_local"].tolist(), fwd["dst_local"].tolist())} - \
        set(zip(fwd["src_local"].tolist(), fwd["dst_local"].tolist()))


def test_induced_returns_every_edge_between_sampled_nodes():
    edges = [(s, (s * 7 + st * 13) % 200) for s in range(200) for st in range(1, 8)]
    src, dst = (np.array(c, dtype=np.uint32) for c in zip(*edges))
    off, d, _ = csr_from_edges(200, src, dst)
    directional = ago.Sampler(off, d, [4, 3, 2], seed=7).sample(np.arange(16, dtype=np.uint32))
    induced = ago.induce(off, d, directional)
    assert np.array_equal(induced["nodes"], directional["nodes"])
    member = set(induced["nodes"].tolist())
    row_of = np.repeat(np.arange(200), np.diff(off).astype(np.int64))
    expected = {e for e in range(len(d)) if int(row_of[e]) in member and int(d[e]) in member}
    got = induced["edge_ids"].tolist()
    assert len(set(got)) == len(got) and set(got) == expected
    assert set(directional["edge_ids"].tolist()) <= expected and len(expected) > len(directional["edge_ids"])
    nodes = induced["nodes"]
    assert np.array_equal(nodes[induced["src_local"]], induced["edge_src"])
    assert np.array_equal(nodes[induced["dst_local"]], induced["edge_dst"])
    for i, e in enumerate(got):
        assert (int(row_of[e]), int(d[e])) == (int(induced["edge_src"][i]), int(induced["edge_dst"][i]))
    # order: by the expanded node's local index, then by position in its row
    key = list(zip(induced["src_local"].tolist(), got))
    assert key == sorted(key)


def test_ring_fixture_properties():
    n, (off, d, _) = _ring()
    fwd = ago.Sampler(off, d, [4, 3], seed=6).sample(np.array([0, 1, 2], dtype=np.uint32))
    bidi = ago.mirror(fwd)
    pairs = set(zip(bidi["dst_local"].tolist(), bidi["src_local"].tolist()))
    assert len(pairs) == len(bidi["src_local"]) and all((v, u) in pairs for u, v in pairs)
    ind = ago.induce(off, d, fwd)
    members = set(ind["nodes"].tolist())
    expected = {(int(v), u) for u in members for v in d[int(off[u]):int(off[u + 1])].tolist() if int(v) in members}
    assert set(zip(ind["edge_dst"].tolist(), ind["edge_src"].tolist())) == expected

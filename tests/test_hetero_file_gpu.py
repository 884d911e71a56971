"""AETHHETG v1 files on the GPU path: HeteroCsrGraph.load / .save against the
oracle-side writer and reader of the same layout
(crates/aethergraph-core/src/internal/mmap_hetero.rs:1-45), and the loader's
rejection of malformed files, one case per header field and section
(mmap_hetero.rs:161-330; its tests reject the same corruptions)."""
import numpy as np
import pytest

from helpers import csr_from_edges

pytestmark = pytest.mark.gpu


def _fixture():
    """Three node types, three relations (one empty, one with an odd edge count so the
    8-byte padding after a u32 section matters, one with weights)."""
    rng = np.random.default_rng(4)
    nt = [("user", 40), ("post", 25), ("tag", 7)]
    count = dict(nt)

    def rel(s, r, d, e, weighted=False):
        src = rng.integers(0, count[s], e).astype(np.uint32)
        dst = rng.integers(0, count[d], e).astype(np.uint32)
        off, dd, _ = csr_from_edges(count[s], src, dst)
        w = rng.random(e).astype(np.float32) + 0.5 if weighted else None
        return (s, r, d, off, dd, w)

    return nt, [rel("user", "likes", "post", 151), rel("post", "has", "tag", 0), rel("tag", "by", "user", 33, True)]


def _write(tmp_path, nt, rels, name="g.hetg"):
    from oracle import ago

    p = tmp_path / name
    ago.write_hetero_file(p, nt, rels)
    return p


def test_load_a_file_written_by_the_oracle_side(tmp_path):
    import aethergraph_b200 as ag
    from oracle import ago

    nt, rels = _fixture()
    g = ag.HeteroCsrGraph.load(_write(tmp_path, nt, rels))
    assert g.node_types() == [n for n, _ in nt] and [g.num_nodes(n) for n, _ in nt] == [c for _, c in nt]
    assert g.edge_types() == [(s, r, d) for (s, r, d, *_) in rels]
    count = dict(nt)
    for (s, r, d, off, dst, _w) in rels:
        assert g.num_edges(s, r, d) == len(dst)
        in_off, in_src = g.in_adjacency(s, r, d)
        t_off, t_src = ago.transpose(off, dst, count[s], count[d])
        assert np.array_equal(in_off, t_off) and np.array_equal(in_src, t_src)
    # ... and sampling over the loaded graph is the oracle's sampling over the same relations
    ids = {n: i for i, (n, _) in enumerate(nt)}
    fan = [[3, 2], [2, 2], [4, 1]]
    o = ago.HeteroSampler([c for _, c in nt], [(ids[s], ids[d], off, dst) for (s, r, d, off, dst, _w) in rels], fan, seed=5)
    seeds = np.arange(0, 25, dtype=np.uint32)
    want = o.sample(ids["post"], seeds)
    cfg = ag.HeteroSamplingConfig({(s, r, d): f for (s, r, d, *_), f in zip(rels, fan)}, seed=5)
    got = ag.HeteroNeighborSampler(g, cfg).sample("post", seeds).raw_u32()
    for k in ("nodes", "edge_src_local", "edge_dst_local"):
        assert all(np.array_equal(a, b) for a, b in zip(got[k], want[k])), k


def test_save_then_read_back_on_both_sides(tmp_path):
    import aethergraph_b200 as ag
    from oracle import ago

    nt, rels = _fixture()
    g = ag.HeteroCsrGraph.load(_write(tmp_path, nt, rels))
    out = tmp_path / "saved.hetg"
    g.save(out)
    nt2, rels2 = ago.read_hetero_file(out)
    assert nt2 == nt
    for (s, r, d, off, dst, _w), (s2, r2, d2, off2, dst2, w2) in zip(rels, rels2):
        assert (s, r, d) == (s2, r2, d2) and w2 is None
        assert np.array_equal(off, off2)
        # rows hold the same destinations, written in ascending order
        for v in range(len(off) - 1):
            a, b = int(off[v]), int(off[v + 1])
            assert np.array_equal(np.sort(dst[a:b]), dst2[a:b])
    g2 = ag.HeteroCsrGraph.load(out)
    for (s, r, d, *_rest) in rels:
        a, b = g.in_adjacency(s, r, d), g2.in_adjacency(s, r, d)
        assert np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])
    out.write_bytes(b"stale")      # save replaces an existing file atomically
    g2.save(out)
    assert ag.HeteroCsrGraph.load(out).edge_types() == g.edge_types()


def _patched(tmp_path, nt, rels, edit, name="bad.hetg"):
    raw = bytearray(_write(tmp_path, nt, rels, "good.hetg").read_bytes())
    raw = edit(raw) or raw
    p = tmp_path / name
    p.write_bytes(bytes(raw))
    return p


@pytest.mark.parametrize("case,match", [
    ("tiny", "too small for header"),
    ("magic", "invalid magic"),
    ("version", "version 2 is not supported"),
    ("too_many_types", "exceed the format limit"),
    ("more_types_than_sampler", "this build samples"),
    ("tables_cut", "type tables need"),
    ("no_nul", "no NUL terminator"),
    ("unknown_dst", "unknown destination type"),
    ("src_rows", "source rows but node type"),
    ("edges_cut", "file truncated"),
    ("offsets_start", r"offsets\[0\] != 0"),
    ("offsets_end", "!= num_edges"),
    ("offsets_order", "not non-decreasing"),
    ("dst_range", "a destination is >="),
    ("huge_edges", "exceeds maximum|file truncated|overflows"),
])
def test_malformed_files_are_rejected(tmp_path, case, match):
    import aethergraph_b200 as ag

    nt, rels = _fixture()
    node_table, edge_table = 64, 64 + 72 * len(nt)
    body = edge_table + 216 * len(rels)            # first relation: offsets of 41 u64, then 151 u32 edges

    def u32(v):
        return np.uint32(v).tobytes()

    def u64(v):
        return np.uint64(v).tobytes()

    def edit(raw):
        if case == "tiny":
            return raw[:40]
        if case == "magic":
            raw[0:8] = b"AETHHETX"
        elif case == "version":
            raw[8:12] = u32(2)
        elif case == "too_many_types":
            raw[12:16] = u32(300)
        elif case == "more_types_than_sampler":
            raw[12:16] = u32(9)
        elif case == "tables_cut":
            return raw[:edge_table + 100]
        elif case == "no_nul":
            raw[node_table:node_table + 64] = b"x" * 64
        elif case == "unknown_dst":
            raw[edge_table + 128:edge_table + 192] = b"ghost" + b"\0" * 59
        elif case == "src_rows":
            raw[edge_table + 192:edge_table + 200] = u64(39)
        elif case == "edges_cut":
            return raw[:body + 41 * 8 + 100]
        elif case == "offsets_start":
            raw[body:body + 8] = u64(1)
        elif case == "offsets_end":
            raw[body + 40 * 8:body + 41 * 8] = u64(150)
        elif case == "offsets_order":
            raw[body + 8:body + 16] = u64(152)
        elif case == "dst_range":
            raw[body + 41 * 8:body + 41 * 8 + 4] = u32(25)
        elif case == "huge_edges":
            raw[edge_table + 200:edge_table + 208] = u64(1 << 62)
        return raw

    with pytest.raises(ag.GraphLoadError, match=match):
        ag.HeteroCsrGraph.load(_patched(tmp_path, nt, rels, edit))


def test_missing_file_and_long_names(tmp_path):
    import aethergraph_b200 as ag

    with pytest.raises(ag.GraphLoadError, match="failed to open"):
        ag.HeteroCsrGraph.load(tmp_path / "nope.hetg")
    g = ag.HeteroCsrGraph.from_edge_arrays({"a" * 70: 3}, [])
    with pytest.raises(ValueError, match="type name too long"):
        g.save(tmp_path / "x.hetg")

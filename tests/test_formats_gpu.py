"""GPU: on-disk formats (AETH v1 graphs, AETHFEAT features) through the C ABI, the
graph accessors, and the committed golden samples."""
import os
import struct

import numpy as np
import pytest

from helpers import assert_same_subgraph

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def ag():
    import aethergraph_b200 as ag

    return ag


@pytest.fixture(scope="module")
def ago():
    from oracle import ago

    return ago


def test_load_reference_fixture_and_round_trip(ag, ago, tmp_path):
    # crates/aethergraph-core/tests/golden_format.rs:22-87
    gold = os.path.join(GOLDEN, "simple_graph_aeth_v1.bin")
    g = ag.Graph.load(gold, validation="full")
    assert (g.num_nodes, g.num_edges, g.has_weights, g.has_timestamps) == (5, 6, False, False)
    assert [g.neighbors(v).tolist() for v in range(5)] == [[1, 2], [2, 3], [3], [4], []]
    assert g.degrees().tolist() == [2, 2, 1, 1, 0] and g.degree(1) == 2 and g.degree(99) == 0
    assert g.degrees_of([4, 0, 77]).tolist() == [0, 2, 0]  # out of range -> 0
    assert len(g) == 5 and g[0].tolist() == [1, 2] and g.neighbor_weights(0) is None
    out = tmp_path / "saved.bin"
    g.save(out)
    raw, ref = out.read_bytes(), open(gold, "rb").read()
    assert raw[:28] == ref[:28] and raw[32:] == ref[32:]        # header fields and body identical
    crc = struct.unpack("<I", raw[28:32])[0]
    assert crc == ago.crc32(raw[32:]) != 0                        # the writer adds the body checksum
    g2 = ag.Graph.load(out, validation="full")                    # and the loader verifies it
    assert g2.neighbors(1).tolist() == [2, 3]
    bad = bytearray(raw); bad[28] ^= 0xFF
    (tmp_path / "badcrc.bin").write_bytes(bad)
    with pytest.raises(ag.GraphLoadError, match="checksum mismatch"):
        ag.Graph.load(tmp_path / "badcrc.bin", validation="full")
    ag.Graph.load(tmp_path / "badcrc.bin", validation="offsets_only")  # only full validation hashes the body


def test_loader_rejects_malformed_graph_files(ag, tmp_path):
    ref = open(os.path.join(GOLDEN, "simple_graph_aeth_v1.bin"), "rb").read()

    def write(name, data):
        p = tmp_path / name
        p.write_bytes(bytes(data))
        return p

    b = bytearray(ref); b[4:8] = struct.pack("<I", 9999)              # golden_format.rs:89-115
    with pytest.raises(ag.GraphLoadError, match="unsupported version: expected 1, got 9999"):
        ag.Graph.load(write("v.bin", b))
    b = bytearray(ref); b[0] ^= 1
    with pytest.raises(ag.GraphLoadError, match="invalid magic"):
        ag.Graph.load(write("m.bin", b))
    with pytest.raises(ag.GraphLoadError, match="file too small"):
        ag.Graph.load(write("t.bin", ref[:-4]))
    with pytest.raises(ag.GraphLoadError, match="insufficient bytes for header"):
        ag.Graph.load(write("h.bin", ref[:20]))
    b = bytearray(ref); b[100:104] = struct.pack("<I", 5)             # destination == num_nodes
    with pytest.raises(ag.GraphLoadError, match="destination"):
        ag.Graph.load(write("d.bin", b))
    b = bytearray(ref); b[40:48] = struct.pack("<Q", 7)               # offsets not monotone
    with pytest.raises(ag.GraphLoadError, match="offsets"):
        ag.Graph.load(write("o.bin", b))
    with pytest.raises(ag.GraphLoadError, match="failed to open"):
        ag.Graph.load(tmp_path / "missing.bin")
    with pytest.raises(ValueError, match="Invalid validation"):
        ag.Graph.load(tmp_path / "v.bin", validation="paranoid")


def test_from_edges_keeps_input_order_and_weights(ag, tmp_path):
    # crates/aethergraph-core/src/graph/csr.rs:568-571, 1388-1426
    src = np.array([2, 0, 2, 1, 0, 2], dtype=np.uint32)
    dst = np.array([5, 4, 3, 2, 1, 0], dtype=np.uint32)
    w = np.arange(6, dtype=np.float32) + 0.5
    g = ag.Graph.from_edges(6, src, dst, w)
    assert g.neighbors(0).tolist() == [4, 1] and g.neighbors(2).tolist() == [5, 3, 0]
    assert g.neighbor_weights(2).tolist() == [0.5, 2.5, 5.5] and g.has_weights
    off, d, ww = g.to_host()
    assert off.tolist() == [0, 2, 3, 6, 6, 6, 6] and d.tolist() == [4, 1, 2, 5, 3, 0]
    g.save(tmp_path / "w.bin")
    g2 = ag.Graph.load(tmp_path / "w.bin")
    assert g2.has_weights and g2.neighbor_weights(0).tolist() == [1.5, 4.5]
    st = g.stats()
    assert st["num_edges"] == 6 and st["max_degree"] == 3 and st["has_weights"]
    with pytest.raises(ValueError, match="out of range"):
        ag.Graph.from_edges(3, [0, 5], [1, 2])
    with pytest.raises(ValueError, match="negative"):
        ag.Graph.from_edges(3, np.array([0, -1]), np.array([1, 2]))
    with pytest.raises(ag.GraphLoadError):
        ag.Graph.from_csr(np.array([0, 2, 1], dtype=np.uint64), np.array([0, 1], dtype=np.uint32))


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_feature_files(ag, ago, tmp_path, dtype):
    # crates/aethergraph-core/src/features/store.rs:1194-1226, 1523-1593
    rng = np.random.default_rng(4)
    feats = rng.standard_normal((300, 20)).astype(np.float32)
    path = tmp_path / f"f_{dtype}.bin"
    ag.save_features(path, feats, dtype=dtype)
    store = ag.FeatureStore.load(path)
    assert (store.num_nodes, store.feature_dim, store.dtype) == (300, 20, dtype)
    ids = rng.integers(0, 300, 50)
    want = ago.gather(ago.encode(feats, dtype), 300, 20, dtype, ids)
    assert np.array_equal(store.get_batch(ids).view(np.uint32), want.view(np.uint32))
    assert np.array_equal(store.get(7), want[0] if ids[0] == 7 else store.get_batch([7])[0])
    if dtype == "f32":
        assert np.array_equal(store.features(), feats)
    shard = ag.FeatureStore.load(path, row_range=(100, 180))
    assert np.array_equal(shard.get_batch([100, 179]), store.get_batch([100, 179]))
    with pytest.raises(ValueError, match="not held by this shard"):
        shard.get_batch([99])


def test_feature_loader_rejects_malformed_headers(ag, tmp_path):
    # crates/aethergraph-core/src/features/header.rs:260-289
    good = tmp_path / "g.bin"
    ag.save_features(good, np.ones((4, 4), dtype=np.float32))
    raw = good.read_bytes()

    def load(mut, match):
        b = bytearray(raw)
        mut(b)
        p = tmp_path / "bad.bin"
        p.write_bytes(bytes(b))
        with pytest.raises(ag.GraphLoadError, match=match):
            ag.FeatureStore.load(p)

    load(lambda b: b.__setitem__(0, 0), "bad magic")
    load(lambda b: b.__setitem__(slice(24, 32), struct.pack("<Q", 32)), "must be > 32")
    load(lambda b: b.__setitem__(slice(24, 32), struct.pack("<Q", 514)), "4-byte aligned")
    load(lambda b: b.__setitem__(slice(24, 32), struct.pack("<Q", 1 << 20)), "for file size")
    load(lambda b: b.__setitem__(32, 9), "unknown feature dtype tag: 9")
    load(lambda b: b.__setitem__(slice(8, 16), struct.pack("<Q", 1000)), "truncated")
    load(lambda b: b.__setitem__(slice(16, 24), struct.pack("<Q", 200_000)), "exceeds maximum")
    (tmp_path / "tiny.bin").write_bytes(raw[:16])
    with pytest.raises(ag.GraphLoadError, match="too small"):
        ag.FeatureStore.load(tmp_path / "tiny.bin")


def test_loader_with_feature_file(ag, ago, tmp_path):
    # python/tests/test_loader.py:87-113: x rows align with n_id
    from helpers import rmat_csr

    n, off, dst, _ = rmat_csr(10, 12, seed=6)
    feats = np.random.default_rng(1).standard_normal((n, 16)).astype(np.float32)
    ag.save_features(tmp_path / "feat.bin", feats, dtype="bf16")
    g = ag.Graph.from_csr(off, dst)
    cfg = ag.SamplingConfig(num_neighbors=[5, 5], seed=3)
    with ag.NeighborLoader.with_features(g, cfg, tmp_path / "feat.bin", 2, 2) as loader:
        loader.submit_epoch([np.arange(i, i + 20) for i in range(0, 100, 20)])
        for i in range(5):
            idx, sg, x = loader.next_batch()
            assert idx == i
            want = ago.gather(ago.encode(feats, "bf16"), n, 16, "bf16", sg.nodes)
            assert np.array_equal(x.cpu().numpy().view(np.uint32), want.view(np.uint32))
    with pytest.raises(ValueError, match="rows but the graph has"):
        ag.save_features(tmp_path / "short.bin", feats[:10])
        ag.NeighborLoader.with_features(g, cfg, tmp_path / "short.bin")


def test_graph_load_features_attaches_the_store(ag, ago, tmp_path):
    """`graph = Graph.load(p); graph.load_features(f)` then the epoch loader, the
    workflow the reference's README shows: batches carry x == features[n_id]."""
    from helpers import rmat_csr

    from aethergraph_b200.pytorch import NeighborLoader

    n, off, dst, _ = rmat_csr(10, 8, seed=4)
    feats = np.random.default_rng(2).standard_normal((n, 32)).astype(np.float32)
    ag.save_features(tmp_path / "feat.bin", feats, dtype="f16")
    ag.Graph.from_csr(off, dst).save(tmp_path / "g.bin")
    graph = ag.Graph.load(tmp_path / "g.bin")
    store = graph.load_features(tmp_path / "feat.bin")
    assert store is graph.features and store.feature_dim == 32
    payload = ago.encode(feats, "f16")
    seen = 0
    for batch in NeighborLoader(graph, num_neighbors=[4, 3], batch_size=64, shuffle=False, seed=1):
        want = ago.gather(payload, n, 32, "f16", batch.n_id.cpu().numpy().astype(np.uint32))
        assert np.array_equal(batch.x.cpu().numpy().view(np.uint32), want.view(np.uint32))
        seen += 1
    assert seen == n // 64
    ag.save_features(tmp_path / "short.bin", feats[:10])
    with pytest.raises(ValueError, match="rows but the graph has"):
        graph.load_features(tmp_path / "short.bin")


def test_gpu_reproduces_the_golden_samples(ag):
    g = np.load(os.path.join(GOLDEN, "golden_samples.npz"))
    off, dst, w, feats = g["offsets"], g["dst"], g["weights"], g["features"]
    for name, kw in (("uniform", {}), ("replace", {"replace": True}), ("weighted", {"weighted": True}), ("deep", {})):
        graph = ag.Graph.from_csr(off, dst, w if kw.get("weighted") else None)
        cfg = ag.SamplingConfig(num_neighbors=g[f"{name}.fanout"].tolist(), seed=int(g[f"{name}.seed"]), **kw)
        s = ag.NeighborSampler(graph, cfg)
        for call in range(2):
            sg = s.sample(g[f"{name}.seeds"])
            want = {k: g[f"{name}.{call}.{k}"] for k in ("nodes", "edge_src", "edge_dst", "edge_ids", "src_local",
                                                         "dst_local", "seed_locals", "num_sampled_nodes",
                                                         "num_sampled_edges")}
            want["draws"] = int(g[f"{name}.{call}.draws"])
            assert_same_subgraph(sg.raw_u32(), want, f"{name} call {call} ")
        for dtype in ("f32", "f16", "bf16"):
            store = ag.FeatureStore.from_array(feats, dtype)
            x = store.get_batch(sg.nodes[:64])
            assert np.array_equal(x.view(np.uint32), g[f"{name}.x.{dtype}"].view(np.uint32))


# ---- AETH version 2 (Elias-Fano offsets + StreamVByte edges), decoded on the GPU ----
def _csr_cases():
    from helpers import rmat_csr

    rng = np.random.default_rng(5)
    n, off, dst, _ = rmat_csr(12, 12, seed=8)
    sorted_rows = np.concatenate([np.sort(dst[off[v]:off[v + 1]]) for v in range(n)]).astype(np.uint32)
    yield "rmat sorted rows", n, off, sorted_rows, None
    yield "rmat unsorted rows, weighted", n, off, dst, rng.random(dst.size).astype(np.float32)  # backward steps: 4-byte deltas
    yield "no edges", 7, np.zeros(8, np.uint64), np.zeros(0, np.uint32), None
    yield "one edge", 2, np.array([0, 1, 1], np.uint64), np.array([1], np.uint32), np.array([0.5], np.float32)
    deg = rng.integers(0, 3, 3000)
    off2 = np.concatenate([[0], np.cumsum(deg)]).astype(np.uint64)
    yield "sparse degrees", 3000, off2, rng.integers(0, 3000, int(off2[-1])).astype(np.uint32), None
    # five deltas (not a multiple of four) of every byte length
    seq = np.array([0, 1, 300, 70_000, 17_000_000, 5], np.uint32)
    yield "delta lengths", 17_000_001, np.concatenate([[0], np.full(17_000_001, 6)]).astype(np.uint64), seq, None


def test_compressed_graph_files_decode_on_the_gpu_and_save_bit_for_bit(ag, ago, tmp_path):
    """Files written by the numpy restatement of the reference's codecs load into the same
    CSR, and what `save(compressed=True)` writes is the same file byte for byte
    (compressed_graph.rs:39-175; round trips of its tests :205-235)."""
    for name, n, off, dst, w in _csr_cases():
        raw = ago.compressed_graph_bytes(off, dst, w)
        p = tmp_path / "g2.bin"
        p.write_bytes(raw)
        g = ag.Graph.load(p)
        assert (g.num_nodes, g.num_edges, g.has_weights) == (n, dst.size, w is not None), name
        o2, d2, w2 = g.to_host()
        assert np.array_equal(o2, off) and np.array_equal(d2, dst), name
        if w is not None:
            assert np.array_equal(w2, w), name
        out = tmp_path / "saved2.bin"
        g.save(out, compressed=True)
        assert out.read_bytes() == raw, name
        flat = tmp_path / "flat.bin"
        g.save(flat)                                     # and back to version 1
        assert np.array_equal(ag.Graph.load(flat).to_host()[1], dst), name


def test_compressed_graph_samples_like_the_flat_one(ag, ago, tmp_path):
    # compressed_graph.rs:281-297
    from helpers import rmat_csr

    n, off, dst, _ = rmat_csr(11, 10, seed=3)
    p = tmp_path / "g2.bin"
    p.write_bytes(ago.compressed_graph_bytes(off, dst))
    g = ag.Graph.load(p)
    seeds = np.arange(64, dtype=np.uint32)
    got = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[5, 3], seed=7)).sample(seeds)
    want = ago.Sampler(off, dst, [5, 3], seed=7).sample(seeds)
    assert_same_subgraph(got.raw_u32(), want)


def test_loader_rejects_malformed_compressed_files(ag, ago, tmp_path):
    """One malformed file per check of the reader (compressed_graph.rs:105-160;
    succinct.rs:225-262 and its tests :735-795, :506-535)."""
    from helpers import rmat_csr

    n, off, dst, _ = rmat_csr(8, 8, seed=1)
    dst = np.concatenate([np.sort(dst[off[v]:off[v + 1]]) for v in range(n)]).astype(np.uint32)
    good = bytearray(ago.compressed_graph_bytes(off, dst, checksum=False))

    def load(data, match):
        p = tmp_path / "bad2.bin"
        p.write_bytes(bytes(data))
        with pytest.raises(ag.GraphLoadError, match=match):
            ag.Graph.load(p)

    ag.Graph.load(_write(tmp_path, "ok2.bin", good))                      # zero checksum: not verified
    with_crc = bytearray(ago.compressed_graph_bytes(off, dst))
    with_crc[-1] ^= 0x01
    load(with_crc, "checksum mismatch")
    load(good[:-1], "truncated|control tags")                             # data stream one byte short
    load(good + b"\0", "trailing bytes")
    ef_len, universe, low_bits, lw = struct.unpack_from("<QQIQ", good, 32)
    hw_at = 32 + 28 + lw * 8
    (hw,) = struct.unpack_from("<Q", good, hw_at)
    bad = bytearray(good); struct.pack_into("<Q", bad, 32, ef_len + 1)
    load(bad, "offsets section has")
    bad = bytearray(good); struct.pack_into("<I", bad, 32 + 16, 64)
    load(bad, "low_bits")
    bad = bytearray(good); bad[hw_at + 8 + hw * 8 - 8: hw_at + 8 + hw * 8] = b"\0" * 8    # a cleared high word
    load(bad, "set bits")
    bad = bytearray(good); struct.pack_into("<Q", bad, 32 + 8, universe + (1 << 40))      # universe the last element misses
    load(bad, "universe")
    svb_at = hw_at + 8 + hw * 8
    bad = bytearray(good); struct.pack_into("<Q", bad, svb_at, dst.size + 1)
    load(bad, "edges section has")
    (nc,) = struct.unpack_from("<Q", good, svb_at + 12)
    bad = bytearray(good); bad[svb_at + 20] |= 0x03                                        # first delta claims 4 bytes
    load(bad, "control tags call for")
    # offsets that decrease through the low bits (succinct.rs:772-781), as a whole file: 1 node, offsets [3, 1]
    payload = struct.pack("<QQIQ", 2, 3, 2, 1) + struct.pack("<Q", 3 | (1 << 2)) + struct.pack("<QQ", 1, 0b11)
    payload += struct.pack("<QIQ", 3, 0, 1) + bytes([0]) + struct.pack("<Q", 2) + bytes([0, 0])
    load(struct.pack("<IIQQII", 0x41455448, 2, 1, 3, 0, 0) + payload, "invalid CSR|universe")
    # a destination outside the graph is caught by the full validation every compressed load runs
    bad_dst = dst.copy(); bad_dst[3] = n + 5
    load(ago.compressed_graph_bytes(off, bad_dst), "destination")


def _write(tmp_path, name, data):
    p = tmp_path / name
    p.write_bytes(bytes(data))
    return p


def test_load_the_compressed_golden_of_the_reference_fixture(ag, tmp_path):
    """tests/golden/simple_graph_aeth_v2.bin decodes to the fixture graph and is written back
    byte for byte (crates/aethergraph-core/tests/golden_format.rs:22-87 for the graph itself)."""
    gold = os.path.join(GOLDEN, "simple_graph_aeth_v2.bin")
    g = ag.Graph.load(gold)
    assert (g.num_nodes, g.num_edges, g.has_weights) == (5, 6, False)
    assert [g.neighbors(v).tolist() for v in range(5)] == [[1, 2], [2, 3], [3], [4], []]
    out = tmp_path / "again.bin"
    g.save(out, compressed=True)
    assert out.read_bytes() == open(gold, "rb").read()
    flat = tmp_path / "flat.bin"
    g.save(flat)
    assert flat.read_bytes()[32:] == open(os.path.join(GOLDEN, "simple_graph_aeth_v1.bin"), "rb").read()[32:]

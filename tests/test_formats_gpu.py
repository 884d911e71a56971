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

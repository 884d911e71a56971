"""CPU tests of the host side: the C ABI library loads and exports every symbol the
header declares (no compute calls), the Python mirror validates like the reference,
the AETHFEAT writer produces the pinned layout, golden fixtures hold, the
data-parallel partition works across two gloo ranks."""
import os
import re
import struct

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def lib():
    from aethergraph_b200 import _lib, build

    build.build()
    return _lib


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "aethergpu.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ag_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(lib):
    import ctypes

    names = _declared_symbols()
    assert len(names) > 50
    so = ctypes.CDLL(lib.LIB_PATH)
    missing = [n for n in names if not hasattr(so, n)]
    assert not missing, f"declared in include/aethergpu.h but not exported: {missing}"
    unbound = [n for n in names if n not in lib.SIGNATURES]
    assert not unbound, f"no ctypes signature for: {unbound}"
    assert lib.lib().ag_abi_version() == 1


def test_batch_seed_through_the_abi(lib):
    from oracle import ago

    for base, idx in [(42, 0), (42, 7), (2**64 - 1, 99)]:
        assert lib.lib().ag_batch_seed(base, idx) == ago.batch_seed(base, idx)


def test_product_never_touches_the_oracle():
    pkg = os.path.join(ROOT, "aethergraph_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".cc")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"


def test_no_cpu_fallback():
    import torch

    import aethergraph_b200 as ag

    if torch.cuda.is_available():
        pytest.skip("needs a machine without a GPU")
    with pytest.raises(RuntimeError, match="no CPU path"):
        ag.Graph.from_edges(3, [0, 0], [1, 2])
    with pytest.raises(RuntimeError, match="no CPU path"):
        ag.FeatureStore.from_array(np.zeros((2, 2), dtype=np.float32))


def test_sampling_config_validation():
    import aethergraph_b200 as ag

    # crates/aethergraph-py/src/sampler.rs:133-176
    with pytest.raises(ValueError, match="non-empty"):
        ag.SamplingConfig(num_neighbors=[])
    with pytest.raises(ValueError, match="non-negative"):
        ag.SamplingConfig(num_neighbors=[5, -1])
    with pytest.raises(ValueError, match="max_degree must be > 0"):
        ag.SamplingConfig(num_neighbors=[5], max_degree=0)
    with pytest.raises(ValueError, match="Invalid subgraph_type 'x'"):
        ag.SamplingConfig(num_neighbors=[5], subgraph_type="x")
    with pytest.raises(ValueError, match="Invalid temporal_strategy 'soon'"):
        ag.SamplingConfig(num_neighbors=[5], temporal_strategy="soon")
    with pytest.raises(ValueError, match="rng_mode"):
        ag.SamplingConfig(num_neighbors=[5], rng_mode="mt19937")
    cfg = ag.SamplingConfig(num_neighbors=[25, 10])
    assert (cfg.replace, cfg.seed, cfg.weighted, cfg.track_edge_ids, cfg.subgraph_type) == (False, None, False, True,
                                                                                          "directional")
    assert cfg._unsupported() is None
    assert ag.SamplingConfig([3], disjoint=True)._unsupported() is None     # the plain sampler runs it seed by seed
    assert ag.SamplingConfig([3], cumulative=True)._unsupported() is None   # the plain sampler runs it hop by hop
    assert ag.SamplingConfig([3], temporal_strategy="last")._unsupported() == "temporal sampling"
    assert ag.SamplingConfig([3], subgraph_type="induced")._unsupported() is None  # rewrites run on the GPU
    assert ag.SamplingConfig([3], subgraph_type="bidirectional")._unsupported() is None
    c = cfg._to_c(7, 128)
    assert (c.num_hops, c.fanout[0], c.fanout[1], c.seed, c.max_seeds, c.rng_mode) == (2, 25, 10, 7, 128, 0)


def test_seed_coercion_follows_the_reference():
    import aethergraph_b200 as ag
    from aethergraph_b200.sampler import coerce_seeds

    # crates/aethergraph-py/src/error.rs:115-153
    assert coerce_seeds([1, 2, 3], 10).dtype == np.uint32
    a = np.array([4, 5], dtype=np.uint32)
    assert coerce_seeds(a, 10) is a
    with pytest.raises(ag.SamplingError, match=r"seed node -1 out of u32 range"):
        coerce_seeds(np.array([0, -1], dtype=np.int64), 10)
    with pytest.raises(ag.SamplingError, match=r"out of u32 range"):
        coerce_seeds(np.array([2**33], dtype=np.int64), 10)
    with pytest.raises(ag.SamplingError, match=r"seed node 10 \(position 2\) is out of range for 10 nodes"):
        coerce_seeds(np.array([0, 1, 10], dtype=np.int64), 10)
    assert len(coerce_seeds([], 10)) == 0


def test_feature_file_layout(lib, tmp_path):
    from oracle import ago

    import aethergraph_b200 as ag

    # features/store.rs:1290-1320 (header) and features/header.rs:165-244 (fields)
    feats = np.random.default_rng(3).standard_normal((10, 4)).astype(np.float32)
    for dtype, tag, esize in (("f32", 0, 4), ("f16", 1, 2), ("bf16", 2, 2)):
        path = tmp_path / f"feat_{dtype}.bin"
        ag.save_features(path, feats, dtype=dtype)
        raw = path.read_bytes()
        assert raw[:8] == b"AETHFEAT"
        n, dim, off = struct.unpack("<QQQ", raw[8:32])
        assert (n, dim, off) == (10, 4, 512) and raw[32] == tag
        assert raw[33:512] == bytes(512 - 33)
        assert len(raw) == 512 + 10 * 4 * esize
        assert raw[512:] == ago.encode(feats, dtype).tobytes()
    with pytest.raises(ValueError, match="Invalid dtype"):
        ag.save_features(tmp_path / "x.bin", feats, dtype="int8")
    with pytest.raises(ValueError, match="2-d"):
        ag.save_features(tmp_path / "x.bin", feats.reshape(-1))
    assert not [p for p in os.listdir(tmp_path) if ".tmp." in p]  # written atomically, no leftovers


def test_aeth_v1_golden_bytes():
    # crates/aethergraph-core/tests/golden_format.rs:22-87 on the reference's fixture graph
    raw = open(os.path.join(GOLDEN, "simple_graph_aeth_v1.bin"), "rb").read()
    magic, version, n, e, has_w, crc = struct.unpack("<IIQQII", raw[:32])
    assert (magic, version, n, e, has_w, crc) == (0x41455448, 1, 5, 6, 0, 0)
    assert np.frombuffer(raw[32:32 + 48], dtype="<u8").tolist() == [0, 2, 4, 5, 6, 6]
    assert np.frombuffer(raw[80:104], dtype="<u4").tolist() == [1, 2, 2, 3, 3, 4]
    assert len(raw) == 104


def test_oracle_reproduces_the_golden_samples():
    from oracle import ago

    g = np.load(os.path.join(GOLDEN, "golden_samples.npz"))
    off, dst, w, feats, n = g["offsets"], g["dst"], g["weights"], g["features"], int(g["n"])
    for name, kw in (("uniform", {}), ("replace", {"replace": True}), ("weighted", {"weighted": True}), ("deep", {})):
        s = ago.Sampler(off, dst, g[f"{name}.fanout"], weights=w if kw.get("weighted") else None,
                        seed=int(g[f"{name}.seed"]), **kw)
        for call in range(2):
            sg = s.sample(g[f"{name}.seeds"])
            for k in ("nodes", "edge_src", "edge_dst", "edge_ids", "src_local", "dst_local", "seed_locals",
                      "num_sampled_nodes", "num_sampled_edges"):
                assert np.array_equal(sg[k], g[f"{name}.{call}.{k}"]), (name, call, k)
            assert sg["draws"] == int(g[f"{name}.{call}.draws"])
        for dtype in ("f32", "f16", "bf16"):
            x = ago.gather(ago.encode(feats, dtype), n, 24, dtype, sg["nodes"][:64])
            assert np.array_equal(x.view(np.uint32), g[f"{name}.x.{dtype}"].view(np.uint32))


def test_partition_helpers():
    from aethergraph_b200 import dist

    assert dist.rank_batches(0, 1, 5) == [0, 1, 2, 3, 4]
    parts = [dist.rank_batches(r, 3, 10) for r in range(3)]
    assert sorted(sum(parts, [])) == list(range(10)) and parts[1] == [1, 4, 7]
    with pytest.raises(ValueError):
        dist.rank_batches(3, 3, 10)
    assert [dist.shard_range(r, 10, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 9), (9, 10)]
    assert [dist.owner_of_row(v, 10, 4) for v in (0, 2, 3, 8, 9)] == [0, 0, 1, 2, 3]


def _gloo_rank(rank, world, port, out):
    """Each rank samples its share of the batch stream with the oracle; the ranks agree
    on totals with an all-reduce, the way bench.py's ranks do."""
    import torch
    import torch.distributed as td

    from aethergraph_b200 import dist
    from helpers import rmat_csr
    from oracle import ago

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    td.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, off, dst, _ = rmat_csr(10, 12, seed=8)
        s = ago.Sampler(off, dst, [6, 4], seed=42)
        rng = np.random.default_rng(0)
        batches = [rng.integers(0, n, 32).astype(np.uint32) for _ in range(9)]
        edges, sums = 0, {}
        for b in dist.rank_batches(rank, world, len(batches)):
            s.reseed(ago.batch_seed(42, b))
            sg = s.sample(batches[b])
            edges += len(sg["edge_ids"])
            sums[b] = int(sg["edge_ids"].astype(np.uint64).sum())
        total = dist.sum_over_ranks(float(edges))
        slowest = dist.max_over_ranks(float(rank + 1))
        gathered = [None] * world
        td.all_gather_object(gathered, sums)
        if rank == 0:
            out.put((total, slowest, gathered))
    finally:
        td.destroy_process_group()


def test_two_gloo_ranks_partition_the_stream():
    import torch.multiprocessing as mp

    from helpers import rmat_csr
    from oracle import ago

    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    total, slowest, gathered = out.get(timeout=120)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    # single-process truth
    n, off, dst, _ = rmat_csr(10, 12, seed=8)
    s = ago.Sampler(off, dst, [6, 4], seed=42)
    rng = np.random.default_rng(0)
    batches = [rng.integers(0, n, 32).astype(np.uint32) for _ in range(9)]
    want = {}
    for b, seeds in enumerate(batches):
        s.reseed(ago.batch_seed(42, b))
        sg = s.sample(seeds)
        want[b] = (len(sg["edge_ids"]), int(sg["edge_ids"].astype(np.uint64).sum()))
    merged = {}
    for d in gathered:
        merged.update(d)
    assert sorted(merged) == list(range(9))           # every batch handled exactly once
    assert all(merged[b] == want[b][1] for b in want)  # same samples whatever the rank count
    assert total == sum(v[0] for v in want.values()) and slowest == 2.0

"""GPU parity: the gather / upcast kernel against the CPU oracle, bit for bit."""
import os

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


def _bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("dim", [1, 3, 8, 64, 100, 128, 256, 260])
def test_gather_matches_oracle(ag, ago, dtype, dim):
    rng = np.random.default_rng(dim)
    n = 1000
    feats = (rng.standard_normal((n, dim)) * 10.0 ** rng.integers(-6, 5, (n, 1))).astype(np.float32)
    payload = ago.encode(feats, dtype)
    store = ag.FeatureStore.from_payload(payload, n, dim, dtype)
    ids = rng.integers(0, n, size=777)
    ids[10] = ids[11]  # duplicates are re-read
    want = ago.gather(payload, n, dim, dtype, ids)
    got = store.get_batch(ids.astype(np.int64))
    assert got.shape == (777, dim)
    assert np.array_equal(_bits(got), _bits(want))
    # device-encoded store holds the same bits as the oracle's encoder
    store2 = ag.FeatureStore.from_array(feats, dtype)
    assert np.array_equal(_bits(store2.get_batch(ids.astype(np.int64))), _bits(want))


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_every_16bit_pattern(ag, ago, dtype):
    bits = np.arange(65536, dtype=np.uint16).reshape(256, 256)
    store = ag.FeatureStore.from_payload(bits, 256, 256, dtype)
    got = store.features()
    want = ago.decode(bits, dtype).reshape(256, 256)
    assert np.array_equal(_bits(got), _bits(want))


def test_encode_special_values(ag, ago):
    x = np.array([[0.0, -0.0, np.inf, -np.inf, np.nan, 65504.0, 65520.0, 65519.99, 1e-8, 6e-8, 5.96e-8,
                   2.98e-8, 2.9802322e-8, 2.99e-8, 1e38, -3e38]], dtype=np.float32)
    for dtype in ("f16", "bf16"):
        store = ag.FeatureStore.from_array(x, dtype)
        want = ago.decode(ago.encode(x, dtype), dtype).reshape(x.shape)
        assert np.array_equal(_bits(store.features()), _bits(want)), dtype


def test_out_of_range_id(ag):
    store = ag.FeatureStore.from_array(np.zeros((10, 4), dtype=np.float32))
    with pytest.raises(ValueError, match="node 10 out of bounds"):
        store.get_batch(np.array([1, 10], dtype=np.int64))
    with pytest.raises(ValueError):
        store.get_batch(np.array([-1], dtype=np.int64))
    assert store.get_batch(np.array([], dtype=np.int64)).shape == (0, 4)


def test_device_gather_and_sticky_error(ag):
    import torch

    feats = np.arange(40, dtype=np.float32).reshape(10, 4)
    store = ag.FeatureStore.from_array(feats, "f32")
    ids = torch.tensor([3, 3, 9, 0], device="cuda")
    out = store.gather(ids)
    assert np.array_equal(out.cpu().numpy(), feats[[3, 3, 9, 0]])
    store.check()
    out = store.gather(torch.tensor([1, 77], device="cuda"))
    assert np.array_equal(out.cpu().numpy()[1], np.zeros(4, dtype=np.float32))
    with pytest.raises(ValueError, match="out of bounds"):
        store.check()
    store.check()  # cleared


def test_sampler_gathers_x_for_nodes(ag, ago):
    from helpers import rmat_csr

    n, off, dst, _ = rmat_csr(12, 16, seed=1)
    rng = np.random.default_rng(0)
    feats = rng.standard_normal((n, 128)).astype(np.float32)
    for dtype in ("f32", "bf16", "f16"):
        store = ag.FeatureStore.from_array(feats, dtype)
        g = ag.Graph.from_csr(off, dst)
        s = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[15, 10], seed=42), features=store)
        sg = s.sample(rng.integers(0, n, 128))
        payload = ago.encode(feats, dtype)
        want = ago.gather(payload, n, 128, dtype, sg.nodes)
        assert np.array_equal(_bits(sg.x.cpu().numpy()), _bits(want)), dtype


_BULK_WORKER = r"""
import os, sys
import numpy as np
sys.path.insert(0, os.environ["AG_ROOT"]); sys.path.insert(0, os.path.join(os.environ["AG_ROOT"], "tests"))
import aethergraph_b200 as ag
from aethergraph_b200 import synth
from oracle import ago
from helpers import rmat_csr
n, off, dst, _ = rmat_csr(13, 10, seed=5)
g = ag.Graph.from_csr(off, dst)
ok = True
for dtype, dim in (("bf16", 256), ("f16", 64), ("f32", 24), ("bf16", 8)):
    feats = synth.features(n, dim, dtype, 7)
    payload = ago.synth_features(n, dim, dtype, 7)
    rng = np.random.default_rng(1)
    batches = [rng.integers(0, n, s).astype(np.uint32) for s in (300, 1, 0, 700, 31, 33, 64)] * 3
    s = ago.Sampler(off, dst, [10, 5], seed=3)
    with ag.NeighborLoader(g, ag.SamplingConfig(num_neighbors=[10, 5], seed=3), prefetch_depth=8, sampler_threads=2,
                           features=feats, group=8) as ld:
        for i, b in enumerate(batches):
            ld.submit(i, b)
        for i, b in enumerate(batches):
            _, sg, x = ld.next_batch()
            s.reseed(ago.batch_seed(3, i))
            w = s.sample(b)
            ok = ok and np.array_equal(sg.raw_u32()["nodes"], w["nodes"])
            ok = ok and np.array_equal(x.cpu().numpy().view(np.uint32), ago.gather(payload, n, dim, dtype, w["nodes"]).view(np.uint32))
    feats.check()
print("BULK ok=%s" % ok)
sys.exit(0 if ok else 1)
"""


def test_staged_bulk_copy_gather_gives_the_same_rows(tmp_path):
    """AG_GATHER_BULK=1 sends the chains' gathers through shared memory (cp.async.bulk + mbarrier):
    same rows, bit for bit, at row sizes from 16 bytes to 512, ragged and empty batches."""
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "bulk_worker.py"
    script.write_text(_BULK_WORKER)
    r = subprocess.run([sys.executable, str(script)], env=dict(os.environ, AG_ROOT=root, AG_GATHER_BULK="1"),
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "BULK ok=True" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]

"""The block-scaled int8 feature payload on the GPU
(crates/aethergraph-core/src/internal/feature_codec.rs; device decode
crates/aether-stream/src/gpu/kernels/quant/feature_dequant.cu:21-75): the encoder's
codes and scales and the gather's decoded rows are bit-identical to the CPU
restatement of the reference codec."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dim", [128, 256, 96, 40, 16, 7, 1])
def test_encode_and_gather_match_the_codec(dim):
    import torch

    import aethergraph_b200 as ag
    from oracle import ago

    n = 3001
    rng = np.random.default_rng(dim)
    x = rng.standard_normal((n, dim)).astype(np.float32) * rng.choice([1e-3, 1.0, 300.0], size=(n, 1)).astype(np.float32)
    x[5] = 0.0                                   # all-zero blocks
    x[6, : min(dim, 32)] = 0.0
    x[7, 0] = 1000.0                             # one block's peak must not crush the others
    store = ag.FeatureStore.from_array(x, dtype="i8")
    codes, scales = ago.encode_i8(x)
    assert store.dtype == "i8" and store.feature_dim == dim
    assert np.array_equal(store.payload_to_host().reshape(n, dim), codes)
    assert np.array_equal(store.scales_to_host().view(np.uint32), scales.view(np.uint32))
    ids = np.concatenate([rng.integers(0, n, 5000), [0, n - 1, 5, 6, 7]])
    want = ago.gather_i8(codes, scales, ids)
    got = store.gather(torch.from_numpy(ids).cuda())
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert np.array_equal(store.get_batch(ids[:64]).view(np.uint32), want[:64].view(np.uint32))
    # the same from a CUDA tensor
    again = ag.FeatureStore.from_array(torch.from_numpy(x).cuda(), dtype="i8")
    assert np.array_equal(again.payload_to_host().reshape(n, dim), codes)
    with pytest.raises(ValueError, match="out of bounds"):
        store.get_batch([n])


def test_int8_refusals():
    import aethergraph_b200 as ag
    from aethergraph_b200 import synth

    bad = np.ones((4, 32), dtype=np.float32)
    bad[2, 3] = np.inf
    with pytest.raises(ValueError, match="finite"):
        ag.FeatureStore.from_array(bad, dtype="i8")
    with pytest.raises(ValueError, match="Invalid dtype"):
        ag.save_features("/tmp/never-written.bin", np.ones((2, 2), dtype=np.float32), dtype="i8")
    shards = [synth.features(64, 32, "i8", 1, row_range=(0, 32)), synth.features(64, 32, "i8", 1, row_range=(32, 64))]
    with pytest.raises(ValueError, match="cannot be sharded"):
        ag.FeatureStore.view_sharded(shards, 0)


def test_loader_gathers_int8_rows_and_generator_matches_its_f32_table():
    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from helpers import rmat_csr
    from oracle import ago

    n, off, dst, _ = rmat_csr(12, 12, seed=2)
    dim = 256
    store = synth.features(n, dim, "i8", 31)
    f32 = ago.decode(ago.synth_features(n, dim, "f32", 31), "f32").reshape(n, dim)
    codes, scales = ago.encode_i8(f32)          # the generator quantises the rows of its f32 table
    assert np.array_equal(store.payload_to_host().reshape(n, dim), codes)
    assert np.array_equal(store.scales_to_host().view(np.uint32), scales.view(np.uint32))
    g = ag.Graph.from_csr(off, dst)
    s = ago.Sampler(off, dst, [10, 5], seed=3)
    rng = np.random.default_rng(0)
    batches = [rng.integers(0, n, 128).astype(np.uint32) for _ in range(10)]
    with ag.NeighborLoader(g, ag.SamplingConfig(num_neighbors=[10, 5], seed=3), prefetch_depth=4, sampler_threads=2,
                           features=store, group=4) as ld:
        ld.submit_epoch(batches)
        for i, b in enumerate(batches):
            idx, sg, x = ld.next_batch()
            s.reseed(ago.batch_seed(3, i))
            want = s.sample(b)
            assert idx == i and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
            assert np.array_equal(x.cpu().numpy().view(np.uint32), ago.gather_i8(codes, scales, want["nodes"]).view(np.uint32))

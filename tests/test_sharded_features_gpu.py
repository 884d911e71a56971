"""Feature stores sharded by vertex range: the gather must return exactly the rows
of the unsharded store (bit-exact), whichever GPU's memory a row lives in.

- one GPU: the shards all live on device 0 and are joined with view_sharded —
  covers the kernel's shard lookup, every dtype, the loader path and the errors;
- two or more GPUs (skipped on a one-GPU box): one process per GPU, shards
  exchanged as CUDA IPC handles, remote rows read over NVLink by the gather kernel.
"""
import os
import subprocess
import sys

import numpy as np
import pytest

from helpers import rmat_csr

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype,dim", [("bf16", 256), ("f16", 64), ("f32", 24), ("bf16", 5)])
@pytest.mark.parametrize("world", [2, 3])
def test_sharded_view_on_one_gpu_matches_the_unsharded_store(dtype, dim, world, tmp_path):
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import dist
    from oracle import ago

    n = 5003
    feats = np.random.default_rng(dim).standard_normal((n, dim)).astype(np.float32)
    path = tmp_path / "f.bin"
    ag.save_features(str(path), feats, dtype=dtype)
    shards = [ag.FeatureStore.load(str(path), row_range=dist.shard_range(r, n, world)) for r in range(world)]
    payload = ago.encode(feats, dtype)
    ids = np.concatenate([np.random.default_rng(1).integers(0, n, 4000), [0, n - 1], np.arange(n - 40, n)])
    want = ago.gather(payload, n, dim, dtype, ids.astype(np.uint32))
    for rank in range(world):
        view = ag.FeatureStore.view_sharded(shards, rank)
        assert view.num_nodes == n and view.feature_dim == dim
        got = view.gather(torch.from_numpy(ids).cuda())
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
        assert np.array_equal(view.get_batch(ids[:100]).view(np.uint32), want[:100].view(np.uint32))
        with pytest.raises(ValueError, match="out of bounds"):
            view.get_batch([n])
    with pytest.raises(ValueError, match="must hold rows"):
        ag.FeatureStore.view_sharded(shards[::-1], 0)


@pytest.mark.parametrize("dtype,dim", [("bf16", 256), ("f32", 24), ("f16", 7)])
@pytest.mark.parametrize("world", [2, 3, 8])
def test_cyclic_shards_from_file_and_generator(dtype, dim, world, tmp_path):
    """Rows dealt round-robin (row v in shard v % world): the view returns the rows of
    the whole table; a bare cyclic shard refuses to be read by global id."""
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from oracle import ago

    n = 5003
    payload = ago.synth_features(n, dim, dtype, 31)
    feats = ago.decode(payload, dtype).reshape(n, dim)
    path = tmp_path / "f.bin"
    ag.save_features(str(path), feats, dtype=dtype)   # re-encoding decoded values is exact
    ids = np.concatenate([np.random.default_rng(2).integers(0, n, 4000), np.arange(0, 3 * world), np.arange(n - 20, n)])
    want = ago.gather(payload, n, dim, dtype, ids.astype(np.uint32))
    from_file = [ag.FeatureStore.load_shard(str(path), r, world, "cyclic") for r in range(world)]
    generated = [synth.features_shard(n, dim, dtype, 31, r, world, "cyclic") for r in range(world)]
    for shards in (from_file, generated):
        assert sum(s.payload_to_host().size for s in shards) == payload.size
        view = ag.FeatureStore.view_sharded(shards, world - 1)
        got = view.gather(torch.from_numpy(ids).cuda())
        assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    with pytest.raises(ValueError, match="sharded view"):
        generated[0].gather(torch.from_numpy(ids).cuda())
    with pytest.raises(ValueError, match="layout"):
        ag.FeatureStore.view_sharded([generated[0]] + [synth.features_shard(n, dim, dtype, 31, r, world, "range")
                                                       for r in range(1, world)], 0)


def test_loader_with_sharded_features_matches_the_oracle():
    import aethergraph_b200 as ag
    from aethergraph_b200 import dist, synth
    from oracle import ago

    n, off, dst, _ = rmat_csr(12, 12, seed=3)
    g = ag.Graph.from_csr(off, dst)
    dim, world = 128, 4
    shards = [synth.features(n, dim, "bf16", 9, row_range=dist.shard_range(r, n, world)) for r in range(world)]
    view = ag.FeatureStore.view_sharded(shards, 1)
    payload = ago.synth_features(n, dim, "bf16", 9)
    cfg = ag.SamplingConfig(num_neighbors=[8, 4], seed=5)
    s = ago.Sampler(off, dst, [8, 4], seed=5)
    rng = np.random.default_rng(0)
    batches = [rng.integers(0, n, 200).astype(np.uint32) for _ in range(12)]
    with ag.NeighborLoader(g, cfg, prefetch_depth=4, sampler_threads=2, features=view) as ld:
        for i, b in enumerate(batches):
            ld.submit(i, b)
        for i, b in enumerate(batches):
            idx, sg, x = ld.next_batch()
            s.reseed(ago.batch_seed(5, i))
            want = s.sample(b)
            assert idx == i and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
            xw = ago.gather(payload, n, dim, "bf16", want["nodes"])
            assert np.array_equal(x.cpu().numpy().view(np.uint32), xw.view(np.uint32))


@pytest.mark.parametrize("order", ["ordered", "direct"])
@pytest.mark.parametrize("layout", ["range", "cyclic"])
def test_chains_over_sharded_features_fetch_each_row_once_and_in_place(layout, order):
    """A launch chain over a sharded store gathers its rows in address order, a row
    named by several batches once ("ordered"), or every row from its owner where the
    request stands ("direct").  Batches that share most of their vertices (the
    same seeds), batches far larger than the chain before them (rows past the
    estimate take the unsorted pass) and empty batches must all come out exactly
    as the oracle's rows."""
    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from oracle import ago

    n, off, dst, _ = rmat_csr(13, 12, seed=4)
    g = ag.Graph.from_csr(off, dst)
    dim, world = 64, 4
    shards = [synth.features_shard(n, dim, "bf16", 17, r, world, layout) for r in range(world)]
    view = ag.FeatureStore.view_sharded(shards, 2)
    view.set_gather_order(order)
    payload = ago.synth_features(n, dim, "bf16", 17)
    s = ago.Sampler(off, dst, [10, 5], seed=11)
    rng = np.random.default_rng(5)
    same = rng.integers(0, n, 300).astype(np.uint32)
    batches = [rng.integers(0, n, 4).astype(np.uint32) for _ in range(8)]          # a small chain first
    batches += [same.copy() for _ in range(8)]                                      # then big, overlapping ones
    batches += [np.empty(0, dtype=np.uint32), rng.integers(0, n, 700).astype(np.uint32)]
    batches += [rng.integers(0, n, 50).astype(np.uint32) for _ in range(6)]
    with ag.NeighborLoader(g, ag.SamplingConfig(num_neighbors=[10, 5], seed=11), prefetch_depth=8, sampler_threads=1,
                           features=view, group=8) as ld:
        for i, b in enumerate(batches):
            ld.submit(i, b)
        for i, b in enumerate(batches):
            idx, sg, x = ld.next_batch()
            s.reseed(ago.batch_seed(11, i))
            want = s.sample(b)
            assert idx == i and np.array_equal(sg.raw_u32()["nodes"], want["nodes"])
            xw = ago.gather(payload, n, dim, "bf16", want["nodes"])
            assert np.array_equal(x.cpu().numpy().view(np.uint32).reshape(-1, dim), xw.view(np.uint32).reshape(-1, dim)), i


def test_sorted_and_unsorted_sharded_gather_agree_on_duplicates():
    """ag_gather on a sharded view: ids with many repeats, in both id widths."""
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from oracle import ago

    n, dim, world = 9001, 256, 8
    shards = [synth.features_shard(n, dim, "f16", 3, r, world, "cyclic") for r in range(world)]
    view = ag.FeatureStore.view_sharded(shards, 0)
    payload = ago.synth_features(n, dim, "f16", 3)
    rng = np.random.default_rng(9)
    ids = np.concatenate([rng.integers(0, 50, 6000), rng.integers(0, n, 6000), [n - 1] * 40, [0] * 40])
    rng.shuffle(ids)
    want = ago.gather(payload, n, dim, "f16", ids.astype(np.uint32))
    for order in ("ordered", "direct", "auto"):
        view.set_gather_order(order)
        before = view.gather_stats()
        for t in (torch.from_numpy(ids).cuda(), torch.from_numpy(ids.astype(np.int32)).cuda()):
            got = view.gather(t)
            assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
        asked, loaded, _ = (a - b for a, b in zip(view.gather_stats(), before))
        assert asked == 2 * len(ids)
        # only the ordered gather merges repeats (a run of equal rows is loaded once per four requests)
        assert (loaded < asked) if order == "ordered" else (loaded == asked)
    with pytest.raises(ValueError, match="gather order"):
        view.set_gather_order("sideways")
    with pytest.raises(ValueError, match="out of bounds"):
        view.gather(torch.from_numpy(np.concatenate([ids, [n]])).cuda())
        view.check()


_WORKER = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, os.environ["AG_ROOT"]); sys.path.insert(0, os.path.join(os.environ["AG_ROOT"], "tests"))
import aethergraph_b200 as ag
from aethergraph_b200 import synth
from aethergraph_b200 import dist as agd
from oracle import ago
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo")
n, dim, dtype = 200_003, 256, "bf16"
local = synth.features_shard(n, dim, dtype, 21, rank, world, "cyclic")   # rows dealt round-robin
view = agd.open_sharded_features(local)
payload = ago.synth_features(n, dim, dtype, 21)
ids = np.random.default_rng(100 + rank).integers(0, n, 50_000)
want = ago.gather(payload, n, dim, dtype, ids.astype(np.uint32))
ok = True
for order in ("auto", "ordered", "direct"):
    view.set_gather_order(order)
    got = view.gather(torch.from_numpy(ids).cuda())
    ok = ok and np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
remote = float(np.mean(ids[:2000] % world != rank))
# the loader path over the sharded view
from helpers import rmat_csr
nn, off, dst, _ = rmat_csr(14, 8, seed=2)
g = ag.Graph.from_csr(off, dst)
loc2 = synth.features(nn, 64, "f16", 4, row_range=agd.shard_range(rank, nn, world))
v2 = agd.open_sharded_features(loc2)
p2 = ago.synth_features(nn, 64, "f16", 4)
s = ago.Sampler(off, dst, [6, 3], seed=8)
with ag.NeighborLoader(g, ag.SamplingConfig(num_neighbors=[6, 3], seed=8), 2, 2, features=v2) as ld:
    seeds = np.random.default_rng(rank).integers(0, nn, 300).astype(np.uint32)
    ld.submit(0, seeds)
    _, sg, x = ld.next_batch()
    s.reseed(ago.batch_seed(8, 0))
    w = s.sample(seeds)
    ok = ok and np.array_equal(sg.raw_u32()["nodes"], w["nodes"])
    ok = ok and np.array_equal(x.cpu().numpy().view(np.uint32), ago.gather(p2, nn, 64, "f16", w["nodes"]).view(np.uint32))
torch.cuda.synchronize()
dist.barrier()   # nobody frees a shard while a peer may still read it
print(f"RANK{rank} ok={ok} remote_share={remote:.2f}", flush=True)
del view, v2
dist.barrier()
dist.destroy_process_group()
sys.exit(0 if ok else 1)
"""


@pytest.mark.parametrize("alloc", ["block", "cudamalloc"])
def test_ipc_shards_across_processes_and_gpus(tmp_path, alloc):
    """Shards mapped across processes: as shareable blocks (file descriptor over a unix
    socket, large pages) and, for payloads that are plain device allocations, through
    legacy CUDA IPC handles."""
    import torch

    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, AG_ROOT=ROOT, NCCL_NVLS_ENABLE="0", AG_FEATURE_ALLOC=alloc)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    for k in range(world):
        assert f"RANK{k} ok=True" in r.stdout


def test_c5_shaped_batch_over_eight_shards():
    """The sharded-feature configuration at small scale: 4096 seeds, fanout [15,10,5],
    128-dim bf16 rows split into 8 vertex-range shards (all on this GPU)."""
    import aethergraph_b200 as ag
    from aethergraph_b200 import dist, synth
    from oracle import ago

    n, off, dst, _ = rmat_csr(16, 12, seed=12)
    g = ag.Graph.from_csr(off, dst)
    shards = [synth.features(n, 128, "bf16", 6, row_range=dist.shard_range(r, n, 8)) for r in range(8)]
    view = ag.FeatureStore.view_sharded(shards, 5)
    payload = ago.synth_features(n, 128, "bf16", 6)
    seeds = np.random.default_rng(3).integers(0, n, 4096).astype(np.uint32)
    sg = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[15, 10, 5], seed=9), features=view).sample(seeds)
    want = ago.Sampler(off, dst, [15, 10, 5], seed=9).sample(seeds)
    got = sg.raw_u32()
    for k in ("nodes", "edge_src", "edge_dst", "src_local", "dst_local", "seed_locals"):
        assert np.array_equal(got[k], want[k]), k
    xw = ago.gather(payload, n, 128, "bf16", want["nodes"])
    assert np.array_equal(sg.x.cpu().numpy().view(np.uint32), xw.view(np.uint32))
    assert len(want["nodes"]) > 20_000


@pytest.mark.parametrize("order", ["ordered", "direct"])
@pytest.mark.parametrize("layout,dtype,dim", [("cyclic", "bf16", 64), ("range", "f16", 24), ("cyclic", "f32", 5)])
def test_hot_rows_copy_serves_the_same_bits(layout, dtype, dim, order):
    """A sharded view with a local copy of the highest in-degree rows returns the same
    rows as without one, through the address-ordered gather (large id lists), the
    plain one (short lists, odd row sizes) and the loader; the counters tell the copy's
    share; the hot list is the in-degree order of the graph."""
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import synth
    from oracle import ago

    n, off, dst, _ = rmat_csr(13, 12, seed=6)
    g = ag.Graph.from_csr(off, dst)
    world = 4
    shards = [synth.features_shard(n, dim, dtype, 23, r, world, layout) for r in range(world)]
    view = ag.FeatureStore.view_sharded(shards, 1)
    view.set_gather_order(order)
    payload = ago.synth_features(n, dim, dtype, 23)
    row = dim * (4 if dtype == "f32" else 2)
    copied = view.cache_hot_rows(g, 300 * row)
    indeg = np.bincount(dst, minlength=n)
    assert copied == min(300, int((indeg > 0).sum()))
    rng = np.random.default_rng(3)
    hot = np.argsort(-indeg, kind="stable")[:copied]
    ids = np.concatenate([rng.integers(0, n, 5000), hot, hot[:50], [0, n - 1]])
    rng.shuffle(ids)
    want = ago.gather(payload, n, dim, dtype, ids.astype(np.uint32))
    got = view.gather(torch.from_numpy(ids).cuda())
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    short = view.gather(torch.from_numpy(ids[:100]).cuda())
    assert np.array_equal(short.cpu().numpy().view(np.uint32), want[:100].view(np.uint32))
    asked, loaded, from_copy = view.gather_stats()
    if row % 16 == 0:
        # the short list takes the direct kernel in either mode
        assert asked == len(ids) + 100 and loaded <= asked and from_copy >= copied * 0.9  # every hot row was asked for
        # rows the degree order puts in the copy are served from it
        assert from_copy <= loaded
    s = ago.Sampler(off, dst, [8, 4], seed=2)
    seeds = rng.integers(0, n, 256).astype(np.uint32)
    sg = ag.NeighborSampler(g, ag.SamplingConfig(num_neighbors=[8, 4], seed=2), features=view).sample(seeds)
    w = s.sample(seeds)
    assert np.array_equal(sg.raw_u32()["nodes"], w["nodes"])
    assert np.array_equal(sg.x.cpu().numpy().view(np.uint32), ago.gather(payload, n, dim, dtype, w["nodes"]).view(np.uint32))
    # dropping the copy gives the plain view back
    assert view.cache_hot_rows(g, 0) == 0
    got = view.gather(torch.from_numpy(ids).cuda())
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))
    assert view.gather_stats()[2] == 0

"""The allocation-free seed registration entry point, ag_register_seeds_static.

It exists for callers that cannot allocate device memory while they run — code
inside a memory-pool or stream callback, a process whose device memory is fully
budgeted to another allocator, a loop that cannot afford the device-wide
synchronisation cudaMalloc / cudaFree imply.  Its scratch is a fixed array inside
the library, shared by every call on the device.

The test calls it through the C ABI twice in a row (the second call meets the
first call's leftovers in the shared scratch) and compares nodes, per-seed local
indices and the distinct count with what the regular, allocating entry point
(ag_sample_into on a sampler handle, fanout 0) returns for the same seeds.
The CPU oracle's seed registration (a sampler with fanout 0) is checked beside
it, so the comparison is anchored to the reference's algorithm and not only to
this library's other path.  Bit-exact: these are ids and indices.  This file
sorts last on purpose, so a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _reference(ag, graph, seeds):
    """Distinct seeds in first-sighting order and each seed's local index, from the
    existing entry point: a sampler with fanout 0 registers the seeds and expands nothing."""
    s = ag.NeighborSampler(graph, ag.SamplingConfig(num_neighbors=[0], seed=1))
    raw = s.sample(seeds).raw_u32()
    return raw["nodes"], raw["seed_locals"]


def _static(lib_mod, device, seeds, num_nodes):
    import torch

    L = lib_mod.lib()
    n = len(seeds)
    dev = torch.device("cuda", device)
    seeds_dev = torch.from_numpy(seeds.view(np.int32)).to(dev)
    nodes = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
    locals_ = torch.full((max(n, 1),), -1, dtype=torch.int32, device=dev)
    count_err = torch.full((2,), -1, dtype=torch.int32, device=dev)
    st = torch.cuda.current_stream(dev).cuda_stream
    lib_mod.check(L.ag_register_seeds_static(device, seeds_dev.data_ptr() if n else None, n, num_nodes,
                                             nodes.data_ptr(), locals_.data_ptr(), count_err.data_ptr(), st))
    torch.cuda.synchronize(dev)
    count, err = (int(v) for v in count_err.cpu().numpy().view(np.uint32))
    return (nodes.cpu().numpy().view(np.uint32)[:count], locals_.cpu().numpy().view(np.uint32)[:n], count, err)


def test_register_seeds_static_matches_sampler_twice():
    import torch

    import aethergraph_b200 as ag
    from aethergraph_b200 import _lib

    device = torch.cuda.current_device()
    num_nodes = 50_000
    # the graph only supplies num_nodes: seed registration reads no edges
    graph = ag.Graph.from_csr(np.zeros(num_nodes + 1, dtype=np.uint64), np.zeros(0, dtype=np.uint32))
    rng = np.random.default_rng(5)
    first = rng.integers(0, 3000, size=8192).astype(np.uint32)      # the maximum size, many duplicates
    second = rng.integers(0, num_nodes, size=1000).astype(np.uint32)  # smaller: must not see stale entries
    from oracle import ago

    off = np.zeros(num_nodes + 1, dtype=np.uint64)
    for seeds in (first, second):
        want_nodes, want_locals = _reference(ag, graph, seeds)
        cpu = ago.Sampler(off, np.zeros(0, dtype=np.uint32), [0], seed=1).sample(seeds)
        assert np.array_equal(want_nodes, cpu["nodes"]) and np.array_equal(want_locals, cpu["seed_locals"])
        nodes, locals_, count, err = _static(_lib, device, seeds, num_nodes)
        assert err == 0
        assert count == len(want_nodes)
        assert np.array_equal(nodes, want_nodes)
        assert np.array_equal(locals_, want_locals)
        assert np.array_equal(nodes[locals_], seeds)


def test_register_seeds_static_limits_and_errors():
    import torch

    import aethergraph_b200 as ag  # noqa: F401  (loads the library)
    from aethergraph_b200 import _lib

    L = _lib.lib()
    device = torch.cuda.current_device()
    assert L.ag_register_seeds_static_max() == 8192
    dummy = torch.zeros(8, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="at most 8192 seeds"):
        _lib.check(L.ag_register_seeds_static(device, dummy.data_ptr(), 8193, 10, dummy.data_ptr(),
                                              dummy.data_ptr(), dummy.data_ptr(), None))
    # an out-of-range seed is reported in the error word, the rest is still registered
    seeds = np.array([3, 99, 3, 7], dtype=np.uint32)
    nodes, locals_, count, err = _static(_lib, device, seeds, 50)
    assert err == 8 and count == 2
    assert nodes.tolist() == [3, 7] and locals_.tolist() == [0, 0xFFFFFFFF, 0, 1]
    # empty batch
    nodes, locals_, count, err = _static(_lib, device, np.zeros(0, dtype=np.uint32), 50)
    assert count == 0 and err == 0

"""Host logic of the epoch driver (no GPU): seed batching, per-epoch seeds, input parsing.
Mirrors python/aethergraph/pytorch/loader.py:54-205 of the reference."""
import math

import numpy as np
import pytest

from aethergraph_b200.pytorch.loader import epoch_sampling_seed, make_batch_getter, normalize_input_nodes


def test_range_and_sliced_batches():
    get = make_batch_getter(None, 10, 4, False, np.random.default_rng(0))
    assert [get(b)[0].tolist() for b in range(3)] == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9]]
    nodes = np.array([5, 9, 2, 7, 1], dtype=np.int64)
    get = make_batch_getter(nodes, 5, 2, False, np.random.default_rng(0))
    seeds, input_id = get(1)
    assert seeds.tolist() == [2, 7] and input_id.tolist() == [2, 3]
    order = np.random.default_rng(4).permutation(5)
    get = make_batch_getter(nodes, 5, 2, True, np.random.default_rng(4))
    seeds, input_id = get(0)
    assert input_id.tolist() == order[:2].tolist() and seeds.tolist() == nodes[order[:2]].tolist()


@pytest.mark.parametrize("n", [1, 2, 97, 1000, 4096])
def test_strided_walk_is_a_permutation_and_consumes_the_generator_like_the_reference(n):
    rng = np.random.default_rng(12)
    get = make_batch_getter(None, n, 64, True, rng)
    ids = np.concatenate([get(b)[0] for b in range((n + 63) // 64)])
    assert np.array_equal(np.sort(ids), np.arange(n))
    # same draws: offset = integers(0, n); then integers(1, n) until coprime with n
    ref = np.random.default_rng(12)
    offset = int(ref.integers(0, n))
    stride = 1
    while n > 1:
        stride = int(ref.integers(1, n))
        if math.gcd(stride, n) == 1:
            break
    assert ids[0] == offset % n and (n == 1 or ids[1] == (offset + stride) % n)
    assert rng.integers(0, 1 << 30) == ref.integers(0, 1 << 30)  # both generators are in the same state


def test_epoch_sampling_seed_sequence():
    assert epoch_sampling_seed(None) is None
    a, b = np.random.SeedSequence(5), np.random.SeedSequence(5)
    s1, s2 = epoch_sampling_seed(a), epoch_sampling_seed(a)
    assert s1 != s2 and 0 <= s1 < 2**64
    assert epoch_sampling_seed(b) == s1 and epoch_sampling_seed(b) == s2
    (child,) = np.random.SeedSequence(5).spawn(1)
    assert s1 == int(child.generate_state(1, dtype=np.uint64)[0])


def test_normalize_input_nodes():
    import torch

    assert normalize_input_nodes([3, 1, 2], num_nodes=4).tolist() == [3, 1, 2]
    assert normalize_input_nodes(np.array([True, False, True]), num_nodes=3).tolist() == [0, 2]
    assert normalize_input_nodes(torch.tensor([False, True]), num_nodes=2).tolist() == [1]
    assert normalize_input_nodes(torch.tensor([1, 0], dtype=torch.int32), num_nodes=2).dtype == np.int64
    with pytest.raises(ValueError, match="integer or bool"):
        normalize_input_nodes(np.array([0.5]), num_nodes=4)
    with pytest.raises(ValueError, match="integer or bool"):
        normalize_input_nodes(torch.tensor([0.5]), num_nodes=4)
    with pytest.raises(ValueError, match="1D"):
        normalize_input_nodes(np.zeros((2, 2), dtype=np.int64), num_nodes=4)
    with pytest.raises(ValueError, match="non-negative"):
        normalize_input_nodes([-1], num_nodes=4)
    with pytest.raises(ValueError, match="out-of-range"):
        normalize_input_nodes([4], num_nodes=4)

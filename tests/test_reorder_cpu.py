"""CPU: the Rabbit Order restatement against the cases of the reference's own tests
(crates/aethergraph-core/src/graph/reorder.rs:465-930), and partition-aligned batches."""
import numpy as np
import pytest

from helpers import csr_from_edges, rmat_csr


def two_cliques():
    # reorder.rs:465-480: two 4-cliques joined by 3 <-> 4
    e = [(i, j) for i in range(4) for j in range(4) if i != j]
    e += [(i, j) for i in range(4, 8) for j in range(4, 8) if i != j] + [(3, 4), (4, 3)]
    src, dst = np.array([a for a, _ in e]), np.array([b for _, b in e])
    off, d, _ = csr_from_edges(8, src, dst)
    return off, d


def test_rabbit_order_keeps_the_cliques_contiguous_and_apart():
    # reorder.rs test_rabbit_valid_permutation / clusters_communities / partitions_two_cliques_separated
    from oracle import ago

    off, dst = two_cliques()
    perm, parts = ago.rabbit_order(off, dst)
    assert sorted(perm.tolist()) == list(range(8)) and parts.size == 8
    pos = {int(old): new for new, old in enumerate(perm)}
    c1, c2 = sorted(pos[v] for v in range(4)), sorted(pos[v] for v in range(4, 8))
    assert c1[3] - c1[0] == 3 and c2[3] - c2[0] == 3
    assert len(set(parts[:4])) == 1 and len(set(parts[4:])) == 1 and parts[0] != parts[4]
    again = ago.rabbit_order(off, dst)
    assert np.array_equal(again[0], perm) and np.array_equal(again[1], parts)   # deterministic


def test_rabbit_order_degenerate_graphs():
    # reorder.rs test_empty_graph / single_node / disconnected
    from oracle import ago

    p, q = ago.rabbit_order(np.zeros(1, np.uint64), np.zeros(0, np.uint32))
    assert p.size == 0 and q.size == 0
    p, q = ago.rabbit_order(np.zeros(2, np.uint64), np.zeros(0, np.uint32))
    assert p.tolist() == [0] and q.tolist() == [0]
    off, dst, _ = csr_from_edges(5, np.array([0, 1, 3]), np.array([1, 0, 4]))
    p, q = ago.rabbit_order(off, dst)
    assert sorted(p.tolist()) == [0, 1, 2, 3, 4] and q[0] == q[1] and q[3] == q[4] and len({q[0], q[2], q[3]}) == 3
    # only self-loops: nothing to merge, the identity
    off, dst, _ = csr_from_edges(3, np.array([0, 1, 2]), np.array([0, 1, 2]))
    p, q = ago.rabbit_order(off, dst)
    assert p.tolist() == [0, 1, 2] and q.tolist() == [0, 1, 2]


def test_rabbit_partitions_follow_backward_edges():
    # reorder.rs test_partitions_follow_backward_edges: arcs only from higher to lower ids still join
    from oracle import ago

    off, dst, _ = csr_from_edges(6, np.array([1, 2, 2, 4, 5, 5]), np.array([0, 0, 1, 3, 3, 4]))
    _, parts = ago.rabbit_order(off, dst)
    assert parts[0] == parts[1] == parts[2] and parts[3] == parts[4] == parts[5] and parts[0] != parts[3]


def test_permute_cases_of_the_reference():
    # reorder.rs test_permute_identity / reverse / preserves_weights / large_matches_reference
    from oracle import ago

    off, dst, w = csr_from_edges(3, np.array([0, 0, 1]), np.array([1, 2, 2]), np.array([1.0, 2.0, 3.0]))
    no, nd, nw = ago.permute_csr(off, dst, w, [2, 1, 0])
    assert no.tolist() == [0, 0, 1, 3] and nd.tolist() == [0, 1, 0] and nw.tolist() == [3.0, 1.0, 2.0]
    n, off, dst, _ = rmat_csr(9, 6, seed=3)
    perm = np.random.default_rng(0).permutation(n)
    no, nd, _ = ago.permute_csr(off, dst, None, perm)
    inv = np.argsort(perm)
    for new_id in (0, 5, n - 1):
        old = perm[new_id]
        assert nd[int(no[new_id]):int(no[new_id + 1])].tolist() == inv[dst[int(off[old]):int(off[old + 1])]].tolist()


def test_partition_aligned_batches():
    # reorder.rs:385-463 and its tests: grouped by partition, order kept inside one, cut into batches
    from aethergraph_b200.graph import partition_aligned_batches

    parts = np.array([0, 0, 1, 1, 2, 2, 0, 1], dtype=np.uint32)
    seeds = np.array([7, 0, 2, 6, 4, 1, 3, 5])
    b = partition_aligned_batches(parts, seeds, 3)
    assert [x.tolist() for x in b] == [[0, 6, 1], [7, 2, 3], [4, 5]]
    flat = np.concatenate(partition_aligned_batches(parts, seeds, 3, shuffle_partitions=True, seed=5))
    assert sorted(flat.tolist()) == sorted(seeds.tolist())
    runs = parts[flat]
    assert all(len(set(runs[runs == p])) == 1 for p in (0, 1, 2))
    changes = int((runs[1:] != runs[:-1]).sum())
    assert changes == 2                                     # three partitions, each visited once
    # the reference's LCG (seed * K + 1, then rng = rng * K + 1 per step, j = (rng >> 33) % (i + 1))
    K, mask = 0x517CC1B727220A95, (1 << 64) - 1
    rng, order = (5 * K + 1) & mask, [0, 1, 2]
    for i in (2, 1):
        rng = (rng * K + 1) & mask
        j = (rng >> 33) % (i + 1)
        order[i], order[j] = order[j], order[i]
    visited = [int(p) for k, p in enumerate(runs) if k == 0 or p != runs[k - 1]]
    assert visited == order
    with pytest.raises(ValueError, match="batch_size"):
        partition_aligned_batches(parts, seeds, 0)
    with pytest.raises(ValueError, match="out of range"):
        partition_aligned_batches(parts, [1, 99], 2)
    assert partition_aligned_batches(parts, [], 4) == []

"""Data-parallel partition of seed batches over ranks (one process per GPU).

The path shards with no data-path collective: batch `b` of the global stream goes
to rank `b % world`, every rank holds the CSR (and, when it fits, the features),
and batch `b` is sampled from `batch_seed(seed, b)` when rank r's loader is created
with `seed_sequence=(r, world)` (its local batch i is global batch r + world * i), so
the result does not depend on the number of ranks — the property the reference tests
for its thread pool (crates/aethergraph-core/src/loader/sampler.rs:3116-3148).
torch.distributed is only used to agree on timings and totals.
"""
from __future__ import annotations


def rank_batches(rank: int, world: int, num_batches: int) -> list[int]:
    """Global batch positions rank `rank` of `world` handles, in order."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    return list(range(rank, num_batches, world))


def owner_of_row(row: int, num_rows: int, world: int) -> int:
    """Rank that holds feature row `row` under contiguous vertex-range sharding."""
    per = -(-num_rows // world)
    return min(row // per, world - 1)


def shard_range(rank: int, num_rows: int, world: int) -> tuple[int, int]:
    per = -(-num_rows // world)
    return min(rank * per, num_rows), min((rank + 1) * per, num_rows)


def max_over_ranks(value: float, device=None) -> float:
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value: float, device=None) -> float:
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def open_sharded_features(local):
    """Every rank passes the FeatureStore holding ITS vertex range
    (`shard_range(rank, num_nodes, world)`); returns a store over all rows whose
    remote rows are read from the owning rank's GPU memory over NVLink.  The only
    communication is the one-off exchange of the 128-byte shard handles (a shard the library
    allocated is then fetched as a file descriptor from its owner and mapped with 2 MB pages)."""
    import torch.distributed as dist

    from .features import FeatureStore

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return FeatureStore.open_sharded(local, [local.ipc_handle()], 0)
    world, rank = dist.get_world_size(), dist.get_rank()
    handles: list = [None] * world
    dist.all_gather_object(handles, local.ipc_handle())
    view = FeatureStore.open_sharded(local, handles, rank)
    dist.barrier()  # every rank has mapped its peers before anyone may free a shard
    return view

"""Bandwidth probe for sharded feature stores: how fast one GPU gathers rows that
live in its peers' HBM, as a function of how much peer memory the rows are spread
over and of the order in which they are requested.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \\
        -m aethergraph_b200.shard_probe [--rows 600000] [--dim 256] [--sizes 24,48,72,96]

Every rank builds its round-robin shard of a synthetic bf16 table of `size` million
rows, maps the peers' shards (CUDA IPC) and times `FeatureStore.gather` of `--rows`
ids that are local, on one peer, on all peers or anywhere, in random order and in
address order (by owner, then by row), once with every rank gathering and once with
rank 0 alone.  The figure is stored bytes read per second.
"""
from __future__ import annotations

import argparse
import os

import torch
import torch.distributed as dist

from . import dist as agd
from . import synth


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=600_000)
    ap.add_argument("--dim", type=int, default=256)
    ap.add_argument("--sizes", default="24,96", help="table sizes in millions of rows")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("gloo")
    rows, dim = args.rows, args.dim
    row_bytes = dim * 2
    for n in [int(float(v) * 1e6) for v in args.sizes.split(",")]:
        local = synth.features_shard(n, dim, "bf16", 5, rank, world, "cyclic")
        view = agd.open_sharded_features(local)
        if rank == 0:
            print(f"table: {n} rows, {n * row_bytes / 1e9:.1f} GB over {world} GPUs", flush=True)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(rank)

        def ids_for(kind: str):
            base = torch.randint(0, n // world - 1, (rows,), device="cuda", generator=gen, dtype=torch.int64)
            if kind == "local":
                return base * world + rank
            if kind == "one_peer":
                return base * world + (rank + 1) % world
            if kind == "all_peers":
                off = torch.randint(1, max(world, 2), (rows,), device="cuda", generator=gen)
                return base * world + (rank + off) % world
            return base * world + torch.randint(0, world, (rows,), device="cuda", generator=gen)

        out = torch.empty((rows, dim), dtype=torch.float32, device="cuda")

        def timed(ids, active: bool) -> float:
            torch.cuda.synchronize()
            dist.barrier()
            ms = 0.0
            if active:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                view.gather(ids, out=out)
                e0.record()
                for _ in range(5):
                    view.gather(ids, out=out)
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / 5
            dist.barrier()
            return ms

        for kind in ("local", "one_peer", "all_peers", "anywhere"):
            for order in ("random", "address order"):
                ids = ids_for(kind)
                if order == "address order":
                    key = (ids % world) * (n // world + 1) + ids // world
                    ids = ids[torch.argsort(key)].contiguous()
                ms_all, ms_solo = timed(ids, True), timed(ids, rank == 0)
                if rank == 0:
                    gb = rows * row_bytes / 1e9
                    print(f"  {kind:9s} {order:13s} all ranks {gb / ms_all * 1e3:6.0f} GB/s   rank 0 alone "
                          f"{gb / ms_solo * 1e3:6.0f} GB/s", flush=True)
        dist.barrier()
        del view, local, out
        torch.cuda.empty_cache()
        dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

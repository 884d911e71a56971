"""Regenerates the committed golden fixtures in this folder.

    python tests/golden/make_golden.py

* simple_graph_aeth_v1.bin — the AETH v1 file of the reference's own fixture graph
  (test_data/simple_graph.txt: 0-1 0-2 1-2 1-3 2-3 3-4), built here from the format
  description (crates/aethergraph-core/src/internal/mmap.rs:114-121; golden layout
  crates/aethergraph-core/tests/golden_format.rs:22-87) with checksum 0, and compared
  byte for byte with the reference's test_data/simple_graph.bin when that tree is present.
* simple_graph_aeth_v2.bin — the same graph in the compressed version-2 format (Elias-Fano
  offsets, StreamVByte edge deltas, payload checksum), written by the numpy restatement of
  the reference's codecs (crates/aethergraph-core/src/internal/compressed_graph.rs:39-88,
  internal/succinct.rs:52-92,198-214,397-420,486-500).
* golden_samples.npz — sampled subgraphs and gathered rows the CPU oracle produces for
  fixed seeds on a small seeded R-MAT graph.  The reference holds no known-answer sample
  vectors, so these pin this repository's oracle and CUDA path against drift.
"""
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import rmat_csr  # noqa: E402
from oracle import ago  # noqa: E402


def aeth_v1_bytes(offsets, edges, weights=None, checksum=0) -> bytes:
    n, e = len(offsets) - 1, len(edges)
    head = struct.pack("<IIQQII", 0x41455448, 1, n, e, 1 if weights is not None else 0, checksum)
    body = np.asarray(offsets, dtype="<u8").tobytes() + np.asarray(edges, dtype="<u4").tobytes()
    if weights is not None:
        body += np.asarray(weights, dtype="<f4").tobytes()
    return head + body


def golden_cases():
    n, off, dst, w = rmat_csr(9, 12, seed=21, weighted=True)
    feats = np.random.default_rng(22).standard_normal((n, 24)).astype(np.float32)
    rng = np.random.default_rng(23)
    out = {"n": np.array(n), "offsets": off, "dst": dst, "weights": w, "features": feats}
    cases = {
        "uniform": dict(fanout=[6, 4], seed=42),
        "replace": dict(fanout=[5, 3], seed=43, replace=True),
        "weighted": dict(fanout=[4, 3, 2], seed=44, weighted=True),
        "deep": dict(fanout=[3, 3, 3, 3], seed=45),
    }
    for name, kw in cases.items():
        fan = kw.pop("fanout")
        seed = kw.pop("seed")
        s = ago.Sampler(off, dst, fan, weights=w if kw.get("weighted") else None, seed=seed, **kw)
        seeds = rng.integers(0, n, 48).astype(np.uint32)
        seeds[7] = seeds[2]
        out[f"{name}.seeds"] = seeds
        out[f"{name}.fanout"] = np.array(fan, dtype=np.uint32)
        out[f"{name}.seed"] = np.array(seed, dtype=np.uint64)
        for call in range(2):  # second call continues the RNG stream
            sg = s.sample(seeds)
            for k in ("nodes", "edge_src", "edge_dst", "edge_ids", "src_local", "dst_local", "seed_locals",
                      "num_sampled_nodes", "num_sampled_edges"):
                out[f"{name}.{call}.{k}"] = sg[k]
            out[f"{name}.{call}.draws"] = np.array(sg["draws"], dtype=np.uint64)
        for dtype in ("f32", "f16", "bf16"):
            payload = ago.encode(feats, dtype)
            out[f"{name}.x.{dtype}"] = ago.gather(payload, n, 24, dtype, sg["nodes"][:64])
    return out


def main():
    off = np.array([0, 2, 4, 5, 6, 6], dtype=np.uint64)
    edges = np.array([1, 2, 2, 3, 3, 4], dtype=np.uint32)
    blob = aeth_v1_bytes(off, edges)
    ref_root = os.environ.get("AETHERGRAPH_REFERENCE") or os.path.normpath(os.path.join(ROOT, "..", "reference"))
    ref = os.path.join(ref_root, "test_data", "simple_graph.bin")
    if os.path.exists(ref):
        assert open(ref, "rb").read() == blob, "format restatement differs from the reference's fixture"
        print("simple_graph: identical to the reference's test_data/simple_graph.bin")
    open(os.path.join(HERE, "simple_graph_aeth_v1.bin"), "wb").write(blob)
    open(os.path.join(HERE, "simple_graph_aeth_v2.bin"), "wb").write(ago.compressed_graph_bytes(off, edges))
    np.savez_compressed(os.path.join(HERE, "golden_samples.npz"), **golden_cases())
    print("wrote", os.listdir(HERE))


if __name__ == "__main__":
    main()

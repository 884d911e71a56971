"""`save_features` and `FeatureStore`: node features resident in GPU memory.

Mirrors `aethergraph._core.save_features` / `FeatureStore`
(python/aethergraph/_core.pyi:136-148, 482-516; crates/aethergraph-core/src/features/store.rs).
The payload keeps its stored dtype (f32 / f16 / bf16) in HBM; gathers upcast to
f32 inside the gather kernel.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib

__all__ = ["FeatureStore", "save_features"]


def save_features(path, features, dtype: str = "f32") -> None:
    """Write an AETHFEAT file: 512-byte header, then rows in `dtype`."""
    if dtype not in ("f32", "f16", "bf16"):
        raise ValueError(f"Invalid dtype '{dtype}'. Must be 'f32', 'f16', or 'bf16'")
    f = np.asarray(features)
    if f.ndim != 2:
        raise ValueError(f"features must be a 2-d array [num_nodes, feature_dim], got shape {f.shape}")
    f = np.ascontiguousarray(f, dtype=np.float32)
    _lib.check(_lib.lib().ag_features_save(os.fspath(path).encode(), f.ctypes.data if f.size else None,
                                           f.shape[0], f.shape[1], _lib.DTYPE_TAG[dtype]))


class FeatureStore:
    """Feature rows in HBM.  `get_batch` takes host ids and returns a host array
    like the reference; `gather` is the device-to-device form."""

    def __init__(self, handle: int):
        self._h = C.c_void_p(handle)
        n, d, t, dev, rb = C.c_uint64(), C.c_uint64(), C.c_int32(), C.c_int32(), C.c_uint64()
        _lib.check(_lib.lib().ag_features_info(self._h, C.byref(n), C.byref(d), C.byref(t), C.byref(dev),
                                               C.byref(rb)))
        self._n, self._dim, self._dtype, self._device, self._row_begin = n.value, d.value, t.value, dev.value, rb.value
        rows = C.c_uint64()
        _lib.check(_lib.lib().ag_features_shard(self._h, None, C.byref(rows)))
        self._rows = rows.value

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _lib.lib().ag_features_free(h)
            except Exception:
                pass
            self._h = None

    @staticmethod
    def _dev(device):
        import torch

        if device is not None:
            return device
        if not torch.cuda.is_available():
            raise RuntimeError("aethergraph_b200 needs a CUDA device; there is no CPU path")
        return torch.cuda.current_device()

    @staticmethod
    def load(path, telemetry: bool = False, *, device: int | None = None,
             row_range: tuple[int, int] | None = None) -> "FeatureStore":
        out = C.c_void_p()
        dev = FeatureStore._dev(device)
        if row_range is None:
            _lib.check(_lib.lib().ag_features_load(os.fspath(path).encode(), dev, C.byref(out)))
        else:
            _lib.check(_lib.lib().ag_features_load_range(os.fspath(path).encode(), dev, row_range[0],
                                                         row_range[1], C.byref(out)))
        return FeatureStore(out.value)

    @staticmethod
    def from_array(features, dtype: str = "f32", *, device: int | None = None) -> "FeatureStore":
        """Encode f32 rows (numpy, or a CUDA float32 tensor) into `dtype` on the device.
        `"i8"` is the reference's block-scaled int8 codec (one byte per element and one f32
        scale per 32 elements of a row, crates/aethergraph-core/src/internal/feature_codec.rs):
        lossy, a quarter of f32's bytes; gathers decode to exactly what the reference's
        `BlockScaledI8::decode` gives."""
        import torch

        if dtype not in _lib.DTYPE_TAG:
            raise ValueError(f"Invalid dtype '{dtype}'. Must be 'f32', 'f16', 'bf16', or 'i8'")
        out = C.c_void_p()
        dev = FeatureStore._dev(device)
        if isinstance(features, torch.Tensor):
            if features.dtype != torch.float32 or features.dim() != 2 or not features.is_contiguous():
                raise ValueError("features tensor must be a contiguous 2-d float32 tensor")
            kind = _lib.AG_MEM_DEVICE if features.is_cuda else _lib.AG_MEM_HOST
            _lib.check(_lib.lib().ag_features_from_f32(features.data_ptr(), features.shape[0], features.shape[1],
                                                       _lib.DTYPE_TAG[dtype], kind, dev, C.byref(out)))
            return FeatureStore(out.value)
        f = np.asarray(features)
        if f.ndim != 2:
            raise ValueError(f"features must be a 2-d array [num_nodes, feature_dim], got shape {f.shape}")
        f = np.ascontiguousarray(f, dtype=np.float32)
        _lib.check(_lib.lib().ag_features_from_f32(f.ctypes.data if f.size else None, f.shape[0], f.shape[1],
                                                   _lib.DTYPE_TAG[dtype], _lib.AG_MEM_HOST, dev, C.byref(out)))
        return FeatureStore(out.value)

    @staticmethod
    def from_payload(payload, num_nodes: int, dim: int, dtype: str, *, device: int | None = None) -> "FeatureStore":
        """Adopt rows already encoded in `dtype` (numpy array of raw bytes / bit patterns)."""
        raw = np.ascontiguousarray(payload).view(np.uint8).reshape(-1)
        want = num_nodes * dim * (4 if dtype == "f32" else 2)
        if raw.size != want:
            raise ValueError(f"payload holds {raw.size} bytes, expected {want}")
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_features_from_memory(raw.ctypes.data if raw.size else None, num_nodes, dim,
                                                      _lib.DTYPE_TAG[dtype], _lib.AG_MEM_HOST,
                                                      FeatureStore._dev(device), C.byref(out)))
        return FeatureStore(out.value)

    # -- shards over the GPUs of one node --------------------------------------
    @staticmethod
    def load_shard(path, rank: int, world: int, layout: str = "cyclic", *, device: int | None = None) -> "FeatureStore":
        """Shard `rank` of `world` of a feature file: `layout="range"` is a contiguous
        block of rows, `"cyclic"` rows rank, rank + world, ... (balanced on skewed graphs)."""
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_features_load_shard(os.fspath(path).encode(), FeatureStore._dev(device), rank, world,
                                                     _lib.SHARD_LAYOUT[layout], C.byref(out)))
        return FeatureStore(out.value)

    def ipc_handle(self) -> bytes:
        """The handle (AG_IPC_HANDLE_BYTES) the other ranks of the node need to map this shard's rows."""
        buf = C.create_string_buffer(_lib.AG_IPC_HANDLE_BYTES)
        _lib.check(_lib.lib().ag_features_ipc_export(self._h, buf))
        return buf.raw

    @staticmethod
    def open_sharded(local: "FeatureStore", handles: list[bytes], rank: int) -> "FeatureStore":
        """A store over ALL rows whose shard `r` lives in rank r's GPU memory: `local`
        is this rank's shard (rows `dist.shard_range(rank, n, world)`), `handles` the
        `ipc_handle()` of every rank in rank order.  Remote rows are read over NVLink
        by the gather kernel itself."""
        world = len(handles)
        blob = b"".join(h if len(h) == _lib.AG_IPC_HANDLE_BYTES else b"\0" * _lib.AG_IPC_HANDLE_BYTES for h in handles)
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_features_open_sharded(local._h, world, rank, blob, C.byref(out)))
        view = FeatureStore(out.value)
        view._keep = local  # the view borrows the local shard's memory
        return view

    @staticmethod
    def view_sharded(shards: list["FeatureStore"], rank: int) -> "FeatureStore":
        """The same view inside ONE process that holds every shard (one per GPU, peer access)."""
        arr = (C.c_void_p * len(shards))(*[s._h for s in shards])
        out = C.c_void_p()
        _lib.check(_lib.lib().ag_features_view_sharded(arr, len(shards), rank, C.byref(out)))
        view = FeatureStore(out.value)
        view._keep = list(shards)
        return view

    @property
    def num_nodes(self) -> int:
        return self._n

    @property
    def feature_dim(self) -> int:
        return self._dim

    @property
    def dtype(self) -> str:
        return _lib.DTYPE_NAME[self._dtype]

    @property
    def device(self) -> int:
        return self._device

    def get_batch(self, nodes) -> np.ndarray:
        """Rows of `nodes` (int64 ids) as f32 [n, dim]; an id outside the store raises ValueError."""
        ids = np.ascontiguousarray(np.asarray(nodes), dtype=np.int64).reshape(-1)
        out = np.empty((len(ids), self._dim), dtype=np.float32)
        _lib.check(_lib.lib().ag_features_get_batch(self._h, ids.ctypes.data if len(ids) else None, len(ids),
                                                    out.ctypes.data if out.size else None))
        return out

    def get(self, node: int) -> np.ndarray:
        return self.get_batch(np.array([node], dtype=np.int64))[0]

    def features(self) -> np.ndarray:
        """The whole store decoded to f32 (host)."""
        return self.get_batch(np.arange(self._row_begin, self._row_begin + self._rows, dtype=np.int64))

    def payload_to_host(self) -> np.ndarray:
        """The stored (encoded) rows held by this handle as a flat host array
        (float32 for f32 stores, uint16 bit patterns for f16 / bf16)."""
        kind = {_lib.AG_F32: np.float32, _lib.AG_I8: np.int8}.get(self._dtype, np.uint16)
        out = np.empty(self._rows * self._dim, dtype=kind)
        if out.size:
            _lib.check(_lib.lib().ag_features_copy_to_host(self._h, out.ctypes.data))
        return out

    def scales_to_host(self) -> np.ndarray:
        """`"i8"` stores: the per-block scales, f32 [rows, ceil(dim / 32)]."""
        out = np.empty((self._rows, (self._dim + 31) // 32), dtype=np.float32)
        if out.size:
            _lib.check(_lib.lib().ag_features_scales_to_host(self._h, out.ctypes.data))
        return out

    def gather(self, ids, out=None, stream=None):
        """Device gather: `ids` is a CUDA tensor (int64, or int32 holding u32 ids);
        returns a float32 CUDA tensor [len(ids), dim]."""
        import torch

        if not ids.is_cuda or not ids.is_contiguous() or ids.dtype not in (torch.int64, torch.int32):
            raise ValueError("ids must be a contiguous CUDA tensor of dtype int64 or int32")
        n = ids.numel()
        if out is None:
            out = torch.empty((n, self._dim), dtype=torch.float32, device=ids.device)
        st = stream if stream is not None else torch.cuda.current_stream(ids.device).cuda_stream
        _lib.check(_lib.lib().ag_gather(self._h, ids.data_ptr() if n else None, int(ids.dtype == torch.int64), n,
                                        None, out.data_ptr() if n else None, st))
        return out

    def gather_stats(self) -> tuple[int, int, int]:
        """Sharded views: `(rows requested, rows loaded, rows loaded from the local copy of
        the hot rows)` by the address-ordered gathers so far; requested - loaded is rows that
        several batches of one launch chain named."""
        a, b, c = C.c_uint64(), C.c_uint64(), C.c_uint64()
        _lib.check(_lib.lib().ag_features_gather_stats(self._h, C.byref(a), C.byref(b), C.byref(c)))
        return a.value, b.value, c.value

    def set_gather_order(self, order: str = "auto") -> None:
        """Sharded views: "direct" loads every row from its owner where the request stands,
        "ordered" sorts the requests of a launch chain into address order first and loads
        repeats once, "auto" (the default) picks direct unless a peer is mapped through a
        legacy CUDA IPC handle.  Same bits either way."""
        modes = {"auto": 0, "ordered": 1, "direct": 2}
        if order not in modes:
            raise ValueError(f"gather order must be one of {sorted(modes)}, got {order!r}")
        _lib.check(_lib.lib().ag_features_set_gather_order(self._h, modes[order]))

    def cache_hot_rows(self, graph, max_bytes: int = 1 << 30) -> int:
        """Sharded views: keep a copy of the rows of the highest in-degree vertices of
        `graph` in this GPU's memory, `max_bytes` of them at most, and serve them from
        there (only the remaining rows cross NVLink).  Returns the number of rows copied."""
        row = self._dim * (4 if self._dtype == _lib.AG_F32 else 2)
        want = int(max_bytes) // max(row, 1)
        ids, n = C.c_void_p(), C.c_uint64()
        _lib.check(_lib.lib().ag_graph_hot_vertices(graph._h, want, C.byref(ids), C.byref(n)))
        try:
            _lib.check(_lib.lib().ag_features_cache_rows(self._h, ids, n.value))
        finally:
            if ids.value:
                _lib.lib().ag_synth_free_device(ids, self._device)
        return n.value

    def check(self) -> None:
        """Raise ValueError if a device gather since the last check saw an out-of-range id."""
        _lib.check(_lib.lib().ag_features_check(self._h))

    def telemetry(self):
        return None

    def __repr__(self) -> str:
        return (f"FeatureStore(num_nodes={self._n}, feature_dim={self._dim}, dtype={self.dtype}, "
                f"device=cuda:{self._device})")

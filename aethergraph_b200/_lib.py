"""ctypes binding of libaethergpu.so (the CUDA kernels behind the C ABI).

There is no fallback of any kind: if the shared library is missing or cannot be
loaded this module raises, and every compute entry point fails loudly when no
CUDA device is usable.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libaethergpu.so")

AG_OK, AG_ERR_VALUE, AG_ERR_LOAD, AG_ERR_SAMPLING, AG_ERR_TIMEOUT, AG_ERR_WORKER, AG_ERR_CUDA, \
    AG_ERR_SHUTDOWN = range(8)
AG_MEM_HOST, AG_MEM_DEVICE = 0, 1
AG_F32, AG_F16, AG_BF16, AG_I8 = 0, 1, 2, 3
DTYPE_TAG = {"f32": AG_F32, "f16": AG_F16, "bf16": AG_BF16, "i8": AG_I8}
DTYPE_NAME = {v: k for k, v in DTYPE_TAG.items()}
VALIDATION = {"auto": 0, "header_only": 1, "offsets_only": 2, "full": 3}
AG_RNG_WYRAND_EXACT, AG_RNG_PHILOX = 0, 1
RNG_MODE = {"wyrand_exact": AG_RNG_WYRAND_EXACT, "philox": AG_RNG_PHILOX,
            "philox_fast": AG_RNG_PHILOX}
AG_MAX_HOPS = 8
AG_IPC_HANDLE_BYTES = 128
SHARD_LAYOUT = {"range": 0, "cyclic": 1}


class GraphLoadError(Exception):
    """Raised when graph loading fails."""


class SamplingError(Exception):
    """Raised when sampling fails."""


class SamplingConfigC(C.Structure):
    _fields_ = [("num_hops", C.c_uint32), ("fanout", C.c_uint32 * AG_MAX_HOPS),
                ("replace", C.c_int32), ("weighted", C.c_int32), ("track_edge_ids", C.c_int32),
                ("seed", C.c_uint64), ("rng_mode", C.c_int32), ("max_seeds", C.c_uint32)]


class SubgraphBuffers(C.Structure):
    _fields_ = [("cap_nodes", C.c_uint64), ("cap_edges", C.c_uint64), ("cap_seeds", C.c_uint64),
                ("nodes", C.c_void_p), ("edge_src", C.c_void_p), ("edge_dst", C.c_void_p),
                ("edge_ids", C.c_void_p), ("src_local", C.c_void_p), ("dst_local", C.c_void_p),
                ("seed_locals", C.c_void_p), ("n_id", C.c_void_p),
                ("edge_index_local", C.c_void_p), ("e_id", C.c_void_p),
                ("seed_index", C.c_void_p), ("x", C.c_void_p), ("cap_x", C.c_uint64)]


class SampleCounts(C.Structure):
    _fields_ = [("num_nodes", C.c_uint32), ("num_edges", C.c_uint32), ("num_seeds", C.c_uint32),
                ("num_hops", C.c_uint32), ("nodes_per_hop", C.c_uint32 * (AG_MAX_HOPS + 1)),
                ("edges_per_hop", C.c_uint32 * AG_MAX_HOPS), ("draws", C.c_uint64),
                ("error", C.c_uint32), ("reserved", C.c_uint32),
                ("sample_ms", C.c_float), ("gather_ms", C.c_float),
                ("gather_begin_ms", C.c_double), ("gather_end_ms", C.c_double)]


class Batch(C.Structure):
    _fields_ = [("batch_idx", C.c_int64), ("seq", C.c_uint64), ("bufs", SubgraphBuffers),
                ("counts", SampleCounts), ("owned", C.c_int32), ("reserved", C.c_int32)]


class LoaderStats(C.Structure):
    _fields_ = [("hits", C.c_uint64), ("misses", C.c_uint64), ("total", C.c_uint64),
                ("sample_time_ns", C.c_uint64), ("feature_load_time_ns", C.c_uint64),
                ("submitted", C.c_uint64), ("edges", C.c_uint64), ("nodes", C.c_uint64),
                ("gather_ms", C.c_double), ("sample_ms", C.c_double), ("chains", C.c_uint64)]


AG_MAX_NODE_TYPES, AG_MAX_EDGE_TYPES = 8, 16


class HeteroBuffers(C.Structure):
    _fields_ = [("cap_nodes", C.c_uint64), ("cap_edges", C.c_uint64), ("cap_seeds", C.c_uint64)] + \
               [(n, C.c_void_p) for n in ("nodes", "edge_src_local", "edge_dst_local", "seed_indices",
                                          "n_id", "edge_index_local", "seed_index")] + \
               [("x", C.c_void_p * AG_MAX_NODE_TYPES), ("cap_x", C.c_uint64 * AG_MAX_NODE_TYPES)]


class HeteroCounts(C.Structure):
    _fields_ = [("num_node_types", C.c_uint32), ("num_edge_types", C.c_uint32), ("num_seeds", C.c_uint32),
                ("error", C.c_uint32), ("nodes", C.c_uint32 * AG_MAX_NODE_TYPES),
                ("edges", C.c_uint32 * AG_MAX_EDGE_TYPES), ("total_nodes", C.c_uint32),
                ("total_edges", C.c_uint32), ("draws", C.c_uint64)]


class HeteroNames(C.Structure):
    _fields_ = [("num_node_types", C.c_uint32), ("num_edge_types", C.c_uint32),
                ("node_type", (C.c_char * 64) * AG_MAX_NODE_TYPES),
                ("src", (C.c_char * 64) * AG_MAX_EDGE_TYPES), ("rel", (C.c_char * 64) * AG_MAX_EDGE_TYPES),
                ("dst", (C.c_char * 64) * AG_MAX_EDGE_TYPES)]


class HeteroBatch(C.Structure):
    _fields_ = [("batch_idx", C.c_int64), ("seq", C.c_uint64), ("bufs", HeteroBuffers), ("counts", HeteroCounts)]


_P = C.c_void_p
_PP = C.POINTER(C.c_void_p)
_U64P = C.POINTER(C.c_uint64)
_I32P = C.POINTER(C.c_int32)

# name -> (restype, argtypes).  Every symbol include/aethergpu.h declares.
SIGNATURES = {
    "ag_last_error": (C.c_char_p, []),
    "ag_abi_version": (C.c_int32, []),
    "ag_batch_seed": (C.c_uint64, [C.c_uint64, C.c_uint64]),
    "ag_graph_load": (C.c_int32, [C.c_char_p, C.c_int32, C.c_int32, _PP]),
    "ag_graph_from_csr": (C.c_int32, [C.c_uint64, C.c_uint64, _P, _P, _P, C.c_int32, C.c_int32, _PP]),
    "ag_graph_adopt_device_csr": (C.c_int32, [C.c_uint64, C.c_uint64, _P, _P, _P, C.c_int32, _PP]),
    "ag_graph_from_edges": (C.c_int32, [C.c_uint64, _P, _P, _P, C.c_uint64, C.c_int32, _PP]),
    "ag_graph_save": (C.c_int32, [_P, C.c_char_p]),
    "ag_graph_save_compressed": (C.c_int32, [_P, C.c_char_p]),
    "ag_graph_rabbit_order": (C.c_int32, [_P, C.c_void_p, C.c_void_p]),
    "ag_graph_permute": (C.c_int32, [_P, C.c_void_p, C.c_uint64, _PP]),
    "ag_graph_info": (C.c_int32, [_P, _U64P, _U64P, _I32P, _I32P]),
    "ag_graph_device_ptrs": (C.c_int32, [_P, _PP, _PP, _PP]),
    "ag_graph_degrees": (C.c_int32, [_P, _P, C.c_uint64, _P]),
    "ag_graph_neighbors": (C.c_int32, [_P, C.c_uint32, _P, _P, C.c_uint64, _U64P]),
    "ag_graph_copy_to_host": (C.c_int32, [_P, _P, _P, _P]),
    "ag_features_copy_to_host": (C.c_int32, [_P, _P]),
    "ag_features_shard": (C.c_int32, [_P, _U64P, _U64P]),
    "ag_features_scales_to_host": (C.c_int32, [_P, _P]),
    "ag_features_gather_stats": (C.c_int32, [_P, _U64P, _U64P, _U64P]),
    "ag_features_set_gather_order": (C.c_int32, [_P, C.c_int32]),
    "ag_graph_hot_vertices": (C.c_int32, [_P, C.c_uint64, _PP, _U64P]),
    "ag_features_cache_rows": (C.c_int32, [_P, _P, C.c_uint64]),
    "ag_graph_free": (None, [_P]),
    "ag_features_save": (C.c_int32, [C.c_char_p, _P, C.c_uint64, C.c_uint64, C.c_int32]),
    "ag_features_load": (C.c_int32, [C.c_char_p, C.c_int32, _PP]),
    "ag_features_load_range": (C.c_int32, [C.c_char_p, C.c_int32, C.c_uint64, C.c_uint64, _PP]),
    "ag_features_from_memory": (C.c_int32, [_P, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32, _PP]),
    "ag_features_from_f32": (C.c_int32, [_P, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, C.c_int32, _PP]),
    "ag_features_adopt_device": (C.c_int32, [_P, C.c_uint64, C.c_uint64, C.c_int32, C.c_int32, _PP]),
    "ag_features_info": (C.c_int32, [_P, _U64P, _U64P, _I32P, _I32P, _U64P]),
    "ag_features_device_ptr": (C.c_int32, [_P, _PP]),
    "ag_features_get_batch": (C.c_int32, [_P, _P, C.c_uint64, _P]),
    "ag_gather": (C.c_int32, [_P, _P, C.c_int32, C.c_uint64, _P, _P, _P]),
    "ag_features_check": (C.c_int32, [_P]),
    "ag_features_load_shard": (C.c_int32, [C.c_char_p, C.c_int32, C.c_uint32, C.c_uint32, C.c_int32, _PP]),
    "ag_synth_features_shard": (C.c_int32, [C.c_uint64, C.c_uint64, C.c_int32, C.c_uint64, C.c_int32, C.c_uint32,
                                            C.c_uint32, C.c_int32, _PP]),
    "ag_features_ipc_export": (C.c_int32, [_P, _P]),
    "ag_features_open_sharded": (C.c_int32, [_P, C.c_uint32, C.c_uint32, _P, _PP]),
    "ag_features_view_sharded": (C.c_int32, [_P, C.c_uint32, C.c_uint32, _PP]),
    "ag_features_free": (None, [_P]),
    "ag_sampler_create": (C.c_int32, [_P, C.POINTER(SamplingConfigC), _PP]),
    "ag_sampler_reseed": (C.c_int32, [_P, C.c_uint64]),
    "ag_sampler_bounds": (C.c_int32, [_P, C.c_uint64, _U64P, _U64P]),
    "ag_sample_into": (C.c_int32, [_P, _P, C.c_uint64, C.c_int32, _P, C.POINTER(SubgraphBuffers), _P]),
    "ag_sample_wait": (C.c_int32, [_P, C.POINTER(SampleCounts)]),
    "ag_sample": (C.c_int32, [_P, _P, C.c_uint64, _P, C.c_int32, C.POINTER(SubgraphBuffers), _P]),
    "ag_subgraph_release": (C.c_int32, [_P, C.POINTER(SubgraphBuffers)]),
    "ag_sampler_free": (None, [_P]),
    "ag_sampler_set_profiling": (C.c_int32, [_P, C.c_int32]),
    "ag_sample_hop_reservoir": (C.c_int32, [_P, _P, C.c_uint64, C.c_uint32, C.c_uint64, C.c_uint32, _P, _P, _P]),
    "ag_register_seeds_static_max": (C.c_uint32, []),
    "ag_register_seeds_static": (C.c_int32, [C.c_int32, _P, C.c_uint32, C.c_uint64, _P, _P, _P, _P]),
    "ag_sampler_create_group": (C.c_int32, [_P, C.POINTER(SamplingConfigC), C.c_uint32, _PP]),
    "ag_sample_group_into": (C.c_int32, [_P, C.c_uint32, _P, _P, C.c_int32, _P, _P, C.POINTER(SubgraphBuffers), _P]),
    "ag_sample_group_wait": (C.c_int32, [_P, C.POINTER(SampleCounts), _I32P]),
    "ag_hetero_create": (C.c_int32, [C.c_uint32, _P, C.c_uint32, _P, _P, _P, _P, _P, _P, C.c_int32, C.c_int32, _PP]),
    "ag_hetero_info": (C.c_int32, [_P, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), _P, _P, _I32P]),
    "ag_hetero_in_adjacency": (C.c_int32, [_P, C.c_uint32, _P, _P]),
    "ag_hetero_free": (None, [_P]),
    "ag_hetero_sampler_create": (C.c_int32, [_P, _P, C.c_uint32, C.c_int32, C.c_uint64, C.c_int32, _PP]),
    "ag_hetero_sampler_create_group": (C.c_int32, [_P, _P, C.c_uint32, C.c_int32, C.c_uint64, C.c_int32, C.c_uint32, _PP]),
    "ag_hetero_sample_group_into": (C.c_int32, [_P, C.c_uint32, C.c_uint32, _P, _P, _P, _P, _P, _P]),
    "ag_hetero_sample_group_wait": (C.c_int32, [_P, _P, _I32P]),
    "ag_hetero_sampler_reseed": (C.c_int32, [_P, C.c_uint64]),
    "ag_hetero_sampler_bounds": (C.c_int32, [_P, C.c_uint64, _U64P, _U64P]),
    "ag_hetero_sample_into": (C.c_int32, [_P, C.c_uint32, _P, C.c_uint64, C.POINTER(HeteroBuffers), _P]),
    "ag_hetero_sample_wait": (C.c_int32, [_P, C.POINTER(HeteroCounts)]),
    "ag_hetero_sampler_free": (None, [_P]),
    "ag_loader_create": (C.c_int32, [_P, _P, C.POINTER(SamplingConfigC), C.c_int32, C.c_uint32, C.c_uint32,
                                     C.c_uint32, C.c_int32, _PP]),
    "ag_hetero_load": (C.c_int32, [C.c_char_p, C.c_int32, _PP, C.POINTER(HeteroNames)]),
    "ag_hetero_save": (C.c_int32, [_P, C.POINTER(HeteroNames), C.c_char_p]),
    "ag_loader_set_seed_sequence": (C.c_int32, [_P, C.c_uint64, C.c_uint64]),
    "ag_loader_bounds": (C.c_int32, [_P, C.c_uint64, _U64P, _U64P]),
    "ag_loader_submit": (C.c_int32, [_P, C.c_int64, _P, C.c_uint64, C.c_int32, C.POINTER(SubgraphBuffers), _P]),
    "ag_loader_next": (C.c_int32, [_P, C.c_int64, C.POINTER(Batch)]),
    "ag_loader_try_next": (C.c_int32, [_P, C.POINTER(Batch)]),
    "ag_loader_release_batch": (C.c_int32, [_P, C.POINTER(Batch), _P]),
    "ag_loader_submit_many": (C.c_int32, [_P, C.c_uint32, _P, _P, _P, C.c_int32, _P, _P, C.POINTER(C.c_uint32)]),
    "ag_loader_next_many": (C.c_int32, [_P, C.c_int64, C.c_uint32, C.POINTER(Batch), C.POINTER(C.c_uint32)]),
    "ag_loader_stats_get": (C.c_int32, [_P, C.POINTER(LoaderStats)]),
    "ag_loader_shutdown": (C.c_int32, [_P]),
    "ag_loader_free": (None, [_P]),
    "ag_subgraph_mirror": (C.c_int32, [C.c_int32, C.c_uint64, C.c_uint64, _P, _P, _P, _P, _P, _P, _U64P, _P]),
    "ag_subgraph_induce_plan": (C.c_int32, [_P, _P, C.c_uint64, _P, _PP, _U64P]),
    "ag_subgraph_induce_fill": (C.c_int32, [_P, C.c_uint64, _P, _P, _P, _P, _P, _P, _P]),
    "ag_subgraph_induce_free": (None, [_P]),
    "ag_hetero_loader_create": (C.c_int32, [_P, C.c_uint32, _P, C.c_uint32, C.c_int32, C.c_uint64, C.c_int32, C.c_int32,
                                            _P, C.c_uint32, C.c_uint32, C.c_uint32, _PP]),
    "ag_hetero_loader_submit": (C.c_int32, [_P, C.c_int64, _P, C.c_uint64]),
    "ag_hetero_loader_next": (C.c_int32, [_P, C.c_int64, C.POINTER(HeteroBatch)]),
    "ag_hetero_loader_next_many": (C.c_int32, [_P, C.c_int64, C.c_uint32, C.POINTER(HeteroBatch), C.POINTER(C.c_uint32)]),
    "ag_hetero_loader_release_batch": (C.c_int32, [_P, C.POINTER(HeteroBatch), _P]),
    "ag_hetero_loader_stats_get": (C.c_int32, [_P, C.POINTER(LoaderStats)]),
    "ag_hetero_loader_shutdown": (C.c_int32, [_P]),
    "ag_hetero_loader_free": (None, [_P]),
    "ag_synth_rmat_graph": (C.c_int32, [C.c_uint64, C.c_uint64, C.c_float, C.c_float, C.c_float, C.c_uint64,
                                        C.c_float, C.c_int32, _PP]),
    "ag_synth_rmat_csr": (C.c_int32, [C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_float, C.c_float,
                                      C.c_uint64, C.c_float, C.c_int32, _PP, _PP, _PP]),
    "ag_synth_fixed_degree_csr": (C.c_int32, [C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint64, C.c_int32, _PP, _PP]),
    "ag_synth_free_device": (C.c_int32, [_P, C.c_int32]),
    "ag_synth_features": (C.c_int32, [C.c_uint64, C.c_uint64, C.c_int32, C.c_uint64, C.c_int32, C.c_uint64,
                                      C.c_uint64, _PP]),
}

_lib = None


def lib():
    """The loaded library.  Raises if it was never built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m aethergraph_b200.build`. "
                "aethergraph_b200 has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the .so lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def last_error() -> str:
    return lib().ag_last_error().decode(errors="replace")


def check(status: int) -> None:
    """Raise the exception class the reference raises for this status."""
    if status == AG_OK:
        return
    msg = last_error()
    if status == AG_ERR_VALUE:
        raise ValueError(msg)
    if status == AG_ERR_LOAD:
        raise GraphLoadError(msg)
    if status == AG_ERR_SAMPLING:
        raise SamplingError(msg)
    if status == AG_ERR_TIMEOUT:
        raise TimeoutError(msg)
    raise RuntimeError(msg)

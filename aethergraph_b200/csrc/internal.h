// Internal declarations shared by the translation units of libaethergpu.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <vector>

#include "../../include/aethergpu.h"

namespace ag {
// Device scratch of the address-ordered gather: two key and two value arrays for
// the radix sort and its temporary storage.  Grows, never shrinks.
struct SortScratch {
    uint32_t *keys[2] = {nullptr, nullptr};
    uint32_t *vals[2] = {nullptr, nullptr};
    void *temp = nullptr;
    uint32_t *counts = nullptr;  // [0]: keys of local rows in the list being sorted
    size_t temp_bytes = 0;
    uint64_t cap = 0;  // items the arrays hold
    cudaError_t ensure(uint64_t items);
    void release();
};
}  // namespace ag

struct ag_graph {
    int device = 0;
    uint64_t num_nodes = 0, num_edges = 0;
    uint64_t *offsets = nullptr;  // device, num_nodes + 1
    uint32_t *dst = nullptr;      // device, num_edges
    float *weights = nullptr;     // device, num_edges or null
};

namespace ag {
// Device memory that peers map with 2 MB pages (peer_block.cu).
struct PeerBlock;
int32_t peer_block_alloc(int device, size_t bytes, PeerBlock **out);
int32_t alloc_feature_payload(int device, size_t bytes, uint8_t **ptr, PeerBlock **block);  // a block, or cudaMalloc when asked
void peer_block_free(PeerBlock *b);
void *peer_block_ptr(const PeerBlock *b);
int32_t peer_block_grant(PeerBlock *b, int reader_device);            // same process, another GPU
int32_t peer_block_export(PeerBlock *b, void *handle_out);            // AG_IPC_HANDLE_BYTES
int32_t peer_block_import(const void *handle, int device, PeerBlock **out);
int peer_handle_kind(const void *handle);                             // 0 empty, 1 legacy CUDA IPC, 2 shareable block
void peer_handle_mark_legacy(void *handle);
}  // namespace ag

struct ag_features {
    int device = 0;
    uint64_t num_nodes = 0;   // rows of the whole store
    uint64_t row_begin = 0;   // first row held here (vertex-range shard)
    uint64_t rows = 0;        // rows held here
    uint64_t row_stride = 1;  // held row i is row row_begin + i * row_stride (cyclic shard: stride = world)
    uint64_t dim = 0;
    int dtype = AG_F32;
    uint8_t *payload = nullptr;  // device, rows * dim * elem_size
    float *scales = nullptr;     // device, AG_I8 only: rows * ceil(dim / 32) per-block scales
    uint32_t *err = nullptr;     // device, 32 bytes: sticky error bits; at +8 / +16 two u64 counters of the
                                 // address-ordered gather (rows asked for, rows actually loaded)
    bool owns_payload = true;
    // A sharded view (ag_features_open_sharded / ag_features_view_sharded): rows
    // [r * shard_rows, (r + 1) * shard_rows) live in shard r's memory, this GPU's
    // own shard or a peer's mapped into this process.
    struct ag_shard_table *shards = nullptr;  // device copy of the table, or null
    uint32_t n_shards = 0;
    uint64_t shard_rows = 0;                  // rows per shard (the last may hold fewer)
    bool shard_cyclic = false;                // rows dealt round-robin instead of contiguous ranges
    // Hot rows replicated on this GPU (ag_features_cache_rows): requests for them never cross NVLink.
    uint8_t *hot_rows = nullptr;              // device, hot_n * row bytes
    uint32_t *hot_slot = nullptr;             // device, num_nodes entries
    uint64_t hot_n = 0;
    void *ipc_opened[8] = {nullptr};          // legacy CUDA IPC mappings this view opened (closed on free)
    struct ag::PeerBlock *peer_opened[8] = {nullptr};  // peers' shareable blocks this view mapped (unmapped on free)
    struct ag::PeerBlock *block = nullptr;    // the payload's own shareable block (null: a plain device allocation)
    bool legacy_peer = false;                 // some peer is mapped through a legacy CUDA IPC handle (small pages)
    int gather_order = 0;                     // AG_GATHER_AUTO / _ORDERED / _DIRECT (ag_features_set_gather_order)
    // ag_gather on a sharded view sorts its ids into address order first; the scratch
    // belongs to the view, calls take turns (mutex on the host, event on the device).
    struct SortState {
        std::mutex m;
        ag::SortScratch scratch;
        cudaEvent_t done = nullptr;
        bool used = false;
    } *sort = nullptr;
};

// Heterogeneous graph: per edge type only the transposed adjacency lives on the
// device (for each destination, its sources ascending).
struct ag_hetero_graph {
    int device = 0;
    uint32_t nt = 0, et = 0;
    uint64_t num_nodes[AG_MAX_NODE_TYPES] = {0};
    uint32_t src_type[AG_MAX_EDGE_TYPES] = {0}, dst_type[AG_MAX_EDGE_TYPES] = {0};
    uint64_t num_edges[AG_MAX_EDGE_TYPES] = {0};
    uint64_t *in_offsets[AG_MAX_EDGE_TYPES] = {nullptr};
    uint32_t *in_sources[AG_MAX_EDGE_TYPES] = {nullptr};
};

// Device-visible table of a sharded feature store.
struct ag_shard_table {
    const uint8_t *base[9];   // shard r's rows; base[n_shards]: this GPU's copy of the hot rows, if any
    uint64_t shard_rows;      // range layout: rows per shard
    uint32_t n_shards;
    uint32_t cyclic;          // 1: row v lives in shard v % n_shards at local row v / n_shards
    uint32_t n_sources;       // n_shards, or n_shards + 1 with a hot-row copy
    uint32_t self;            // the shard that lives in this GPU's own memory
    const uint32_t *hot_slot; // per vertex: its row in the hot-row copy, or 0xFFFFFFFF (null: no copy)
};

namespace ag {

inline uint32_t elem_size(int dtype) { return dtype == AG_F32 ? 4u : dtype == AG_I8 ? 1u : 2u; }
constexpr uint32_t kQuantBlock = 32;  // elements per scale of the int8 payload (feature_codec.rs: BlockScaledI8::BLOCK)

struct GatherArgs {
    const uint8_t *payload;
    uint64_t row_begin, rows;
    uint32_t row_bytes, dim;
    const void *ids;
    int ids64;
    uint64_t n;
    const uint32_t *n_dev;
    float *out;
    uint32_t *err;
    const ag_shard_table *shards;  // non-null: rows are looked up through the shard table
    const uint32_t *ids_off;       // non-null (u32 ids only): the ids start at ids + *ids_off (device value)
    const float *scales;           // AG_I8 stores: per-block scales
};

// The source half of a gather's arguments, from a feature store handle.
inline void set_gather_source(GatherArgs &a, const ag_features *f) {
    a.payload = f->payload; a.row_begin = f->row_begin; a.rows = f->rows;
    a.row_bytes = (uint32_t)(f->dim * elem_size(f->dtype)); a.dim = (uint32_t)f->dim;
    a.err = f->err; a.shards = f->shards; a.scales = f->scales;
}

cudaError_t launch_gather(const GatherArgs &a, int dtype, cudaStream_t st);
cudaError_t launch_gather_group(const GatherArgs *group_dev, uint32_t n_batches, uint32_t row_bytes,
                                uint32_t dim, uint64_t n_bound, bool aligned, int dtype, bool sharded,
                                cudaStream_t st);
// Address-ordered gather over a sharded view (see gather.cu).
bool sorted_gather_applies(const ag_features *f, uint32_t row_bytes, bool aligned);
cudaError_t launch_sort_keys(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                             const ag_features *f, SortScratch &sc, cudaStream_t st);
cudaError_t launch_sorted_fetch(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                                uint32_t row_bytes, uint32_t dim, int dtype, const ag_features *f, SortScratch &sc,
                                cudaStream_t st_local, cudaStream_t st_remote);
cudaError_t launch_gather_sorted(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                                 uint32_t row_bytes, uint32_t dim, int dtype, const ag_features *f, SortScratch &sc,
                                 cudaStream_t st);
cudaError_t launch_encode(const float *src, void *dst, uint64_t count, int dtype, cudaStream_t st);
// f32 rows -> block-scaled int8 codes + scales; *bad_dev is set when a value is not finite.
cudaError_t launch_encode_i8(const float *src, uint64_t rows, uint64_t dim, int8_t *codes, float *scales, uint32_t *bad_dev,
                             cudaStream_t st);
int gather_grid_blocks(uint64_t n, uint32_t row_bytes);
int32_t sampler_set_yielding_wait(ag_sampler *s, bool on);  // poll + yield instead of spinning in ag_sample_group_wait

// Device-side validation of a CSR: offsets monotone, offsets[n] == e, dst < n.
// Writes a non-zero code to *flag_dev on failure.
cudaError_t launch_validate_csr(const uint64_t *offsets, const uint32_t *dst, uint64_t n,
                                uint64_t e, uint64_t dst_bound, uint32_t *flag_dev,
                                cudaStream_t st);
cudaError_t launch_degrees(const uint64_t *offsets, uint64_t num_nodes, const uint32_t *ids,
                           uint64_t n, uint32_t *out, cudaStream_t st);

// Sorts n keys (row << 32 | value) and builds the CSR over num_rows rows from them
// (rows ascending, values ascending within a row).  Consumes (frees) keys.
int32_t keys_to_sorted_csr(uint64_t *keys, uint64_t n, uint64_t num_rows, uint64_t **offsets_out,
                           uint32_t **vals_out);

}  // namespace ag

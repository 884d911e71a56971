/*
 * aethergpu.h — C ABI of the B200 minibatch path.
 *
 * One shared library (libaethergpu.so) implements, on the GPU, the path the
 * reference runs on the CPU: k-hop neighbor sampling over a static CSR graph,
 * frontier dedup + relabel into a local edge index, and the feature-row
 * gather with fused f16/bf16 -> f32 upcast.  The reference exposes this path
 * through its PyO3 extension module `aethergraph._core`
 * (python/aethergraph/_core.pyi is the contract); it has no C ABI of its own.
 * Each entry point below names the reference interface it stands in for
 * (file:line relative to the reference project root).
 *
 * Conventions
 *   - Every function returns an ag_status (0 = OK).  On failure a
 *     thread-local, NUL-terminated message is available from ag_last_error().
 *     Status classes map onto the reference's Python exceptions
 *     (crates/aethergraph-py/src/error.rs:29-70, prefetch.rs:35-55):
 *       AG_ERR_VALUE -> ValueError,  AG_ERR_LOAD -> GraphLoadError,
 *       AG_ERR_SAMPLING -> SamplingError,  AG_ERR_TIMEOUT -> TimeoutError,
 *       AG_ERR_WORKER -> RuntimeError,  AG_ERR_CUDA -> RuntimeError.
 *   - Host input arrays are borrowed for the duration of the call only.
 *   - Pointers named *_dev are device pointers on the handle's device.
 *   - `stream` is a cudaStream_t passed as void* (NULL = default stream).
 *   - There is no CPU fallback: every compute entry point launches CUDA
 *     kernels and fails with AG_ERR_CUDA when no device is usable.
 *   - Handles may be used from any thread; a sampler handle is not
 *     re-entrant (the reference's samplers are `&mut self`, one per worker:
 *     crates/aethergraph-core/src/loader/prefetch.rs:918,959).
 */
#ifndef AETHERGPU_H
#define AETHERGPU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    AG_OK = 0,
    AG_ERR_VALUE = 1,
    AG_ERR_LOAD = 2,
    AG_ERR_SAMPLING = 3,
    AG_ERR_TIMEOUT = 4,
    AG_ERR_WORKER = 5,
    AG_ERR_CUDA = 6,
    AG_ERR_SHUTDOWN = 7
} ag_status;

typedef struct ag_graph ag_graph;
typedef struct ag_features ag_features;
typedef struct ag_sampler ag_sampler;
typedef struct ag_hetero_graph ag_hetero_graph;
typedef struct ag_hetero_sampler ag_hetero_sampler;
typedef struct ag_loader ag_loader;

const char *ag_last_error(void);
/* ABI version of this header; bumped on any incompatible change. */
int32_t ag_abi_version(void);

/* ------------------------------------------------------------------ RNG --
 * crates/aethergraph-core/src/loader/sampler.rs:69-75 (batch_seed). */
uint64_t ag_batch_seed(uint64_t base, uint64_t batch_idx);

/* ---------------------------------------------------------------- graph --
 * Stands in for CsrGraph.load / CsrGraph.from_edges / CsrGraph.save and the
 * row accessors (_core.pyi:68-131; crates/aethergraph-py/src/graph.rs:51-88;
 * file format crates/aethergraph-core/src/internal/mmap.rs:114-121).
 * The CSR (u64 offsets, u32 destinations, optional f32 weights) lives in HBM.
 */
enum { AG_VALIDATE_AUTO = 0, AG_VALIDATE_HEADER = 1, AG_VALIDATE_OFFSETS = 2, AG_VALIDATE_FULL = 3 };
enum { AG_MEM_HOST = 0, AG_MEM_DEVICE = 1 };

int32_t ag_graph_load(const char *path, int32_t validation, int32_t device, ag_graph **out);
/* Copies a CSR from host or device memory (mem_kind) into library-owned HBM.
 * Offsets must be non-decreasing with offsets[n] == num_edges, and every
 * destination < num_nodes (checked on the device; AG_ERR_LOAD otherwise). */
int32_t ag_graph_from_csr(uint64_t num_nodes, uint64_t num_edges, const uint64_t *offsets,
                          const uint32_t *dst, const float *weights, int32_t mem_kind,
                          int32_t device, ag_graph **out);
/* Takes ownership of device arrays produced by this library's generators or
 * allocated with cudaMalloc on `device`; validates like ag_graph_from_csr. */
int32_t ag_graph_adopt_device_csr(uint64_t num_nodes, uint64_t num_edges, uint64_t *offsets_dev,
                                  uint32_t *dst_dev, float *weights_dev, int32_t device,
                                  ag_graph **out);
/* Counting-sort CSR build that keeps input order within each row
 * (crates/aethergraph-core/src/graph/csr.rs:568-571, 631-750). */
int32_t ag_graph_from_edges(uint64_t num_nodes, const uint32_t *src, const uint32_t *dst,
                            const float *weights, uint64_t num_edges, int32_t device,
                            ag_graph **out);
int32_t ag_graph_save(const ag_graph *g, const char *path);
/* The version-2 file: the same 32-byte header with version = 2, the offsets as
 * Elias-Fano and the edge array as StreamVByte wrapping deltas, weights raw, checksum
 * over the payload (crates/aethergraph-core/src/internal/compressed_graph.rs:39-88;
 * codecs and wire formats internal/succinct.rs:52-92,198-214,397-420,486-500).
 * ag_graph_load recognises the version, decodes both sections on the GPU and always
 * verifies the checksum and the whole CSR (compressed_graph.rs:99-175). */
int32_t ag_graph_save_compressed(const ag_graph *g, const char *path);
/* Locality reordering (crates/aethergraph-core/src/graph/reorder.rs:142-383;
 * Graph.reorder_rabbit / rabbit_partitions / permute, python/aethergraph/_core.pyi:121-130).
 * ag_graph_rabbit_order: Rabbit Order community detection — vertices in ascending
 * (undirected degree, id) order, each merged into the neighbouring community of largest
 * positive modularity gain (exact integers, ties to the smaller id) — sequential and
 * deterministic as in the reference, run on the host over a copy of the CSR.
 * perm_out[new_id] = old_id (pre-order walk of the dendrogram) and partitions_out[v] =
 * dense id of v's top-level community, numbered by first vertex; either may be NULL;
 * both are host arrays of num_nodes entries.
 * ag_graph_permute: the relabelled graph, built on the GPU; row new_id holds the edges
 * of row perm[new_id] in their order, endpoints relabelled, weights carried along.
 * AG_ERR_VALUE for a permutation of the wrong length, with an out-of-range or a
 * duplicate entry. */
int32_t ag_graph_rabbit_order(const ag_graph *g, uint32_t *perm_out, uint32_t *partitions_out);
int32_t ag_graph_permute(const ag_graph *g, const uint32_t *perm, uint64_t perm_len, ag_graph **out);
int32_t ag_graph_info(const ag_graph *g, uint64_t *num_nodes, uint64_t *num_edges,
                      int32_t *has_weights, int32_t *device);
int32_t ag_graph_device_ptrs(const ag_graph *g, const uint64_t **offsets_dev,
                             const uint32_t **dst_dev, const float **weights_dev);
/* degrees_of (out-of-range id -> 0); ids == NULL means all nodes in order. */
int32_t ag_graph_degrees(const ag_graph *g, const uint32_t *ids, uint64_t n, uint32_t *out);
/* neighbors(node): copies up to cap destinations (and weights when
 * weights_out != NULL) to host; *degree receives the full row length. */
int32_t ag_graph_neighbors(const ag_graph *g, uint32_t node, uint32_t *out, float *weights_out,
                           uint64_t cap, uint64_t *degree);
/* Copies the CSR back to host arrays sized num_nodes + 1 / num_edges (any may be NULL). */
int32_t ag_graph_copy_to_host(const ag_graph *g, uint64_t *offsets, uint32_t *dst, float *weights);
void ag_graph_free(ag_graph *g);

/* ------------------------------------------------------------- features --
 * Stands in for save_features / FeatureStore (_core.pyi:136-148, 482-516;
 * crates/aethergraph-core/src/features/store.rs:384-440, 691-838;
 * header crates/aethergraph-core/src/features/header.rs:165-244).
 * The payload (num_nodes x dim elements of f32 / f16 / bf16) lives in HBM.
 */
enum { AG_F32 = 0, AG_F16 = 1, AG_BF16 = 2,
       /* Block-scaled int8 (crates/aethergraph-core/src/internal/feature_codec.rs:1-60): one
        * signed byte per element, row-major, plus one f32 scale per 32 elements of a row;
        * scale = max|x| / 127 over the block, code = round(x / scale) clamped to +-127,
        * decode = code * scale (one IEEE multiply: the gather's rows are bit-identical to
        * the reference's BlockScaledI8::decode).  In-memory only (the reference defines no
        * file layout for it): ag_features_from_f32, ag_synth_features.  Not shardable. */
       AG_I8 = 3 };

int32_t ag_features_save(const char *path, const float *features, uint64_t num_nodes,
                         uint64_t dim, int32_t dtype);
int32_t ag_features_load(const char *path, int32_t device, ag_features **out);
/* Loads rows [row_begin, row_end) only (a vertex-range shard). */
int32_t ag_features_load_range(const char *path, int32_t device, uint64_t row_begin,
                               uint64_t row_end, ag_features **out);
/* payload holds stored elements (not f32 unless dtype == AG_F32). */
int32_t ag_features_from_memory(const void *payload, uint64_t num_nodes, uint64_t dim,
                                int32_t dtype, int32_t mem_kind, int32_t device,
                                ag_features **out);
/* Encodes f32 rows on the device into `dtype` (RNE for f16; the reference's
 * bf16 rule, store.rs:1094-1104) and keeps the encoded payload. */
int32_t ag_features_from_f32(const float *features, uint64_t num_nodes, uint64_t dim,
                             int32_t dtype, int32_t mem_kind, int32_t device, ag_features **out);
int32_t ag_features_adopt_device(void *payload_dev, uint64_t num_nodes, uint64_t dim,
                                 int32_t dtype, int32_t device, ag_features **out);
int32_t ag_features_info(const ag_features *f, uint64_t *num_nodes, uint64_t *dim,
                         int32_t *dtype, int32_t *device, uint64_t *row_begin);
/* The vertex range [row_begin, row_begin + rows) this handle holds. */
int32_t ag_features_shard(const ag_features *f, uint64_t *row_begin, uint64_t *rows);
int32_t ag_features_device_ptr(const ag_features *f, const void **payload_dev);

/* Vertex-range shards over the GPUs of one node (the partitioned-features
 * layout of python/aethergraph/ray/datasource.py:6-10; the reference fetches
 * remote rows through its RDMA gather, here a remote row is a plain load over
 * NVLink from the owner's HBM, upcast at the reader).  Shard r of `world` holds
 * rows [r * S, min((r + 1) * S, num_nodes)) with S = ceil(num_nodes / world)
 * (load it with ag_features_load_range or build it with ag_synth_features).
 * One process per GPU: every rank exports its shard's 64-byte IPC handle,
 * exchanges the handles by any means (the Python layer uses
 * torch.distributed.all_gather_object) and opens the view with all of them
 * (`handles` = world x 64 bytes, own entry ignored).  One process driving
 * several GPUs: ag_features_view_sharded over the shard handles themselves.
 * The view gathers any row in [0, num_nodes); it borrows the local shard,
 * which must outlive it, and is freed with ag_features_free.
 *
 * Layouts.  AG_SHARD_RANGE is the contiguous layout above (the reference's).
 * AG_SHARD_CYCLIC deals rows round-robin: shard r holds rows r, r + world, ...
 * and row v lives in shard v % world at local row v / world.  On skewed graphs
 * the hub vertices sit in the low id range, so under the range layout most
 * gathered rows come from shard 0 and that GPU's NVLink egress throttles every
 * reader; the cyclic layout spreads any id range evenly over the GPUs.  A
 * cyclic shard can only be read through a view. */
enum { AG_SHARD_RANGE = 0, AG_SHARD_CYCLIC = 1 };
int32_t ag_features_load_shard(const char *path, int32_t device, uint32_t rank, uint32_t world,
                               int32_t layout, ag_features **out);
/* ag_features_ipc_export writes the AG_IPC_HANDLE_BYTES another process needs to map
 * this shard; the ranks exchange them (all-gather over any transport) and hand
 * the table to ag_features_open_sharded.  A payload the library allocated (every
 * loader, ag_features_from_f32, the synthetic generators) is exported as a file
 * descriptor of a driver memory handle, served to the peers over an abstract unix
 * socket until the store is freed, and mapped there with 2 MB pages; a payload
 * adopted from the caller (ag_features_adopt_device) is exported as a legacy CUDA
 * IPC handle, whose mapping reads an order of magnitude slower at random once tens
 * of GB are mapped. */
#define AG_IPC_HANDLE_BYTES 128
int32_t ag_features_ipc_export(const ag_features *f, void *handle_out);
int32_t ag_features_open_sharded(const ag_features *local, uint32_t world, uint32_t rank,
                                 const void *handles, ag_features **out);
int32_t ag_features_view_sharded(const ag_features *const *shards, uint32_t world, uint32_t rank,
                                 ag_features **out);
/* A gather over a sharded view (ag_gather, or the chain of a sampler / loader)
 * requests its rows in address order: the ids of the launch are turned into
 * keys (row within shard, owner), sorted in local memory, and fetched in that
 * order, a row named more than once only once — the counterpart of the
 * reference's request coalescing in its one-sided remote gather
 * (crates/aether-stream/src/rdma/sharded.rs:1-33, rdma/gather.rs:1-9).  The
 * counters say how many rows such gathers were asked for, how many they loaded
 * (the rest were repeats within a launch) and how many of the loaded ones came
 * from the local copy of the hot rows, since the view was opened (or since
 * ag_features_cache_rows). */
int32_t ag_features_gather_stats(const ag_features *f, uint64_t *rows_requested,
                                 uint64_t *rows_fetched, uint64_t *rows_local_copy);
/* How a sharded view fetches.  AG_GATHER_DIRECT: every row is loaded from its owner
 * where the request stands, no sort, repeats loaded again (the counters then count
 * every requested row as loaded).  AG_GATHER_ORDERED: the address-ordered gather
 * above.  AG_GATHER_AUTO (the default): direct when every peer is mapped with large
 * pages (all payloads the library allocated), ordered when a peer came through a
 * legacy CUDA IPC handle.  Same bits either way. */
enum { AG_GATHER_AUTO = 0, AG_GATHER_ORDERED = 1, AG_GATHER_DIRECT = 2 };
int32_t ag_features_set_gather_order(ag_features *view, int32_t order);
/* Hot rows.  On a skewed graph a small share of the vertices receives most of the
 * row requests (a vertex is gathered in proportion to its in-degree).
 * ag_graph_hot_vertices returns the `max_rows` vertices of highest in-degree,
 * hottest first, as a device array (free it with ag_synth_free_device);
 * ag_features_cache_rows copies the stored rows of such a list into this GPU's
 * memory and lets the sharded view serve them locally, so only the cold rows
 * cross NVLink.  Same bits either way; nothing to keep coherent, the rows never
 * change.  Counterpart: the GPU-resident hot tier of the reference's feature
 * cache, which pins the hottest nodes when frequencies are known
 * (crates/aethergraph-core/src/features/cache/mod.rs:1-20), in front of its
 * remote gather (crates/aether-stream/src/rdma/sharded.rs:1-33).  No gather over
 * the view may run while ag_features_cache_rows does. */
int32_t ag_graph_hot_vertices(const ag_graph *g, uint64_t max_rows, uint32_t **ids_dev,
                              uint64_t *n_out);
int32_t ag_features_cache_rows(ag_features *view, const uint32_t *ids_dev, uint64_t n);
/* AG_I8 stores: the per-block scales (rows x ceil(dim / 32) f32) to host memory. */
int32_t ag_features_scales_to_host(const ag_features *f, float *scales);
/* Copies the stored (encoded) rows held by this handle back to host memory. */
int32_t ag_features_copy_to_host(const ag_features *f, void *payload);

/* FeatureStore.get_batch on host ids (store.rs:691-769): range-checks every
 * id first (AG_ERR_VALUE "node N out of bounds"), gathers on the device and
 * copies the [n, dim] f32 result to `out` (host).  Synchronous. */
int32_t ag_features_get_batch(const ag_features *f, const int64_t *ids, uint64_t n, float *out);

/* Device gather (store.rs:777-838 get_batch_into): out_dev[i, :] =
 * upcast(row ids[i]).  ids are u32 (ids_are_i64 == 0) or i64 device arrays.
 * The row count is `n`, or *n_dev (a device u32) clamped to n when n_dev is
 * not NULL.  An id outside the store writes a zero row and raises a sticky
 * error reported by ag_features_check. */
int32_t ag_gather(const ag_features *f, const void *ids_dev, int32_t ids_are_i64, uint64_t n,
                  const uint32_t *n_dev, float *out_dev, void *stream);
/* Returns AG_ERR_VALUE if any device gather since the last check saw an
 * out-of-range id (synchronises the device). */
int32_t ag_features_check(const ag_features *f);
void ag_features_free(ag_features *f);

/* -------------------------------------------------------------- sampler --
 * Stands in for SamplingConfig / NeighborSampler / ParallelBatchSampler
 * (_core.pyi:152-198, 263-288; crates/aethergraph-core/src/loader/sampler.rs:
 * 78-158 config, 525-557 sample, 845-961 sample_neighbors_inner).
 */
enum { AG_RNG_WYRAND_EXACT = 0, AG_RNG_PHILOX = 1 };
#define AG_MAX_HOPS 8

typedef struct {
    uint32_t num_hops;
    uint32_t fanout[AG_MAX_HOPS];
    int32_t replace;        /* sampler.rs:85 */
    int32_t weighted;       /* sampler.rs:112; needs graph weights */
    int32_t track_edge_ids; /* sampler.rs:120 */
    uint64_t seed;          /* sampler.rs:88 (the caller resolves None) */
    /* AG_RNG_WYRAND_EXACT replays the reference's sequential WyRand stream
     * (internal/genstamp.rs:181-202) draw for draw.  AG_RNG_PHILOX keys every
     * draw on (seed, hop, vertex, slot) with Philox4x32-10
     * (internal/philox.rs:15-52): same distribution, different samples. */
    int32_t rng_mode;
    uint32_t max_seeds;     /* sizing hint for scratch; grows on demand */
} ag_sampling_config;

/* Output buffers of one sampled batch, all device memory.  Arrays marked
 * "optional" may be NULL in a caller-supplied struct and are then skipped.
 * Layout follows SampledSubgraph (sampler.rs:1512-1543) and the Python view
 * (crates/aethergraph-py/src/sampler.rs:329-370): edge_index_local is
 * [2, num_edges] row-major int64, row 0 = sampled neighbor (dst_local),
 * row 1 = expanded node (src_local). */
typedef struct {
    uint64_t cap_nodes, cap_edges, cap_seeds; /* capacities of the arrays below */
    uint32_t *nodes;        /* [cap_nodes] global ids in discovery order */
    uint32_t *edge_src;     /* [cap_edges] expanded node                (optional) */
    uint32_t *edge_dst;     /* [cap_edges] sampled neighbor */
    uint64_t *edge_ids;     /* [cap_edges] CSR position                 (optional) */
    uint32_t *src_local;    /* [cap_edges] */
    uint32_t *dst_local;    /* [cap_edges] */
    uint32_t *seed_locals;  /* [cap_seeds] */
    int64_t *n_id;          /* [cap_nodes] int64(nodes)                 (optional) */
    int64_t *edge_index_local; /* [2 * num_edges] packed at the final count (optional) */
    int64_t *e_id;          /* [cap_edges] int64(edge_ids)              (optional) */
    int64_t *seed_index;    /* [cap_seeds] int64(seed_locals)           (optional) */
    float *x;               /* [cap_x or cap_nodes, dim] gathered rows  (optional) */
    uint64_t cap_x;         /* rows x holds; 0 = cap_nodes.  A batch with more nodes gets its first
                             * cap_x rows only (compare ag_sample_counts.num_nodes): the worst-case
                             * node bound is many times a typical batch, so a caller may reserve x
                             * from observed counts and gather the rare overflow again (ag_gather). */
} ag_subgraph_buffers;

typedef struct {
    uint32_t num_nodes, num_edges, num_seeds, num_hops;
    uint32_t nodes_per_hop[AG_MAX_HOPS + 1]; /* [distinct seeds, new@hop1, ...] sampler.rs:876-883 */
    uint32_t edges_per_hop[AG_MAX_HOPS];
    uint64_t draws;          /* RNG draws consumed by this batch */
    uint32_t error;          /* device-side error bits, 0 = none */
    uint32_t reserved;
    /* Device time of the sampling kernels and of the gather kernel for this
     * batch, in milliseconds; filled only after ag_sampler_set_profiling(s, 1). */
    float sample_ms, gather_ms;
    /* When the gather of this batch's launch chain began and ended on the device, in
     * milliseconds since the library's first profiled launch on that GPU (all batches
     * of a chain carry the same pair).  Chains of different handles overlap; the union
     * of these intervals is the time some gather kernel was running. */
    double gather_begin_ms, gather_end_ms;
} ag_sample_counts;

int32_t ag_sampler_create(const ag_graph *g, const ag_sampling_config *cfg, ag_sampler **out);
/* NeighborSampler::reseed (sampler.rs:509-511): restarts the stream at draw 0. */
int32_t ag_sampler_reseed(ag_sampler *s, uint64_t seed);
/* Upper bounds on nodes / edges for a batch of n_seeds (for sizing buffers). */
int32_t ag_sampler_bounds(const ag_sampler *s, uint64_t n_seeds, uint64_t *max_nodes,
                          uint64_t *max_edges);
/* Enqueues one batch on `stream`.  seeds: host array (range-checked here like
 * Seeds::new, sampler.rs:230-239 -> AG_ERR_SAMPLING) when seeds_mem ==
 * AG_MEM_HOST, else a device array (checked on the device, reported through
 * counts.error).  When `feats` is not NULL and buf->x is set, the gather of
 * the batch's nodes is enqueued right behind the sampler.  Returns as soon as
 * the work is queued; ag_sample_wait blocks until it is done and returns the
 * counts.  A bare sampler keeps consuming one RNG stream across calls
 * (crates/aethergraph-py/src/sampler.rs:782-785). */
int32_t ag_sample_into(ag_sampler *s, const uint32_t *seeds, uint64_t n_seeds, int32_t seeds_mem,
                       const ag_features *feats, ag_subgraph_buffers *buf, void *stream);
int32_t ag_sample_wait(ag_sampler *s, ag_sample_counts *counts);
/* Library-allocated variant: fills *buf with buffers sized by
 * ag_sampler_bounds; release them with ag_subgraph_release. */
int32_t ag_sample(ag_sampler *s, const uint32_t *seeds, uint64_t n_seeds,
                  const ag_features *feats, int32_t want_int64, ag_subgraph_buffers *buf,
                  void *stream);
int32_t ag_subgraph_release(ag_sampler *s, ag_subgraph_buffers *buf);

/* Groups.  Batches are independent, so one launch chain can serve several of
 * them: every kernel's grid gets the batch as a second dimension and a group
 * of 16 batches costs the same dozen launches as one.  This is the device form
 * of ParallelBatchSampler::sample_batches (sampler.rs:1726-1751): with
 * batch_seeds[b] = ag_batch_seed(seed, position of batch b) it reproduces it
 * bit for bit.  A sampler created with ag_sampler_create_group(.., group, ..)
 * holds scratch for `group` batches; n_batches may be anything up to that.
 * seeds[b] / n_seeds[b] / bufs[b] describe batch b; batch_seeds == NULL lets
 * the handle's own RNG stream continue (single batch only makes sense).
 * ag_sample_group_wait fills counts[b] and statuses[b] (either may be NULL)
 * and returns the first failing status. */
int32_t ag_sampler_create_group(const ag_graph *g, const ag_sampling_config *cfg, uint32_t group,
                                ag_sampler **out);
int32_t ag_sample_group_into(ag_sampler *s, uint32_t n_batches, const uint32_t *const *seeds,
                             const uint64_t *n_seeds, int32_t seeds_mem,
                             const uint64_t *batch_seeds, const ag_features *feats,
                             ag_subgraph_buffers *bufs, void *stream);
int32_t ag_sample_group_wait(ag_sampler *s, ag_sample_counts *counts, int32_t *statuses);
/* When on, every batch records CUDA events around its sampling chain and its
 * gather on the launching stream (ag_sample_counts.sample_ms / gather_ms). */
int32_t ag_sampler_set_profiling(ag_sampler *s, int32_t on);
void ag_sampler_free(ag_sampler *s);

/* ------------------------------------------- fast mode: one-hop reservoir --
 * Stands in for the reference's Philox fast-mode sampler, bit for bit: CPU
 * `reservoir_sample` (crates/aethergraph-core/src/internal/philox.rs:59-82) and
 * its GPU kernel `warp_sample_neighbors`
 * (crates/aether-stream/src/gpu/kernels/sampler/sampler.cu, launched by
 * sampler/mod.rs:180-230).  For each of node_count nodes (u64 ids, device
 * array; an id outside the graph gives an empty row) writes `fanout` slots to
 * neighbors_out_dev[row * fanout ..] and the number of real ones to
 * counts_out_dev[row]; unused slots hold AG_SAMPLE_PAD.  fanout >= degree
 * copies the row; fanout <= 32 runs Algorithm R keyed on (seed, layer, node, t);
 * fanout > 32 draws with replacement, slot d = row[philox(d) % degree]. */
#define AG_SAMPLE_PAD 0xffffffffu
int32_t ag_sample_hop_reservoir(const ag_graph *g, const uint64_t *nodes_dev, uint64_t node_count,
                                uint32_t fanout, uint64_t seed, uint32_t layer,
                                uint32_t *neighbors_out_dev, uint32_t *counts_out_dev, void *stream);

/* ------------------------------------------------ allocation-free entry --
 * No counterpart in the reference.  For callers that must not allocate device
 * memory while they run (a memory-pool or stream callback, a process whose
 * device memory is fully budgeted to another allocator, a loop that cannot
 * afford the device-wide synchronisation of cudaMalloc / cudaFree): the first
 * step of the sampling path, seed registration, with its scratch in a fixed
 * 160 KiB `static __device__` array inside the library instead of an
 * allocation.  Collapses duplicate seeds in first-sighting order into
 * nodes_out_dev and writes each input seed's local index to
 * seed_locals_out_dev; count_err_out_dev[0] receives the distinct count,
 * count_err_out_dev[1] error bits (8 = a seed >= num_nodes).  All buffers are
 * the caller's device memory (capacity n_seeds each).  At most
 * ag_register_seeds_static_max() (8192) seeds per call; more is AG_ERR_VALUE.
 * The call allocates nothing.  Every call on a device shares the one scratch
 * array, so calls that may overlap on the GPU must be ordered by the caller
 * (same stream, or events).  The first call on a device resolves the array's
 * device address (cudaGetSymbolAddress): make it before any stream capture. */
uint32_t ag_register_seeds_static_max(void);
int32_t ag_register_seeds_static(int32_t device, const uint32_t *seeds_dev, uint32_t n_seeds,
                                 uint64_t num_nodes, uint32_t *nodes_out_dev,
                                 uint32_t *seed_locals_out_dev, uint32_t *count_err_out_dev,
                                 void *stream);

/* --------------------------------------------------- heterogeneous path --
 * Stands in for HeteroCsrGraph + HeteroNeighborSampler (_core.pyi:609-720;
 * crates/aethergraph-core/src/graph/hetero.rs:312-423 from_relations,
 * crates/aethergraph-core/src/loader/hetero_sampler.rs:174-330 sample_neighbors).
 * Node and edge types are dense ids in the caller's order (the Python layer
 * maps names).  A node of type T is expanded along every edge type whose
 * destination type is T, in ascending edge type id, over the transposed
 * adjacency (hetero.rs:70-97); nodes are deduplicated per node type; an edge is
 * (source local, destination local) in its edge type's arrays, the locals
 * indexing the source / destination TYPE's nodes.  One WyRand stream per batch;
 * same picks, same order as the reference for the same seed.
 * Limits: <= 8 node types, <= 16 edge types, fewer than 2^32 nodes over all
 * types, fanout <= 32 per (edge type, hop). */
#define AG_MAX_NODE_TYPES 8
#define AG_MAX_EDGE_TYPES 16

/* Relation e is an edge list (rel_offsets == NULL or rel_offsets[e] == NULL:
 * rel_a[e] = sources, rel_b[e] = destinations, num_edges[e] each) or a CSR over
 * its source type (rel_offsets[e] = num_nodes[src_type[e]] + 1 offsets,
 * rel_b[e] = destinations); all arrays of one call in host or all in device
 * memory (mem_kind).  An endpoint outside its node type's range is
 * AG_ERR_VALUE (hetero.rs:346-379). */
int32_t ag_hetero_create(uint32_t num_node_types, const uint64_t *num_nodes, uint32_t num_edge_types,
                         const uint32_t *src_type, const uint32_t *dst_type,
                         const uint64_t *const *rel_offsets, const uint32_t *const *rel_a,
                         const uint32_t *const *rel_b, const uint64_t *num_edges, int32_t mem_kind,
                         int32_t device, ag_hetero_graph **out);
int32_t ag_hetero_info(const ag_hetero_graph *h, uint32_t *num_node_types, uint32_t *num_edge_types,
                       uint64_t *num_nodes /* [types] */, uint64_t *num_edges /* [edge types] */,
                       int32_t *device);
/* Host copy of one edge type's transposed adjacency (hetero.rs:70-97):
 * offsets[num_nodes[dst_type] + 1], sources[num_edges]. */
int32_t ag_hetero_in_adjacency(const ag_hetero_graph *h, uint32_t edge_type, uint64_t *offsets,
                               uint32_t *sources);
void ag_hetero_free(ag_hetero_graph *h);

/* AETHHETG v1 files (crates/aethergraph-core/src/internal/mmap_hetero.rs:1-45;
 * HeteroCsrGraph.save / .load, _core.pyi:609-660).  The type names travel in
 * ag_hetero_names (64-byte fields as in the file).  Loading checks every size
 * against the file length before reading, streams each relation's CSR into GPU
 * memory and proves it in full (offsets start at 0, never decrease, end at the
 * edge count; destinations below the destination type's count) as
 * mmap_hetero.rs:161-330 does; a bad file is AG_ERR_LOAD.  Edge weights, if the
 * file has them, are skipped: heterogeneous sampling is uniform
 * (hetero_sampler.rs:36-39).  Saving writes to a temporary file that is fsynced
 * and renamed over `path`. */
typedef struct {
    uint32_t num_node_types, num_edge_types;
    char node_type[AG_MAX_NODE_TYPES][64];
    char src[AG_MAX_EDGE_TYPES][64], rel[AG_MAX_EDGE_TYPES][64], dst[AG_MAX_EDGE_TYPES][64];
} ag_hetero_names;
int32_t ag_hetero_load(const char *path, int32_t device, ag_hetero_graph **out, ag_hetero_names *names);
int32_t ag_hetero_save(const ag_hetero_graph *h, const ag_hetero_names *names, const char *path);

/* Device output buffers of one heterogeneous batch.  Node type t's nodes are
 * nodes[node_start(t) .. +counts.nodes[t]) with node_start(t) = sum of the
 * counts of the types before it; edge type e's edges likewise in
 * edge_src_local / edge_dst_local.  edge_index_local (optional) holds, per edge
 * type, a contiguous int64 [2, E_e] block at element offset 2 * edge_start(e):
 * row 0 sources, row 1 destinations (aethergraph-py/src/hetero.rs:178-200). */
typedef struct {
    uint64_t cap_nodes, cap_edges, cap_seeds;
    uint32_t *nodes, *edge_src_local, *edge_dst_local, *seed_indices;
    int64_t *n_id, *edge_index_local, *seed_index;   /* optional int64 views */
    /* optional, per node type: f32 [cap_x[t], dim of that type's feature store]
     * rows of the type's `nodes` segment, filled when feature stores are passed.
     * cap_x[t] = 0 means cap_nodes rows.  A type with more nodes than cap_x[t]
     * gets its first cap_x[t] rows only (compare ag_hetero_counts.nodes[t]). */
    float *x[AG_MAX_NODE_TYPES];
    uint64_t cap_x[AG_MAX_NODE_TYPES];
} ag_hetero_buffers;

typedef struct {
    uint32_t num_node_types, num_edge_types, num_seeds, error;
    uint32_t nodes[AG_MAX_NODE_TYPES];
    uint32_t edges[AG_MAX_EDGE_TYPES];
    uint32_t total_nodes, total_edges;
    uint64_t draws;
} ag_hetero_counts;

/* fanout: [num_edge_types][num_hops] row-major, 0 = do not follow that edge
 * type at that hop (hetero_sampler.rs:25-60). */
int32_t ag_hetero_sampler_create(const ag_hetero_graph *h, const uint32_t *fanout, uint32_t num_hops,
                                 int32_t replace, uint64_t seed, int32_t rng_mode,
                                 ag_hetero_sampler **out);
/* A handle with scratch for `group` (<= 64) batches per launch chain. */
int32_t ag_hetero_sampler_create_group(const ag_hetero_graph *h, const uint32_t *fanout,
                                       uint32_t num_hops, int32_t replace, uint64_t seed,
                                       int32_t rng_mode, uint32_t group, ag_hetero_sampler **out);
int32_t ag_hetero_sampler_reseed(ag_hetero_sampler *s, uint64_t seed);
int32_t ag_hetero_sampler_bounds(const ag_hetero_sampler *s, uint64_t n_seeds, uint64_t *max_nodes,
                                 uint64_t *max_edges);
/* Seeds are host ids of node type seed_type, checked before anything is
 * launched (hetero_sampler.rs:174-187: AG_ERR_SAMPLING names the seed). */
int32_t ag_hetero_sample_into(ag_hetero_sampler *s, uint32_t seed_type, const uint32_t *seeds,
                              uint64_t n_seeds, ag_hetero_buffers *buf, void *stream);
int32_t ag_hetero_sample_wait(ag_hetero_sampler *s, ag_hetero_counts *counts);
/* One launch chain for n_batches batches rooted at the same node type (the batch
 * is blockIdx.y of every kernel).  batch_seeds[b] starts batch b's own RNG stream
 * (the loader's per-batch reseed, prefetch.rs:1003-1005); NULL (one batch only)
 * continues the handle's stream.  feats: NULL, or num_node_types feature stores
 * (entries may be NULL): node type t's rows are gathered into bufs[b].x[t] in the
 * same chain.  The wait returns per-batch counts and statuses. */
int32_t ag_hetero_sample_group_into(ag_hetero_sampler *s, uint32_t n_batches, uint32_t seed_type,
                                    const uint32_t *const *seeds, const uint64_t *n_seeds,
                                    const uint64_t *batch_seeds, const ag_features *const *feats,
                                    ag_hetero_buffers *bufs, void *stream);
int32_t ag_hetero_sample_group_wait(ag_hetero_sampler *s, ag_hetero_counts *counts,
                                    int32_t *statuses);
void ag_hetero_sampler_free(ag_hetero_sampler *s);

/* --------------------------------------------------------------- loader --
 * Stands in for the prefetching NeighborLoader (_core.pyi:380-464;
 * crates/aethergraph-core/src/loader/prefetch.rs:402-560 pipeline,
 * :911-1073 workers).  `sampler_threads` host threads each own one sampler
 * handle and one CUDA stream; a worker takes up to `group` queued batches at a
 * time and runs them as one launch chain (see "Groups" above), so up to
 * sampler_threads x group batches are in flight on the GPU.
 *   - submit assigns a sequence number; the work queue holds 8 x prefetch_depth
 *     items and submit blocks while it is full (prefetch.rs:457-477).
 *   - With seeded = 1 batch number seq is sampled from
 *     ag_batch_seed(cfg->seed, seq) and results are delivered in submission
 *     order; with seeded = 0 each worker's stream simply continues and results
 *     arrive as they finish (prefetch.rs:486-491, 926-930).
 *   - ag_loader_next waits up to timeout_ms (the reference waits 30 s) and
 *     returns AG_ERR_TIMEOUT, AG_ERR_SHUTDOWN after ag_loader_shutdown, or
 *     AG_ERR_WORKER once a worker failed (prefetch.rs:479-523).
 * Output buffers: pass your own with the submission (device memory, sized with
 * ag_loader_bounds) and get the same pointers back in the ag_batch; or pass
 * bufs == NULL and the loader takes a set from its pool (one device allocation
 * per batch, with the int64 views and, when a feature store is attached, x),
 * which ag_loader_release_batch hands back for reuse. `after_stream`, when not NULL, is a
 * stream whose already-queued work must finish before the batch's kernels
 * may write the buffers (the stream that last used recycled memory). */
typedef struct {
    int64_t batch_idx;
    uint64_t seq;
    ag_subgraph_buffers bufs;
    ag_sample_counts counts;
    int32_t owned;      /* 1 when bufs were allocated by the library */
    int32_t reserved;
} ag_batch;

typedef struct {
    uint64_t hits, misses, total;            /* prefetch.rs:853-899 */
    uint64_t sample_time_ns, feature_load_time_ns;
    uint64_t submitted, edges, nodes;        /* totals over delivered batches */
    double gather_ms, sample_ms;             /* device time, when profiling is on */
    uint64_t chains;                         /* launch chains run (a chain covers up to `group` batches) */
} ag_loader_stats;

int32_t ag_loader_create(const ag_graph *g, const ag_features *f, const ag_sampling_config *cfg,
                         int32_t seeded, uint32_t prefetch_depth, uint32_t sampler_threads,
                         uint32_t group, int32_t profiling, ag_loader **out);
/* Data-parallel ranks: batch number seq of this loader is sampled from
 * ag_batch_seed(cfg->seed, base + stride * seq).  Rank r of W ranks that takes
 * global batches r, r + W, ... sets (r, W) and every global batch draws from
 * the same stream at any W — the invariance the reference tests for its thread
 * pool (loader/sampler.rs:3116-3148; prefetch.rs:926-930 is the per-batch
 * reseed).  Default (0, 1).  Only before the first submit. */
int32_t ag_loader_set_seed_sequence(ag_loader *l, uint64_t base, uint64_t stride);
int32_t ag_loader_bounds(const ag_loader *l, uint64_t n_seeds, uint64_t *max_nodes,
                         uint64_t *max_edges);
int32_t ag_loader_submit(ag_loader *l, int64_t batch_idx, const uint32_t *seeds, uint64_t n_seeds,
                         int32_t seeds_mem, const ag_subgraph_buffers *bufs, void *after_stream);
/* submit_epoch (_core.pyi:425): n submissions in one call; bufs == NULL means
 * pooled buffers for all of them.  *n_done = how many were queued. */
int32_t ag_loader_submit_many(ag_loader *l, uint32_t n, const int64_t *batch_idx,
                              const uint32_t *const *seeds, const uint64_t *n_seeds,
                              int32_t seeds_mem, const ag_subgraph_buffers *bufs,
                              void *after_stream, uint32_t *n_done);
int32_t ag_loader_next(ag_loader *l, int64_t timeout_ms, ag_batch *out);
/* Like ag_loader_next for the first batch, then also returns every further
 * batch that is already deliverable (up to max_n) without waiting. */
int32_t ag_loader_next_many(ag_loader *l, int64_t timeout_ms, uint32_t max_n, ag_batch *out,
                            uint32_t *n_out);
/* Non-blocking: AG_ERR_TIMEOUT when nothing is ready. */
int32_t ag_loader_try_next(ag_loader *l, ag_batch *out);
/* Returns a pooled batch (owned == 1).  `stream` is the stream whose queued
 * work is the consumer's last use of the batch; the buffers' next batch waits
 * for it.  The memory stays valid until then or until ag_loader_free. */
int32_t ag_loader_release_batch(ag_loader *l, ag_batch *batch, void *stream);
int32_t ag_loader_stats_get(const ag_loader *l, ag_loader_stats *stats);
int32_t ag_loader_shutdown(ag_loader *l);
void ag_loader_free(ag_loader *l);

/* ---------------------------------------------------- subgraph rewrites --
 * SamplingConfig.subgraph_type other than "directional"
 * (crates/aethergraph-core/src/loader/sampler.rs:964-1040 apply_subgraph_type),
 * applied to the device arrays of a finished batch.  Per-hop counts keep
 * describing the sampling pass (sampler.rs:1533-1536).  All calls synchronise
 * `stream` before they return.
 *
 * Bidirectional (`mirror`, sampler.rs:1015-1040): the n_edges sampled edges stay;
 * walking them in order, the reverse of edge i (endpoints and locals swapped, same
 * edge id) is appended unless its (src_local, dst_local) pair is already among the
 * sampled edges or the reverses appended before it.  The u32 arrays (and edge_ids,
 * optional) need room for cap_edges >= 2 * n_edges entries; edge_index_local
 * (optional, room for [2, cap_edges]) is rewritten as [2, *n_edges_out]. */
int32_t ag_subgraph_mirror(int32_t device, uint64_t n_edges, uint64_t cap_edges, uint32_t *edge_src,
                           uint32_t *edge_dst, uint32_t *src_local, uint32_t *dst_local,
                           uint64_t *edge_ids, int64_t *edge_index_local, uint64_t *n_edges_out,
                           void *stream);
/* Induced (`induce`, sampler.rs:972-1013): the edges become every stored edge
 * u -> w with both ends among the n_nodes sampled nodes (device u32 ids, distinct),
 * ordered by u's local index, then by position in u's row; edge id = CSR position.
 * Two steps, because the edge count is only known after counting: plan (returns
 * the count), then fill into arrays of at least that capacity.  nodes_dev must
 * stay valid until the plan is freed. */
typedef struct ag_induce_plan ag_induce_plan;
int32_t ag_subgraph_induce_plan(const ag_graph *g, const uint32_t *nodes_dev, uint64_t n_nodes,
                                void *stream, ag_induce_plan **out, uint64_t *n_edges_out);
int32_t ag_subgraph_induce_fill(ag_induce_plan *plan, uint64_t cap_edges, uint32_t *edge_src,
                                uint32_t *edge_dst, uint32_t *src_local, uint32_t *dst_local,
                                uint64_t *edge_ids, int64_t *edge_index_local, void *stream);
void ag_subgraph_induce_free(ag_induce_plan *plan);

/* -------------------------------------------------- heterogeneous loader --
 * Stands in for HeteroNeighborLoader (_core.pyi:680-720;
 * crates/aethergraph-core/src/loader/prefetch.rs:984-1022 hetero workers,
 * :1940-2060).  The contract of the loader above (sequence numbers, a work queue
 * of 8 x prefetch_depth, in-order delivery and ag_batch_seed(seed, seq) per batch
 * when seeded, 30 s timeouts, a failed worker poisons the loader) over the
 * heterogeneous sampler: every batch is rooted at seed_type; `feats` is NULL or
 * one feature store per node type (entries may be NULL), whose rows arrive in
 * bufs.x[t].  Buffers always come from the loader's pool.  The rows reserved for
 * x[t] follow the counts seen so far; a batch with counts.nodes[t] > bufs.cap_x[t]
 * holds only the first cap_x[t] rows of that type, and the caller gathers the
 * type again from bufs.nodes. */
typedef struct ag_hetero_loader ag_hetero_loader;
typedef struct {
    int64_t batch_idx;
    uint64_t seq;
    ag_hetero_buffers bufs;
    ag_hetero_counts counts;
} ag_hetero_batch;

int32_t ag_hetero_loader_create(const ag_hetero_graph *g, uint32_t seed_type, const uint32_t *fanout,
                                uint32_t num_hops, int32_t replace, uint64_t seed, int32_t rng_mode,
                                int32_t seeded, const ag_features *const *feats,
                                uint32_t prefetch_depth, uint32_t sampler_threads, uint32_t group,
                                ag_hetero_loader **out);
/* Seeds are host ids of the seed type; one outside its range is AG_ERR_SAMPLING. */
int32_t ag_hetero_loader_submit(ag_hetero_loader *l, int64_t batch_idx, const uint32_t *seeds,
                                uint64_t n_seeds);
int32_t ag_hetero_loader_next(ag_hetero_loader *l, int64_t timeout_ms, ag_hetero_batch *out);
int32_t ag_hetero_loader_next_many(ag_hetero_loader *l, int64_t timeout_ms, uint32_t max_n,
                                   ag_hetero_batch *out, uint32_t *n_out);
int32_t ag_hetero_loader_release_batch(ag_hetero_loader *l, ag_hetero_batch *batch, void *stream);
int32_t ag_hetero_loader_stats_get(const ag_hetero_loader *l, ag_loader_stats *stats);
int32_t ag_hetero_loader_shutdown(ag_hetero_loader *l);
void ag_hetero_loader_free(ag_hetero_loader *l);

/* ------------------------------------------------------ synthetic inputs --
 * Seeded generators that build test and benchmark inputs directly in HBM
 * (no counterpart in the reference library; its benches generate synthetic
 * graphs on the host: crates/aethergraph-core/benches/sampling_scale.rs:29-49).
 * R-MAT over num_src x num_dst ids with quadrant probabilities a, b, c
 * (d = 1 - a - b - c); rows sorted by (source, destination); duplicates and
 * self-loops kept.  weight_sigma > 0 adds lognormal(0, sigma) f32 weights. */
int32_t ag_synth_rmat_graph(uint64_t num_nodes, uint64_t num_edges, float a, float b, float c,
                            uint64_t seed, float weight_sigma, int32_t device, ag_graph **out);
int32_t ag_synth_rmat_csr(uint64_t num_src, uint64_t num_dst, uint64_t num_edges, float a, float b,
                          float c, uint64_t seed, float weight_sigma, int32_t device,
                          uint64_t **offsets_dev, uint32_t **dst_dev, float **weights_dev);
/* Every source gets exactly `degree` destinations drawn uniformly. */
int32_t ag_synth_fixed_degree_csr(uint64_t num_src, uint64_t num_dst, uint32_t degree,
                                  uint64_t seed, int32_t device, uint64_t **offsets_dev,
                                  uint32_t **dst_dev);
int32_t ag_synth_free_device(void *ptr, int32_t device);
/* Rows [row_begin, row_end) of a num_nodes x dim table of ~N(0,1) values
 * (8-term Irwin-Hall), encoded as `dtype`. */
int32_t ag_synth_features(uint64_t num_nodes, uint64_t dim, int32_t dtype, uint64_t seed,
                          int32_t device, uint64_t row_begin, uint64_t row_end,
                          ag_features **out);
/* Shard `rank` of `world` of the same table in either layout (same bits as the
 * corresponding rows of the whole table). */
int32_t ag_synth_features_shard(uint64_t num_nodes, uint64_t dim, int32_t dtype, uint64_t seed,
                                int32_t device, uint32_t rank, uint32_t world, int32_t layout,
                                ag_features **out);

#ifdef __cplusplus
}
#endif
#endif /* AETHERGPU_H */

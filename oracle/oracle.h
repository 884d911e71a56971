/*
 * CPU oracle for the minibatch path — TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's CPU algorithm (the Rust crate
 * aethergraph-core): k-hop neighbor sampling over a static CSR, frontier dedup
 * and relabel, and the feature-row gather with f16/bf16 -> f32 upcast.  It
 * exists so the CUDA path can be checked bit for bit and so a CPU baseline can
 * be timed beside it.  Only the test-suite, the smoke check and the bench's
 * cpu_baseline / reference arm may link or load it.  The shipped library never
 * does.
 *
 * Parity status.  The reference is Rust and cannot be built where this file is
 * developed, so the oracle is pinned against every known-answer vector the
 * reference's own tests carry for this path (see tests/golden/ and the
 * "pins" list in tests/test_oracle_pins.py): the Philox4x32-10 zero vector,
 * the AETH v1 golden bytes and test_data/simple_graph.bin, the AETHFEAT header
 * layout, the GenSlots first-sighting cases, the take-all cases, the hetero
 * fixture counts, and exhaustive f16/bf16 decode against an independent
 * IEEE implementation (numpy).  The reference holds NO known-answer vector
 * for WyRand output or for a sampled subgraph with fanout < degree; there the
 * oracle is pinned by restatement of the cited lines only.
 * Weighted sampling: PARITY UNPINNED — the order in which the reference emits
 * the k selected neighbors is decided by Rust libcore's
 * select_nth_unstable_by, which is not part of the reference tree.  This
 * oracle emits them in ascending key order (ties by row position).
 *
 * Every function cites the reference file:line it follows (paths relative to
 * the reference project root).
 */
#ifndef AGO_ORACLE_H
#define AGO_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- RNG -------------------------------------------------------------- */

/* crates/aethergraph-core/src/loader/sampler.rs:69-75 */
uint64_t ago_batch_seed(uint64_t base, uint64_t batch_idx);

/* crates/aethergraph-core/src/internal/genstamp.rs:181-202.  Sequential form. */
typedef struct { uint64_t state; } ago_wyrand;
uint64_t ago_wyrand_next_u64(ago_wyrand *r);
uint32_t ago_wyrand_next_u32(ago_wyrand *r);
/* Random-access form: the value the (d+1)-th call of next_u64 returns for a
 * generator created with `seed`. */
uint64_t ago_wyrand_at(uint64_t seed, uint64_t d);

/* crates/aethergraph-core/src/internal/philox.rs:15-52 */
void ago_philox4x32_10(uint64_t seed, uint32_t layer, uint64_t node,
                       uint32_t draw_group, uint32_t out[4]);
uint32_t ago_philox_u32(uint64_t seed, uint32_t layer, uint64_t node,
                        uint32_t draw_index);
/* crates/aethergraph-core/src/internal/philox.rs:59-82.  Returns the number
 * of ids written to out (<= fanout). */
size_t ago_reservoir_sample(const uint32_t *neighbors, size_t degree,
                            size_t fanout, uint64_t seed, uint32_t layer,
                            uint64_t node, uint32_t *out);

/* crates/aethergraph-core/src/loader/sampler.rs:52-55 */
double ago_neg_ln_u64(uint64_t bits);

/* ---- feature codecs --------------------------------------------------- */

enum { AGO_F32 = 0, AGO_F16 = 1, AGO_BF16 = 2 };

/* crates/aethergraph-core/src/features/store.rs:1094-1104 */
uint16_t ago_f32_to_bf16(float v);
/* IEEE-754 binary32 -> binary16, round to nearest even (what half::f16::from_f32
 * computes; call site crates/aethergraph-core/src/features/store.rs:964-967). */
uint16_t ago_f32_to_f16(float v);
/* crates/aethergraph-core/src/internal/simd.rs:233-238 */
float ago_bf16_to_f32(uint16_t bits);
/* crates/aethergraph-core/src/internal/simd.rs:97-101 (half::f16::to_f32: exact) */
float ago_f16_to_f32(uint16_t bits);

void ago_encode_rows(const float *src, size_t count, int dtype, void *dst);
/* header.rs:110-116: decode `count` stored elements into f32 */
void ago_decode_rows(const void *src, size_t count, int dtype, float *dst);

/* crates/aethergraph-core/src/features/store.rs:777-838 (get_batch_into).
 * payload: num_nodes rows of dim elements of `dtype`; ids are checked against
 * num_nodes first.  Returns 0, or -1 - (position of the first bad id). */
/* internal/feature_codec.rs:73-133 (block-scaled int8) */
int ago_encode_i8(const float *values, size_t rows, size_t dim, int8_t *codes, float *scales);
int64_t ago_gather_i8(const int8_t *codes, const float *scales, uint64_t num_nodes, uint64_t dim,
                      const uint32_t *ids, size_t n, float *out);
int64_t ago_gather(const void *payload, uint64_t num_nodes, uint64_t dim,
                   int dtype, const uint32_t *ids, size_t n, float *out);

/* ---- file formats ----------------------------------------------------- */

/* crates/aethergraph-core/src/internal/mmap.rs:601-652 (CRC32 IEEE) */
uint32_t ago_crc32(uint32_t crc, const void *data, size_t len);

/* ---- homogeneous sampler --------------------------------------------- */

typedef struct {
    const uint64_t *offsets; /* num_nodes + 1 */
    const uint32_t *edges;   /* num_edges */
    const float *weights;    /* num_edges or NULL */
    uint64_t num_nodes;
    uint64_t num_edges;
} ago_csr;

typedef struct {
    const uint32_t *fanout; /* one per hop */
    uint32_t num_hops;
    int replace;
    int weighted;       /* uses csr.weights when set and present */
    int track_edge_ids; /* sampler.rs:117-120 */
    uint64_t seed;
    /* sampler.rs:416: above this node count the reference swaps its dense
     * dedup table for a hash map; results are identical, only speed differs.
     * 0 selects the reference's bound (8 << 20). */
    uint64_t dense_dedup_max_nodes;
} ago_config;

typedef struct {
    uint32_t *nodes;      size_t num_nodes;
    uint32_t *edge_src;   /* num_edges each */
    uint32_t *edge_dst;
    uint64_t *edge_ids;   /* NULL when !track_edge_ids */
    uint32_t *src_local;
    uint32_t *dst_local;  size_t num_edges;
    uint32_t *seed_locals; size_t num_seeds;
    uint64_t *num_sampled_nodes; /* num_hops + 1 */
    uint64_t *num_sampled_edges; /* num_hops */
    uint32_t num_hops;
    uint64_t draws;       /* RNG draws this call consumed */
} ago_subgraph;

typedef struct ago_sampler ago_sampler;

ago_sampler *ago_sampler_new(const ago_csr *g, const ago_config *cfg);
void ago_sampler_free(ago_sampler *s);
/* sampler.rs:509-511 */
void ago_sampler_reseed(ago_sampler *s, uint64_t seed);
/* sampler.rs:525-557 + 845-961.  Returns 0; -1 - position for the first seed
 * that is out of range (sampler.rs:230-239). */
int64_t ago_sample(ago_sampler *s, const uint32_t *seeds, size_t n,
                   ago_subgraph *out);
void ago_subgraph_free(ago_subgraph *sg);

/* ---- heterogeneous sampler -------------------------------------------- */

typedef struct {
    uint32_t src_type, dst_type;
    ago_csr csr; /* rows are sources of src_type, entries ids of dst_type */
} ago_relation;

typedef struct {
    uint64_t *offsets; /* num_dst + 1 */
    uint32_t *sources;
    uint64_t num_dst;
} ago_in_adjacency;

/* crates/aethergraph-core/src/graph/hetero.rs:70-97 */
void ago_transpose(const ago_csr *csr, uint64_t num_src, uint64_t num_dst,
                   ago_in_adjacency *out);
void ago_in_adjacency_free(ago_in_adjacency *a);

typedef struct {
    uint32_t num_node_types;
    const uint64_t *num_nodes; /* per node type */
    uint32_t num_edge_types;
    const ago_relation *relations;
    const uint32_t *fanout; /* [edge_type][hop], row-major */
    uint32_t num_hops;
    int replace;
    uint64_t seed;
    uint64_t dense_dedup_max_nodes; /* 0 = reference bound (1 << 20), hetero_sampler.rs:28 */
} ago_hetero_config;

typedef struct {
    uint32_t num_node_types, num_edge_types;
    uint32_t **nodes;   size_t *num_nodes;      /* per node type */
    uint32_t **edge_src_local;                  /* per edge type */
    uint32_t **edge_dst_local; size_t *num_edges;
    uint32_t *seed_indices; size_t num_seeds;
    uint64_t draws;
} ago_hetero_subgraph;

typedef struct ago_hetero_sampler ago_hetero_sampler;
ago_hetero_sampler *ago_hetero_sampler_new(const ago_hetero_config *cfg);
void ago_hetero_sampler_free(ago_hetero_sampler *s);
void ago_hetero_sampler_reseed(ago_hetero_sampler *s, uint64_t seed);
/* crates/aethergraph-core/src/loader/hetero_sampler.rs:174-330 */
int64_t ago_hetero_sample(ago_hetero_sampler *s, uint32_t seed_type,
                          const uint32_t *seeds, size_t n,
                          ago_hetero_subgraph *out);
void ago_hetero_subgraph_free(ago_hetero_subgraph *sg);
/* Incoming adjacency the sampler built, for the transpose pins. */
const ago_in_adjacency *ago_hetero_in_adjacency(const ago_hetero_sampler *s,
                                                uint32_t edge_type);

/* ---- timed CPU baseline ---------------------------------------------- */

typedef struct {
    uint64_t batches;
    uint64_t edges;       /* sampled edges over all batches */
    uint64_t nodes;       /* gathered rows over all batches */
    double seconds;       /* wall time of the timed loop */
    int threads;
    uint64_t checksum;    /* folds every output so the work cannot be elided */
} ago_bench_result;

/* Mirrors ParallelBatchSampler (sampler.rs:1726-1751): batch p reseeds with
 * batch_seed(cfg->seed, first_position + p); one sampler per thread; each
 * batch is sampled and, when payload != NULL, its nodes are gathered
 * (store.rs:777-838).  seeds holds num_batches * batch_size ids. */
int ago_bench_run(const ago_csr *g, const ago_config *cfg,
                  const void *payload, uint64_t dim, int dtype,
                  const uint32_t *seeds, size_t batch_size, size_t num_batches,
                  uint64_t first_position, int threads, ago_bench_result *res);

#ifdef __cplusplus
}
#endif
#endif

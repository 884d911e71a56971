// Heterogeneous k-hop neighbor sampler.
//
// Computes what the reference's HeteroNeighborSampler::sample_neighbors computes
// (crates/aethergraph-core/src/loader/hetero_sampler.rs:192-330): a node of type
// T is expanded along every edge type whose DESTINATION is T, in ascending edge
// type id, drawing sources from the transposed adjacency
// (crates/aethergraph-core/src/graph/hetero.rs:70-97); one WyRand stream per
// batch; dedup, `nodes` and local ids are per node type; edges are kept per edge
// type as (source local, destination local).
//
// The kernels are the homogeneous chain (insert -> assign -> pick -> ...) over a
// single id space: vertex (type, id) is the key type_base[type] + id, discovery
// order is global, and every edge carries its edge type.  What the reference
// keeps per type falls out at the end: a node's per-type local id is its rank
// among the nodes of its type in global discovery order, an edge's position in
// its edge type's arrays is its rank among that type's edges in emission order —
// two small multi-channel scans — followed by one scatter.
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "common.cuh"
#include "internal.h"
#include "sampler.cuh"

namespace ag {
namespace {

constexpr int kTile = 512;
constexpr int kPickThreads = 256;
constexpr int kMaxNT = AG_MAX_NODE_TYPES, kMaxET = AG_MAX_EDGE_TYPES;
constexpr int kChan = 16;  // channels of the class-rank scan (>= kMaxNT and kMaxET)
static_assert(kMaxNT <= kChan && kMaxET <= kChan, "class-rank scan has 16 channels");

struct HeteroMeta {
    uint32_t nt, et, num_hops;
    int replace, rng_mode;
    uint32_t type_base[kMaxNT + 1];      // key of (type t, id) = type_base[t] + id
    uint64_t type_nodes[kMaxNT];
    const uint64_t *in_offsets[kMaxET];  // transposed adjacency: rows are destinations
    const uint32_t *in_sources[kMaxET];
    uint64_t in_edges[kMaxET];
    uint8_t src_type[kMaxET], dst_type[kMaxET];
    uint32_t fanout[kMaxET][AG_MAX_HOPS];
    uint8_t in_count[kMaxNT];            // edge types into each node type, ascending id
    uint8_t in_list[kMaxNT][kMaxET];
};

struct HParams {
    const HeteroMeta *meta;
    DedupTable table;
    BatchState *state;
    TileDesc *tiles;
    uint32_t epoch_base;
    uint32_t n_seeds, seed_type;
    const uint32_t *seeds;
    uint64_t seed;
    // scratch, all in global discovery / emission order
    uint32_t *slot_of_seed, *slot_of_edge;
    FrontierEntry *frontier;
    uint64_t frontier_cap;
    uint32_t *node_key;     // [cap_nodes] key of the g-th discovered node
    uint8_t *node_tag;      // its node type
    uint32_t *node_rank;    // its rank within its type (= per-type local id)
    uint32_t *edge_exp;     // [cap_edges] global local id of the expanded (destination) node
    uint8_t *edge_tag;      // edge type
    uint32_t *edge_rank;    // rank within its edge type
    uint64_t cap_nodes, cap_edges;
    uint32_t *class_tiles;  // descriptors of the class-rank scans
    uint32_t class_epoch;   // the node scan runs under class_epoch, the edge scan under class_epoch + 1
    uint32_t *class_ticket;
    uint32_t *type_count, *et_count;  // totals per node type / edge type (device)
    uint32_t *type_start;   // first position of each node type's segment in `nodes`
    uint64_t start_draw;    // absolute index of the batch's first RNG draw (0 for a freshly seeded batch)
    // outputs
    uint32_t *nodes, *edge_src_local, *edge_dst_local, *seed_indices;
    int64_t *n_id, *edge_index_local, *seed_index;
    ag_hetero_counts *counts;
};

__device__ __forceinline__ uint32_t type_of_key(const HeteroMeta &m, uint32_t key) {
    uint32_t t = 0;
    while (t + 1 < m.nt && key >= m.type_base[t + 1]) ++t;
    return t;
}

// take / draws for one (node, incoming edge type) unit (hetero_sampler.rs:278-284).
__device__ __forceinline__ void unit_demand(int replace, uint64_t deg, uint32_t k, uint32_t &take, uint64_t &draws) {
    take = 0; draws = 0;
    if (deg == 0 || k == 0) return;
    if (replace) { take = k; draws = k; return; }
    if (deg <= (uint64_t)k) { take = (uint32_t)deg; return; }
    take = k; draws = k;
}

__device__ __forceinline__ void in_row(const HeteroMeta &m, uint32_t et, uint32_t id, uint64_t &off, uint64_t &deg) {
    const uint64_t a = __ldg(m.in_offsets[et] + id), b = __ldg(m.in_offsets[et] + id + 1);
    off = a; deg = b >= a ? b - a : 0;
    if (b > m.in_edges[et]) deg = 0;
}

// Every kernel's grid has the batch as blockIdx.y; the group's parameter blocks
// sit in one device array.
__global__ void k_het_insert_seeds(const HParams *__restrict__ pa) {
    const HParams &p = pa[blockIdx.y];
    const HeteroMeta &m = *p.meta;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n_seeds) return;
    const uint32_t id = p.seeds[i];
    if ((uint64_t)id >= m.type_nodes[p.seed_type]) {
        atomicOr(&p.state->error, kErrBadSeed);
        p.slot_of_seed[i] = 0xFFFFFFFFu;
        return;
    }
    p.slot_of_seed[i] = table_insert_min(p.table, m.type_base[p.seed_type] + id, enc_pending(p.table.gen, 0, i),
                                         &p.state->error);
}

// Same single-pass scan as the homogeneous assign; the demand of a new node is
// the sum over the edge types into its type.
__global__ void __launch_bounds__(kTile)
k_het_assign(const HParams *__restrict__ pa, uint32_t stage, int has_next) {
    __shared__ uint32_t s_tile;
    __shared__ ScanVal s_warp[kTile / 32];
    __shared__ ScanVal s_prefix;
    const HParams &p = pa[blockIdx.y];
    const HeteroMeta &m = *p.meta;
    BatchState *bs = p.state;
    StageInfo si = bs->stage[stage];
    if (stage == 0) {
        // A reseeded batch starts its stream at draw 0; otherwise the handle's stream
        // continues where its previous batch stopped (the host keeps that position).
        si = StageInfo{};
        si.draws = p.start_draw;
    }
    const uint32_t count = (stage == 0) ? p.n_seeds : si.hop_edges;
    const uint32_t n_tiles = max(1u, (count + kTile - 1) / kTile);
    const uint32_t edges_before_next = si.n_edges + ((stage == 0) ? 0u : count);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t gen = p.table.gen;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_tile = atomicAdd(&bs->ticket, 1u);
        __syncthreads();
        const uint32_t tile = s_tile;
        if (tile >= n_tiles) {
            if (threadIdx.x == 0 && tile == n_tiles + gridDim.x - 1) bs->ticket = 0;
            return;
        }
        const uint32_t item = tile * kTile + threadIdx.x;
        uint32_t slot = 0xFFFFFFFFu, key = 0;
        bool first = false;
        if (item < count) {
            slot = (stage == 0) ? p.slot_of_seed[item] : p.slot_of_edge[si.n_edges + item];
            if (slot != 0xFFFFFFFFu) {
                const uint64_t cur = __ldcg((const unsigned long long *)&p.table.slots[slot]);
                first = ((uint32_t)cur == enc_pending(gen, stage, item));
                key = (uint32_t)(cur >> 32);
            }
        }
        ScanVal v{first ? 1u : 0u, 0u, 0ull};
        uint32_t type = 0;
        if (first) {
            type = type_of_key(m, key);
            if (has_next) {
                const uint32_t id = key - m.type_base[type];
                for (uint32_t i = 0; i < m.in_count[type]; ++i) {
                    const uint32_t et = m.in_list[type][i];
                    const uint32_t k = m.fanout[et][stage];
                    if (!k) continue;
                    uint64_t off, deg;
                    in_row(m, et, id, off, deg);
                    uint32_t take;
                    uint64_t draws;
                    unit_demand(m.replace, deg, k, take, draws);
                    v.take += take; v.draws += draws;
                }
            }
        }
        const ScanVal incl = warp_inclusive_scan(v, lane);
        if (lane == 31) s_warp[warp] = incl;
        __syncthreads();
        if (warp == 0) {
            ScanVal w = (lane < kTile / 32) ? s_warp[lane] : ScanVal{0, 0, 0};
            const ScanVal wi = warp_inclusive_scan(w, lane);
            const ScanVal block_total = ScanVal{__shfl_sync(0xffffffffu, wi.flags, 31),
                                                __shfl_sync(0xffffffffu, wi.take, 31),
                                                __shfl_sync(0xffffffffu, wi.draws, 31)};
            if (lane < kTile / 32) s_warp[lane] = ScanVal{wi.flags - w.flags, wi.take - w.take, wi.draws - w.draws};
            const ScanVal prefix = lookback_exclusive(p.tiles, tile, p.epoch_base + stage, block_total, lane, &bs->error);
            if (lane == 0) {
                s_prefix = prefix;
                if (tile == n_tiles - 1) {
                    const ScanVal tot = prefix + block_total;
                    StageInfo nx;
                    nx.n_nodes = si.n_nodes + tot.flags;
                    nx.n_edges = edges_before_next;
                    nx.frontier_n = tot.flags;
                    nx.hop_edges = tot.take;
                    nx.draws = si.draws + tot.draws;
                    nx.hop_draws = 0;
                    bs->stage[stage + 1] = nx;
                    bs->nodes_per_stage[stage] = tot.flags;
                    if (stage == 0) bs->stage[0] = si;
                }
            }
        }
        __syncthreads();
        if (first) {
            const ScanVal base = s_prefix + s_warp[warp];
            const ScanVal excl = ScanVal{base.flags + incl.flags - v.flags, base.take + incl.take - v.take,
                                         base.draws + incl.draws - v.draws};
            const uint32_t local = si.n_nodes + excl.flags;
            if ((uint64_t)local >= p.cap_nodes || (uint64_t)local >= kMaxPos ||
                (has_next && (uint64_t)excl.flags >= p.frontier_cap)) {
                atomicOr(&bs->error, kErrCapacity);
                if (has_next && (uint64_t)excl.flags < p.frontier_cap) {
                    FrontierEntry none{};
                    none.deg = 0xFFFFFFFFu;  // no such node type: the pick kernel skips it
                    p.frontier[excl.flags] = none;
                }
            } else {
                p.node_key[local] = key;
                p.node_tag[local] = (uint8_t)type;
                p.table.slots[slot] = ((uint64_t)key << 32) | enc_final(gen, local);
                if (has_next) {
                    FrontierEntry fe{};
                    fe.dbase = si.draws + excl.draws;
                    fe.id = key;
                    fe.local = local;
                    fe.deg = type;  // node type rides in the unused degree field
                    fe.ebase = excl.take;
                    p.frontier[excl.flags] = fe;
                }
            }
        }
    }
}

// One warp per frontier node; for each edge type into its type, in ascending
// edge type id, the lanes reproduce take-all / Floyd / replace
// (hetero_sampler.rs:364-422) and emit the edges at consecutive slots.
__global__ void __launch_bounds__(kPickThreads)
k_het_pick(const HParams *__restrict__ pa, uint32_t hop) {
    const HParams &p = pa[blockIdx.y];
    const HeteroMeta &m = *p.meta;
    const StageInfo nx = p.state->stage[hop + 1];
    const int lane = threadIdx.x & 31;
    for (uint32_t j = (blockIdx.x * kPickThreads + threadIdx.x) >> 5; j < nx.frontier_n;
         j += gridDim.x * (kPickThreads / 32)) {
        const FrontierEntry fe = p.frontier[j];
        const uint32_t type = fe.deg;
        if (type >= m.nt) continue;  // placeholder left by a capacity overflow (warp-uniform)
        const uint32_t id = fe.id - m.type_base[type];
        uint32_t e_off = fe.ebase;
        uint64_t d_off = fe.dbase;
        for (uint32_t i = 0; i < m.in_count[type]; ++i) {
            const uint32_t et = m.in_list[type][i];
            const uint32_t k = m.fanout[et][hop];
            if (!k) continue;
            uint64_t off, deg64;
            in_row(m, et, id, off, deg64);
            uint32_t take;
            uint64_t draws;
            unit_demand(m.replace, deg64, k, take, draws);
            if (!take) continue;
            const uint32_t deg = (uint32_t)min(deg64, (uint64_t)0xFFFFFFFFu);
            const bool sampled = !m.replace && deg64 > k;
            for (uint32_t c = 0; c < take; c += 32) {  // k <= 32: one round; take-all of a long row: several
                const uint32_t t = c + lane;
                uint32_t pick = t, ip = 0;
                if (t < take && (m.replace || sampled)) {
                    const uint32_t r = (m.rng_mode == AG_RNG_PHILOX)
                        ? philox_u32(p.seed, hop, ((uint64_t)et << 32) | fe.id, t)
                        : (uint32_t)wyrand_at(p.seed, d_off + t);
                    if (m.replace) pick = (uint32_t)(((uint64_t)r * deg) >> 32);
                    else { ip = deg - k + t; pick = (uint32_t)(((uint64_t)r * ((uint64_t)ip + 1)) >> 32); }
                }
                if (sampled) {
                    for (uint32_t s = 1; s < k; ++s) {
                        const uint32_t js = __shfl_sync(0xffffffffu, pick, s);
                        const bool hit = (uint32_t)lane < s && pick == js;
                        const uint32_t mm = __ballot_sync(0xffffffffu, hit);
                        if ((uint32_t)lane == s && mm) pick = ip;
                    }
                }
                if (t < take) {
                    const uint32_t e_rel = e_off + t;
                    const uint64_t e = (uint64_t)nx.n_edges + e_rel;
                    if (e >= p.cap_edges || e_rel >= kMaxPos) { atomicOr(&p.state->error, kErrCapacity); continue; }
                    const uint32_t src = ld_stream_u32(m.in_sources[et] + off + pick);
                    p.edge_exp[e] = fe.local;
                    p.edge_tag[e] = (uint8_t)et;
                    p.slot_of_edge[e] = table_insert_min(p.table, m.type_base[m.src_type[et]] + src,
                                                         enc_pending(p.table.gen, hop + 1, e_rel), &p.state->error);
                }
            }
            e_off += take;
            d_off += draws;
        }
    }
}

// Rank of every item among the items with the same tag, in item order, plus the
// per-tag totals: a 16-channel single-pass scan (same look-back scheme, bounded
// polls).  Descriptor layout per tile: status, agg[16], incl[16].
constexpr int kClassTile = 1024;
constexpr int kClassThreads = 256;
constexpr int kDescWords = 1 + 2 * kChan;

__global__ void __launch_bounds__(kClassThreads)
k_class_rank(const HParams *__restrict__ pa, int edges) {
    __shared__ uint32_t s_tile;
    __shared__ uint32_t s_cnt[kClassThreads / 32][kChan];   // per warp, per channel: count within the tile
    __shared__ uint32_t s_base[kChan];                      // exclusive prefix of the tile per channel
    const HParams &p = pa[blockIdx.y];
    const StageInfo fin = p.state->stage[p.meta->num_hops + 1];
    const uint8_t *__restrict__ tags = edges ? p.edge_tag : p.node_tag;
    uint32_t *ranks = edges ? p.edge_rank : p.node_rank;
    uint32_t *totals = edges ? p.et_count : p.type_count;
    uint32_t *tiles = p.class_tiles, *ticket = p.class_ticket, *err = &p.state->error;
    const uint32_t epoch = p.class_epoch + (edges ? 1u : 0u);
    const uint32_t n = edges ? (uint32_t)min((uint64_t)fin.n_edges, p.cap_edges) : (uint32_t)min((uint64_t)fin.n_nodes, p.cap_nodes);
    const uint32_t n_tiles = max(1u, (n + kClassTile - 1) / kClassTile);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (;;) {
        __syncthreads();
        if (threadIdx.x == 0) s_tile = atomicAdd(ticket, 1u);
        __syncthreads();
        const uint32_t tile = s_tile;
        if (tile >= n_tiles) {
            if (threadIdx.x == 0 && tile == n_tiles + gridDim.x - 1) *ticket = 0;
            return;
        }
        // each warp owns 128 consecutive items = 4 rounds of 32
        uint32_t my_tag[4], my_rank[4];
        uint32_t run[kChan];
#pragma unroll
        for (int c = 0; c < kChan; ++c) run[c] = 0;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t i = tile * kClassTile + warp * 128 + r * 32 + lane;
            const uint32_t tag = i < n ? tags[i] : 0xFFu;
            my_tag[r] = tag;
            my_rank[r] = 0;
#pragma unroll
            for (int c = 0; c < kChan; ++c) {
                const uint32_t b = __ballot_sync(0xffffffffu, tag == (uint32_t)c);
                if (tag == (uint32_t)c) my_rank[r] = run[c] + __popc(b & ((1u << lane) - 1u));
                run[c] += __popc(b);
            }
        }
        if (lane < kChan) {
            uint32_t v = 0;
#pragma unroll
            for (int c = 0; c < kChan; ++c) if (lane == c) v = run[c];
            s_cnt[warp][lane] = v;
        }
        __syncthreads();
        if (warp == 0) {
            // per channel: exclusive prefix over the warps, tile aggregate, look-back
            uint32_t agg = 0;
            if (lane < kChan) {
                for (int w = 0; w < kClassThreads / 32; ++w) { const uint32_t v = s_cnt[w][lane]; s_cnt[w][lane] = agg; agg += v; }
            }
            uint32_t *desc = tiles + (uint64_t)tile * kDescWords;
            uint32_t prefix = 0;
            if (tile == 0) {
                if (lane < kChan) { desc[1 + lane] = agg; desc[1 + kChan + lane] = agg; }
                __syncwarp();
                if (lane == 0) st_release_u32(&desc[0], (epoch << 2) | kTileIncl);
            } else {
                if (lane < kChan) desc[1 + lane] = agg;
                __syncwarp();
                if (lane == 0) st_release_u32(&desc[0], (epoch << 2) | kTileAgg);
                // lane c < 16 accumulates channel c while walking back one tile at a time
                for (int look = (int)tile - 1; look >= 0; --look) {
                    uint32_t *d = tiles + (uint64_t)look * kDescWords;
                    uint32_t st = 0, spins = 0;
                    if (lane == 0) {
                        for (;;) {
                            st = ld_acquire_u32(&d[0]);
                            if ((st >> 2) == epoch && (st & 3u) != 0) break;
                            if (++spins > kSpinLimit) { atomicOr(err, kErrSpinTimeout); st = (epoch << 2) | kTileIncl; break; }
                            __nanosleep(32);
                        }
                    }
                    st = __shfl_sync(0xffffffffu, st, 0);
                    spins = __shfl_sync(0xffffffffu, spins, 0);
                    __syncwarp();
                    const bool incl = (st & 3u) == kTileIncl;
                    if (lane < kChan && spins <= kSpinLimit) {
                        // the acquire above was done by lane 0; order this lane's reads behind it
                        __threadfence();
                        prefix += incl ? d[1 + kChan + lane] : d[1 + lane];
                    }
                    if (incl) break;
                }
                if (lane < kChan) desc[1 + kChan + lane] = prefix + agg;
                __syncwarp();
                if (lane == 0) st_release_u32(&desc[0], (epoch << 2) | kTileIncl);
            }
            if (lane < kChan) {
                s_base[lane] = prefix;
                if (tile == n_tiles - 1) totals[lane] = prefix + agg;
            }
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const uint32_t i = tile * kClassTile + warp * 128 + r * 32 + lane;
            if (i < n && my_tag[r] < kChan) ranks[i] = s_base[my_tag[r]] + s_cnt[warp][my_tag[r]] + my_rank[r];
        }
    }
}

// Per-type arrays out of the global ones.  Segments: node type t starts at the
// sum of the counts of the types before it; edge type likewise.
__global__ void k_het_scatter(const HParams *__restrict__ pa) {
    const HParams &p = pa[blockIdx.y];
    const HeteroMeta &m = *p.meta;
    BatchState *bs = p.state;
    const StageInfo fin = bs->stage[m.num_hops + 1];
    const uint32_t n_nodes = min((uint64_t)fin.n_nodes, p.cap_nodes);
    const uint32_t n_edges = min((uint64_t)fin.n_edges, p.cap_edges);
    __shared__ uint32_t s_toff[kChan + 1], s_eoff[kChan + 1];
    if (threadIdx.x == 0) {
        uint32_t a = 0, b = 0;
        for (uint32_t t = 0; t < kChan; ++t) { s_toff[t] = a; a += (t < m.nt) ? p.type_count[t] : 0; }
        for (uint32_t t = 0; t < kChan; ++t) { s_eoff[t] = b; b += (t < m.et) ? p.et_count[t] : 0; }
        s_toff[kChan] = a; s_eoff[kChan] = b;
        if (blockIdx.x == 0) for (uint32_t t = 0; t < kChan; ++t) p.type_start[t] = s_toff[t];  // for the gathers
    }
    __syncthreads();
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t g = tid; g < n_nodes; g += stride) {
        const uint32_t t = p.node_tag[g];
        const uint32_t at = s_toff[t] + p.node_rank[g];
        const uint32_t id = p.node_key[g] - m.type_base[t];
        p.nodes[at] = id;
        if (p.n_id) p.n_id[at] = (int64_t)id;
    }
    for (uint64_t e = tid; e < n_edges; e += stride) {
        const uint32_t et = p.edge_tag[e];
        const uint32_t slot = p.slot_of_edge[e];
        const uint32_t src_g = (slot == 0xFFFFFFFFu) ? 0 : ((uint32_t)__ldcg((const unsigned long long *)&p.table.slots[slot]) & kPosMask);
        const uint32_t sl = src_g < n_nodes ? p.node_rank[src_g] : 0xFFFFFFFFu;
        const uint32_t dl = p.node_rank[p.edge_exp[e]];
        const uint32_t at = s_eoff[et] + p.edge_rank[e];
        p.edge_src_local[at] = sl;
        p.edge_dst_local[at] = dl;
        if (p.edge_index_local) {
            // each edge type's [2, E_et] block is contiguous: row 0 sources, row 1 destinations
            int64_t *blk = p.edge_index_local + 2ull * s_eoff[et];
            blk[p.edge_rank[e]] = (int64_t)sl;
            blk[(uint64_t)p.et_count[et] + p.edge_rank[e]] = (int64_t)dl;
        }
    }
    for (uint64_t i = tid; i < p.n_seeds; i += stride) {
        const uint32_t slot = p.slot_of_seed[i];
        uint32_t v = 0xFFFFFFFFu;
        if (slot != 0xFFFFFFFFu) {
            const uint32_t g = (uint32_t)__ldcg((const unsigned long long *)&p.table.slots[slot]) & kPosMask;
            if (g < n_nodes) v = p.node_rank[g];
        }
        p.seed_indices[i] = v;
        if (p.seed_index) p.seed_index[i] = (int64_t)v;
    }
    if (tid == 0) {
        ag_hetero_counts c{};
        c.num_node_types = m.nt; c.num_edge_types = m.et; c.num_seeds = p.n_seeds;
        for (uint32_t t = 0; t < m.nt; ++t) c.nodes[t] = p.type_count[t];
        for (uint32_t t = 0; t < m.et; ++t) c.edges[t] = p.et_count[t];
        c.total_nodes = n_nodes; c.total_edges = n_edges;
        c.draws = fin.draws - bs->stage[0].draws;
        c.error = bs->error;
        if ((uint64_t)fin.n_nodes > p.cap_nodes || (uint64_t)fin.n_edges > p.cap_edges) c.error |= kErrCapacity;
        *p.counts = c;
        bs->stream_pos = fin.draws;
        bs->error = 0;
        bs->ticket = 0;
    }
}

// key = dst << 32 | src for every edge of a relation given as an edge list
__global__ void k_transpose_keys_edges(const uint32_t *src, const uint32_t *dst, uint64_t e, uint64_t num_src,
                                       uint64_t num_dst, uint64_t *keys, uint32_t *bad) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t s = src[i], d = dst[i];
        if ((uint64_t)s >= num_src || (uint64_t)d >= num_dst) atomicOr(bad, 1u);
        keys[i] = ((uint64_t)d << 32) | s;
    }
}

// the same from a CSR (rows are sources): thread per edge, the row found by search
__global__ void k_transpose_keys_csr(const uint64_t *offsets, const uint32_t *dst, uint64_t e, uint64_t num_src,
                                     uint64_t num_dst, uint64_t *keys, uint32_t *bad) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t lo = 0, hi = num_src;  // last row with offsets[row] <= i
        while (hi - lo > 1) { const uint64_t mid = (lo + hi) >> 1; if (offsets[mid] <= i) lo = mid; else hi = mid; }
        const uint32_t d = dst[i];
        if ((uint64_t)d >= num_dst) atomicOr(bad, 1u);
        keys[i] = ((uint64_t)d << 32) | (uint32_t)lo;
    }
}

int grid_for(uint64_t n) {
    const uint64_t b = (n + 255) / 256;
    return (int)std::max<uint64_t>(1, std::min<uint64_t>(b, (uint64_t)kSMs * 16));
}

uint64_t next_pow2(uint64_t v) { uint64_t p = 1; while (p < v) p <<= 1; return p; }

}  // namespace
}  // namespace ag

using namespace ag;


struct ag_hetero_sampler {
    const ag_hetero_graph *g = nullptr;
    int device = 0;
    uint32_t group = 1;
    HeteroMeta meta{};
    HeteroMeta *meta_dev = nullptr;
    uint64_t seed = 0;
    bool dirty = true, in_flight = false;
    uint64_t stream_pos = 0;   // draws consumed by earlier continuing batches (host-side, survives scratch growth)
    bool pending_pos = false;  // a continuing batch was launched and not yet accounted
    uint32_t epoch = 0, gen = 0, class_epoch = 0, last_batches = 0;
    uint64_t cap_seeds = 0, max_nodes = 0, max_edges = 0, max_hop_edges = 0, max_frontier = 0, table_cap = 0, n_tiles = 0,
             class_tiles_n = 0;
    // scratch, each array x group
    uint64_t *table = nullptr;
    uint32_t *slot_of_seed = nullptr, *slot_of_edge = nullptr, *node_key = nullptr, *node_rank = nullptr,
             *edge_exp = nullptr, *edge_rank = nullptr, *class_tiles = nullptr, *class_misc = nullptr, *seeds_dev = nullptr;
    uint8_t *node_tag = nullptr, *edge_tag = nullptr;
    FrontierEntry *frontier = nullptr;
    TileDesc *tiles = nullptr;
    BatchState *state = nullptr;
    HParams *params_dev = nullptr, *params_host = nullptr;
    GatherArgs *gather_dev = nullptr, *gather_host = nullptr;  // [node type][batch]
    ag_hetero_counts *counts_dev = nullptr, *counts_host = nullptr;
    uint32_t *seeds_pinned = nullptr;
    cudaEvent_t done = nullptr;
};

constexpr int kMiscWords = 3 * kChan + 2;  // type_count, et_count, type_start, ticket (per batch)

extern "C" void ag_hetero_free(ag_hetero_graph *h) {
    if (!h) return;
    DeviceGuard guard(h->device);
    for (uint32_t e = 0; e < h->et; ++e) { cudaFree(h->in_offsets[e]); cudaFree(h->in_sources[e]); }
    delete h;
}

// One relation per edge type, each either an edge list (rel_offsets[e] == NULL:
// rel_a[e] = sources, rel_b[e] = destinations) or a CSR over the source type
// (rel_offsets[e] = offsets, rel_b[e] = destinations), in host or device memory.
// Only the transposed adjacency is kept: for each destination its sources in
// ascending order, which is the stored edge order the reference's transpose
// yields (graph/hetero.rs:70-97).
extern "C" int32_t ag_hetero_create(uint32_t num_node_types, const uint64_t *num_nodes, uint32_t num_edge_types,
                                    const uint32_t *src_type, const uint32_t *dst_type,
                                    const uint64_t *const *rel_offsets, const uint32_t *const *rel_a,
                                    const uint32_t *const *rel_b, const uint64_t *num_edges, int32_t mem_kind,
                                    int32_t device, ag_hetero_graph **out) {
    if (!num_nodes || !out || (num_edge_types && (!src_type || !dst_type || !rel_b || !num_edges)))
        return fail(AG_ERR_VALUE, "ag_hetero_create: null argument");
    if (num_node_types == 0 || num_node_types > (uint32_t)kMaxNT)
        return fail(AG_ERR_VALUE, "between 1 and %d node types are supported (got %u)", kMaxNT, num_node_types);
    if (num_edge_types > (uint32_t)kMaxET)
        return fail(AG_ERR_VALUE, "at most %d edge types are supported (got %u)", kMaxET, num_edge_types);
    uint64_t total = 0;
    for (uint32_t t = 0; t < num_node_types; ++t) total += num_nodes[t];
    if (total >= 0xFFFFFFFFull) return fail(AG_ERR_VALUE, "the node types together hold %llu nodes; the limit is 2^32 - 1",
                                            (unsigned long long)total);
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_hetero_graph *h = new ag_hetero_graph();
    h->device = device; h->nt = num_node_types; h->et = num_edge_types;
    for (uint32_t t = 0; t < num_node_types; ++t) h->num_nodes[t] = num_nodes[t];
    int32_t st = AG_OK;
    uint32_t *bad = nullptr;
    if (cudaMalloc(&bad, 4) != cudaSuccess) { delete h; return fail(AG_ERR_CUDA, "out of device memory"); }
    for (uint32_t e = 0; e < num_edge_types && st == AG_OK; ++e) {
        if (src_type[e] >= num_node_types || dst_type[e] >= num_node_types) { st = fail(AG_ERR_VALUE, "edge type %u names an unknown node type", e); break; }
        h->src_type[e] = src_type[e]; h->dst_type[e] = dst_type[e]; h->num_edges[e] = num_edges[e];
        const uint64_t E = num_edges[e], ns = num_nodes[src_type[e]], nd = num_nodes[dst_type[e]];
        const bool csr = rel_offsets && rel_offsets[e];
        uint64_t *keys = nullptr, *off_dev = nullptr;
        uint32_t *a_dev = nullptr, *b_dev = nullptr;
        bool own = false;
        do {
            if (cudaMalloc(&keys, std::max<uint64_t>(E, 1) * 8) != cudaSuccess) { st = fail(AG_ERR_CUDA, "out of device memory"); break; }
            cudaMemset(bad, 0, 4);
            if (mem_kind == AG_MEM_HOST) {
                own = true;
                if (csr) {
                    if (cudaMalloc(&off_dev, (ns + 1) * 8) != cudaSuccess || cudaMemcpy(off_dev, rel_offsets[e], (ns + 1) * 8, cudaMemcpyHostToDevice) != cudaSuccess) { st = fail(AG_ERR_CUDA, "upload failed"); break; }
                } else if (E) {
                    if (cudaMalloc(&a_dev, E * 4) != cudaSuccess || cudaMemcpy(a_dev, rel_a[e], E * 4, cudaMemcpyHostToDevice) != cudaSuccess) { st = fail(AG_ERR_CUDA, "upload failed"); break; }
                }
                if (E && (cudaMalloc(&b_dev, E * 4) != cudaSuccess || cudaMemcpy(b_dev, rel_b[e], E * 4, cudaMemcpyHostToDevice) != cudaSuccess)) { st = fail(AG_ERR_CUDA, "upload failed"); break; }
            } else {
                off_dev = csr ? (uint64_t *)rel_offsets[e] : nullptr;
                a_dev = csr ? nullptr : (uint32_t *)rel_a[e];
                b_dev = (uint32_t *)rel_b[e];
            }
            if (E) {
                if (csr) k_transpose_keys_csr<<<grid_for(E), 256>>>(off_dev, b_dev, E, ns, nd, keys, bad);
                else k_transpose_keys_edges<<<grid_for(E), 256>>>(a_dev, b_dev, E, ns, nd, keys, bad);
            }
            uint32_t hb = 0;
            if (cudaMemcpy(&hb, bad, 4, cudaMemcpyDeviceToHost) != cudaSuccess) { st = fail(AG_ERR_CUDA, "transpose failed: %s", cudaGetErrorString(cudaGetLastError())); break; }
            if (hb) { st = fail(AG_ERR_VALUE, "edge type %u holds an endpoint outside its node type's range", e); break; }
            st = keys_to_sorted_csr(keys, E, nd, &h->in_offsets[e], &h->in_sources[e]);
            keys = nullptr;  // consumed
        } while (0);
        cudaFree(keys);
        if (own) { cudaFree(off_dev); cudaFree(a_dev); cudaFree(b_dev); }
    }
    cudaFree(bad);
    if (st != AG_OK) { ag_hetero_free(h); return st; }
    *out = h;
    return AG_OK;
}

extern "C" int32_t ag_hetero_info(const ag_hetero_graph *h, uint32_t *num_node_types, uint32_t *num_edge_types,
                                  uint64_t *num_nodes, uint64_t *num_edges, int32_t *device) {
    if (!h) return fail(AG_ERR_VALUE, "ag_hetero_info: null graph");
    if (num_node_types) *num_node_types = h->nt;
    if (num_edge_types) *num_edge_types = h->et;
    if (num_nodes) for (uint32_t t = 0; t < h->nt; ++t) num_nodes[t] = h->num_nodes[t];
    if (num_edges) for (uint32_t e = 0; e < h->et; ++e) num_edges[e] = h->num_edges[e];
    if (device) *device = h->device;
    return AG_OK;
}

// Copies the transposed adjacency of one edge type to host arrays
// (offsets: num_nodes[dst_type] + 1, sources: num_edges).
extern "C" int32_t ag_hetero_in_adjacency(const ag_hetero_graph *h, uint32_t edge_type, uint64_t *offsets, uint32_t *sources) {
    if (!h || edge_type >= h->et) return fail(AG_ERR_VALUE, "ag_hetero_in_adjacency: bad argument");
    DeviceGuard guard(h->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint64_t nd = h->num_nodes[h->dst_type[edge_type]];
    if (offsets) AG_CUDA(cudaMemcpy(offsets, h->in_offsets[edge_type], (nd + 1) * 8, cudaMemcpyDeviceToHost));
    if (sources && h->num_edges[edge_type])
        AG_CUDA(cudaMemcpy(sources, h->in_sources[edge_type], h->num_edges[edge_type] * 4, cudaMemcpyDeviceToHost));
    return AG_OK;
}

namespace {

uint64_t het_per_node(const HeteroMeta &m, uint32_t hop) {
    uint64_t per_node = 0;  // most edges any node can emit at this hop
    for (uint32_t t = 0; t < m.nt; ++t) {
        uint64_t k = 0;
        for (uint32_t i = 0; i < m.in_count[t]; ++i) k += m.fanout[m.in_list[t][i]][hop];
        per_node = std::max(per_node, k);
    }
    return per_node;
}

void het_bounds(const ag_hetero_sampler *s, uint64_t n_seeds, uint64_t *nodes, uint64_t *edges, uint64_t *hop_edges,
                uint64_t *frontier) {
    const HeteroMeta &m = s->meta;
    uint64_t total = 0;
    for (uint32_t t = 0; t < m.nt; ++t) total += m.type_nodes[t];
    uint64_t f = std::min<uint64_t>(n_seeds, total), n = f, e = 0, mhe = 0, mf = f;
    for (uint32_t h = 0; h < m.num_hops; ++h) {
        const uint64_t he = f * het_per_node(m, h);
        e += he; mhe = std::max(mhe, he);
        f = std::min<uint64_t>(he, total);
        if (h + 1 < m.num_hops) mf = std::max(mf, f);
        n += f;
    }
    if (nodes) *nodes = std::min<uint64_t>(n, total);
    if (edges) *edges = e;
    if (hop_edges) *hop_edges = mhe;
    if (frontier) *frontier = mf;
}

void het_free_scratch(ag_hetero_sampler *s) {
    void *ptrs[] = {s->table, s->slot_of_seed, s->slot_of_edge, s->node_key, s->node_rank, s->edge_exp, s->edge_rank,
                    s->class_tiles, s->seeds_dev, s->node_tag, s->edge_tag, s->frontier, s->tiles};
    for (void *p : ptrs) cudaFree(p);
    if (s->seeds_pinned) cudaFreeHost(s->seeds_pinned);
    s->table = nullptr; s->slot_of_seed = s->slot_of_edge = s->node_key = s->node_rank = s->edge_exp = s->edge_rank = nullptr;
    s->class_tiles = s->seeds_dev = nullptr; s->node_tag = s->edge_tag = nullptr; s->frontier = nullptr; s->tiles = nullptr;
    s->seeds_pinned = nullptr;
}

// A finished continuing batch moves the handle's stream on by the draws it consumed.
void het_account(ag_hetero_sampler *s) {
    if (s->pending_pos) s->stream_pos += s->counts_host[0].draws;
    s->pending_pos = false;
}

// Scratch for `group` batches of up to n_seeds seeds each.
int32_t het_ensure(ag_hetero_sampler *s, uint64_t n_seeds) {
    if (n_seeds <= s->cap_seeds && s->table) return AG_OK;
    if (s->in_flight) { AG_CUDA(cudaEventSynchronize(s->done)); s->in_flight = false; het_account(s); }
    het_free_scratch(s);
    s->cap_seeds = 0;
    const uint64_t cap = std::max<uint64_t>(n_seeds, 1), G = s->group;
    het_bounds(s, cap, &s->max_nodes, &s->max_edges, &s->max_hop_edges, &s->max_frontier);
    if (s->max_nodes >= kMaxPos || s->max_hop_edges >= kMaxPos || cap >= kMaxPos || s->max_edges >= 0xFFFFFFFFull)
        return fail(AG_ERR_VALUE, "batch too large: %llu seeds with these fanouts can reach %llu nodes and %llu edges in a hop "
                    "(limit %llu each)", (unsigned long long)n_seeds, (unsigned long long)s->max_nodes,
                    (unsigned long long)s->max_hop_edges, (unsigned long long)kMaxPos - 1);
    const uint64_t cn = std::max<uint64_t>(s->max_nodes, 1), ce = std::max<uint64_t>(s->max_edges, 1);
    s->table_cap = std::max<uint64_t>(1024, next_pow2(2 * s->max_nodes));
    AG_CUDA(cudaMalloc(&s->table, G * s->table_cap * 8));
    AG_CUDA(cudaMalloc(&s->slot_of_seed, G * cap * 4));
    AG_CUDA(cudaMalloc(&s->slot_of_edge, G * ce * 4));
    AG_CUDA(cudaMalloc(&s->node_key, G * cn * 4));
    AG_CUDA(cudaMalloc(&s->node_rank, G * cn * 4));
    AG_CUDA(cudaMalloc(&s->node_tag, G * cn));
    AG_CUDA(cudaMalloc(&s->edge_exp, G * ce * 4));
    AG_CUDA(cudaMalloc(&s->edge_rank, G * ce * 4));
    AG_CUDA(cudaMalloc(&s->edge_tag, G * ce));
    AG_CUDA(cudaMalloc(&s->frontier, G * std::max<uint64_t>(s->max_frontier, 1) * sizeof(FrontierEntry)));
    s->n_tiles = std::max<uint64_t>(std::max(cap, s->max_hop_edges) / kTile + 2, 2);
    AG_CUDA(cudaMalloc(&s->tiles, G * s->n_tiles * sizeof(TileDesc)));
    AG_CUDA(cudaMemset(s->tiles, 0, G * s->n_tiles * sizeof(TileDesc)));
    s->class_tiles_n = std::max(cn, ce) / kClassTile + 2;
    AG_CUDA(cudaMalloc(&s->class_tiles, G * s->class_tiles_n * kDescWords * 4));
    AG_CUDA(cudaMemset(s->class_tiles, 0, G * s->class_tiles_n * kDescWords * 4));
    AG_CUDA(cudaMalloc(&s->seeds_dev, G * cap * 4));
    AG_CUDA(cudaHostAlloc(&s->seeds_pinned, G * cap * 4, cudaHostAllocDefault));
    s->cap_seeds = cap; s->epoch = 0; s->class_epoch = 0; s->dirty = true;
    return AG_OK;
}

}  // namespace

extern "C" void ag_hetero_sampler_free(ag_hetero_sampler *s) {
    if (!s) return;
    DeviceGuard guard(s->device);
    if (s->in_flight && s->done) cudaEventSynchronize(s->done);
    het_free_scratch(s);
    cudaFree(s->meta_dev); cudaFree(s->state); cudaFree(s->counts_dev); cudaFree(s->class_misc);
    cudaFree(s->params_dev); cudaFree(s->gather_dev);
    if (s->params_host) cudaFreeHost(s->params_host);
    if (s->gather_host) cudaFreeHost(s->gather_host);
    if (s->counts_host) cudaFreeHost(s->counts_host);
    if (s->done) cudaEventDestroy(s->done);
    delete s;
}

// fanout: [num_edge_types][num_hops] row-major (hetero_sampler.rs:32-33; the
// Python mapping fills zeros for edge types left out, aethergraph-py/src/hetero.rs:309-328).
extern "C" int32_t ag_hetero_sampler_create_group(const ag_hetero_graph *h, const uint32_t *fanout, uint32_t num_hops,
                                                  int32_t replace, uint64_t seed, int32_t rng_mode, uint32_t group,
                                                  ag_hetero_sampler **out) {
    if (!h || !fanout || !out) return fail(AG_ERR_VALUE, "ag_hetero_sampler_create: null argument");
    if (num_hops == 0 || num_hops > AG_MAX_HOPS)
        return fail(AG_ERR_VALUE, "between 1 and %d hops are supported (got %u)", AG_MAX_HOPS, num_hops);
    if (group == 0 || group > 64) return fail(AG_ERR_VALUE, "group size must be between 1 and 64 (got %u)", group);
    if (rng_mode != AG_RNG_WYRAND_EXACT && rng_mode != AG_RNG_PHILOX) return fail(AG_ERR_VALUE, "unknown rng_mode %d", rng_mode);
    for (uint32_t e = 0; e < h->et; ++e)
        for (uint32_t k = 0; k < num_hops; ++k)
            if (fanout[e * num_hops + k] > 32)
                return fail(AG_ERR_VALUE, "heterogeneous sampling supports a fanout of at most 32 per edge type and hop "
                            "(edge type %u, hop %u asks %u)", e, k, fanout[e * num_hops + k]);
    DeviceGuard guard(h->device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_hetero_sampler *s = new ag_hetero_sampler();
    s->g = h; s->device = h->device; s->seed = seed; s->group = group;
    HeteroMeta &m = s->meta;
    m.nt = h->nt; m.et = h->et; m.num_hops = num_hops; m.replace = replace ? 1 : 0; m.rng_mode = rng_mode;
    uint32_t base = 0;
    for (uint32_t t = 0; t < h->nt; ++t) { m.type_base[t] = base; m.type_nodes[t] = h->num_nodes[t]; base += (uint32_t)h->num_nodes[t]; }
    for (uint32_t t = h->nt; t <= (uint32_t)kMaxNT; ++t) m.type_base[t] = base;
    for (uint32_t e = 0; e < h->et; ++e) {
        m.in_offsets[e] = h->in_offsets[e]; m.in_sources[e] = h->in_sources[e]; m.in_edges[e] = h->num_edges[e];
        m.src_type[e] = (uint8_t)h->src_type[e]; m.dst_type[e] = (uint8_t)h->dst_type[e];
        for (uint32_t k = 0; k < num_hops; ++k) m.fanout[e][k] = fanout[e * num_hops + k];
        const uint32_t t = h->dst_type[e];  // ascending edge type id (graph/hetero.rs:396-403)
        m.in_list[t][m.in_count[t]++] = (uint8_t)e;
    }
    int32_t st = AG_OK;
    do {
        const size_t G = group;
        if (cudaMalloc(&s->meta_dev, sizeof(HeteroMeta)) != cudaSuccess ||
            cudaMemcpy(s->meta_dev, &m, sizeof(HeteroMeta), cudaMemcpyHostToDevice) != cudaSuccess ||
            cudaMalloc(&s->state, G * sizeof(BatchState)) != cudaSuccess ||
            cudaMemset(s->state, 0, G * sizeof(BatchState)) != cudaSuccess ||
            cudaMalloc(&s->counts_dev, G * sizeof(ag_hetero_counts)) != cudaSuccess ||
            cudaMalloc(&s->class_misc, G * kMiscWords * 4) != cudaSuccess ||
            cudaMemset(s->class_misc, 0, G * kMiscWords * 4) != cudaSuccess ||
            cudaMalloc(&s->params_dev, G * sizeof(HParams)) != cudaSuccess ||
            cudaMalloc(&s->gather_dev, G * kMaxNT * sizeof(GatherArgs)) != cudaSuccess ||
            cudaHostAlloc(&s->params_host, G * sizeof(HParams), cudaHostAllocDefault) != cudaSuccess ||
            cudaHostAlloc(&s->gather_host, G * kMaxNT * sizeof(GatherArgs), cudaHostAllocDefault) != cudaSuccess ||
            cudaHostAlloc(&s->counts_host, G * sizeof(ag_hetero_counts), cudaHostAllocDefault) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->done, cudaEventDisableTiming) != cudaSuccess) {
            st = fail(AG_ERR_CUDA, "hetero sampler allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        st = het_ensure(s, 1024);
    } while (0);
    if (st != AG_OK) { ag_hetero_sampler_free(s); return st; }
    *out = s;
    return AG_OK;
}

extern "C" int32_t ag_hetero_sampler_create(const ag_hetero_graph *h, const uint32_t *fanout, uint32_t num_hops,
                                            int32_t replace, uint64_t seed, int32_t rng_mode, ag_hetero_sampler **out) {
    return ag_hetero_sampler_create_group(h, fanout, num_hops, replace, seed, rng_mode, 1, out);
}

extern "C" int32_t ag_hetero_sampler_reseed(ag_hetero_sampler *s, uint64_t seed) {
    if (!s) return fail(AG_ERR_VALUE, "ag_hetero_sampler_reseed: null sampler");
    if (s->in_flight) { DeviceGuard guard(s->device); cudaEventSynchronize(s->done); }
    s->seed = seed; s->stream_pos = 0; s->pending_pos = false;
    return AG_OK;
}

extern "C" int32_t ag_hetero_sampler_bounds(const ag_hetero_sampler *s, uint64_t n_seeds, uint64_t *max_nodes, uint64_t *max_edges) {
    if (!s) return fail(AG_ERR_VALUE, "ag_hetero_sampler_bounds: null sampler");
    het_bounds(s, n_seeds, max_nodes, max_edges, nullptr, nullptr);
    return AG_OK;
}

// One launch chain for a group of batches rooted at the same node type.  With
// batch_seeds, batch b starts its own RNG stream at draw 0 of batch_seeds[b]
// (the loader's per-batch reseed, prefetch.rs:1003-1005); without (single batch
// only) the handle's stream continues.  feats: NULL, or one feature store per
// node type (entries may be NULL); node type t's rows are gathered into
// bufs[b].x[t] in the order of its `nodes` segment.
namespace {
int32_t hetero_group_into(ag_hetero_sampler *s, uint32_t n_batches, uint32_t seed_type, const uint32_t *const *seeds,
                          const uint64_t *n_seeds, const uint64_t *batch_seeds, const ag_features *const *feats,
                          ag_hetero_buffers *bufs, void *stream);
}  // namespace

// A failure after the first kernel of the chain was queued leaves work running on the
// stream: wait for it and mark the handle's device state unknown, so the next call
// clears it instead of reusing staging buffers and table generations under it.
extern "C" int32_t ag_hetero_sample_group_into(ag_hetero_sampler *s, uint32_t n_batches, uint32_t seed_type,
                                               const uint32_t *const *seeds, const uint64_t *n_seeds,
                                               const uint64_t *batch_seeds, const ag_features *const *feats,
                                               ag_hetero_buffers *bufs, void *stream) {
    const int32_t st = hetero_group_into(s, n_batches, seed_type, seeds, n_seeds, batch_seeds, feats, bufs, stream);
    if (st != AG_OK && s && !s->in_flight) {
        const std::string msg = ag_last_error();
        DeviceGuard guard(s->device);
        cudaStreamSynchronize((cudaStream_t)stream);
        cudaDeviceSynchronize();
        cudaGetLastError();
        s->dirty = true;
        s->pending_pos = false;
        set_error("%s", msg.c_str());
    }
    return st;
}

namespace {
int32_t hetero_group_into(ag_hetero_sampler *s, uint32_t n_batches, uint32_t seed_type, const uint32_t *const *seeds,
                          const uint64_t *n_seeds, const uint64_t *batch_seeds, const ag_features *const *feats,
                          ag_hetero_buffers *bufs, void *stream) {
    if (!s || !bufs || !seeds || !n_seeds) return fail(AG_ERR_VALUE, "ag_hetero_sample_group_into: null argument");
    if (n_batches == 0 || n_batches > s->group)
        return fail(AG_ERR_VALUE, "group of %u batches does not fit a sampler created for %u", n_batches, s->group);
    if (!batch_seeds && n_batches > 1) return fail(AG_ERR_VALUE, "a group of several batches needs batch_seeds");
    const HeteroMeta &m = s->meta;
    if (seed_type >= m.nt) return fail(AG_ERR_VALUE, "unknown seed node type %u", seed_type);
    uint64_t max_n = 0;
    for (uint32_t b = 0; b < n_batches; ++b) {
        const ag_hetero_buffers &B = bufs[b];
        if (!seeds[b] && n_seeds[b]) return fail(AG_ERR_VALUE, "ag_hetero_sample_group_into: null seeds");
        if (!B.nodes || !B.edge_src_local || !B.edge_dst_local || !B.seed_indices)
            return fail(AG_ERR_VALUE, "nodes, edge_src_local, edge_dst_local and seed_indices buffers are required");
        if (B.cap_seeds < n_seeds[b]) return fail(AG_ERR_VALUE, "seed_indices capacity %llu < %llu seeds",
                                                  (unsigned long long)B.cap_seeds, (unsigned long long)n_seeds[b]);
        // Seeds are checked against the seed type's node count (hetero_sampler.rs:174-187).
        for (uint64_t i = 0; i < n_seeds[b]; ++i)
            if ((uint64_t)seeds[b][i] >= m.type_nodes[seed_type])
                return fail(AG_ERR_SAMPLING, "seed node %u (position %llu) is out of range for %llu nodes",
                            seeds[b][i], (unsigned long long)i, (unsigned long long)m.type_nodes[seed_type]);
        max_n = std::max(max_n, n_seeds[b]);
    }
    if (feats)
        for (uint32_t t = 0; t < m.nt; ++t)
            if (feats[t]) {
                if (feats[t]->device != s->device) return fail(AG_ERR_VALUE, "feature store of node type %u lives on another device", t);
                if (feats[t]->num_nodes < m.type_nodes[t]) return fail(AG_ERR_VALUE, "feature store of node type %u has too few rows", t);
                if (feats[t]->row_stride != 1 && !feats[t]->shards) return fail(AG_ERR_VALUE, "a cyclic feature shard is read through a sharded view");
            }
    DeviceGuard guard(s->device);
    if (!guard.ok) return AG_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    if (s->in_flight) { AG_CUDA(cudaEventSynchronize(s->done)); s->in_flight = false; het_account(s); }
    AG_TRY(het_ensure(s, max_n));
    const uint64_t G = s->group;
    if (s->dirty || s->gen >= kGens) { AG_CUDA(cudaMemsetAsync(s->table, 0xFF, G * s->table_cap * 8, st)); s->gen = 0; }
    if (s->dirty) { AG_CUDA(cudaMemsetAsync(s->state, 0, G * sizeof(BatchState), st)); s->dirty = false; }
    const uint32_t H = m.num_hops;
    if (s->epoch + (H + 2) > 0x3FFFFF00u) { AG_CUDA(cudaMemsetAsync(s->tiles, 0, G * s->n_tiles * sizeof(TileDesc), st)); s->epoch = 0; }
    if (s->class_epoch + 4 > 0x3FFFFF00u) {
        AG_CUDA(cudaMemsetAsync(s->class_tiles, 0, G * s->class_tiles_n * kDescWords * 4, st));
        s->class_epoch = 0;
    }
    uint32_t log2cap = 0;
    while ((1ull << log2cap) < s->table_cap) ++log2cap;
    const uint64_t cn = std::max<uint64_t>(s->max_nodes, 1), ce = std::max<uint64_t>(s->max_edges, 1);
    const uint64_t fcap = std::max<uint64_t>(s->max_frontier, 1);
    bool want_x = false;
    for (uint32_t b = 0; b < n_batches; ++b) {
        const ag_hetero_buffers &B = bufs[b];
        const uint32_t n = (uint32_t)n_seeds[b];
        HParams p{};
        p.meta = s->meta_dev;
        p.table = DedupTable{s->table + b * s->table_cap, (uint32_t)(s->table_cap - 1), 32u - log2cap, s->gen};
        p.state = s->state + b; p.tiles = s->tiles + b * s->n_tiles; p.epoch_base = s->epoch + 1;
        p.n_seeds = n; p.seed_type = seed_type;
        if (n) memcpy(s->seeds_pinned + b * s->cap_seeds, seeds[b], (size_t)n * 4);
        p.seeds = s->seeds_dev + b * s->cap_seeds;
        p.seed = batch_seeds ? batch_seeds[b] : s->seed;
        p.start_draw = batch_seeds ? 0ull : s->stream_pos;
        p.slot_of_seed = s->slot_of_seed + b * s->cap_seeds; p.slot_of_edge = s->slot_of_edge + b * ce;
        p.frontier = s->frontier + b * fcap; p.frontier_cap = fcap;
        p.node_key = s->node_key + b * cn; p.node_tag = s->node_tag + b * cn; p.node_rank = s->node_rank + b * cn;
        p.edge_exp = s->edge_exp + b * ce; p.edge_tag = s->edge_tag + b * ce; p.edge_rank = s->edge_rank + b * ce;
        p.cap_nodes = std::min<uint64_t>(B.cap_nodes, cn);
        p.cap_edges = std::min<uint64_t>(B.cap_edges, ce);
        p.class_tiles = s->class_tiles + b * s->class_tiles_n * kDescWords;
        p.class_epoch = s->class_epoch + 1;
        uint32_t *misc = s->class_misc + b * kMiscWords;
        p.type_count = misc; p.et_count = misc + kChan; p.type_start = misc + 2 * kChan; p.class_ticket = misc + 3 * kChan;
        p.nodes = B.nodes; p.edge_src_local = B.edge_src_local; p.edge_dst_local = B.edge_dst_local;
        p.seed_indices = B.seed_indices; p.n_id = B.n_id; p.edge_index_local = B.edge_index_local;
        p.seed_index = B.seed_index; p.counts = s->counts_dev + b;
        s->params_host[b] = p;
        for (uint32_t t = 0; t < m.nt; ++t) {
            GatherArgs ga{};
            if (feats && feats[t] && B.x[t]) {
                set_gather_source(ga, feats[t]);
                ga.ids = B.nodes; ga.ids64 = 0; ga.ids_off = p.type_start + t;
                ga.n = std::min<uint64_t>(p.cap_nodes, m.type_nodes[t]);
                if (B.cap_x[t]) ga.n = std::min<uint64_t>(ga.n, B.cap_x[t]);
                ga.n_dev = p.type_count + t;
                ga.out = B.x[t];
                want_x = true;
            }
            s->gather_host[(size_t)t * G + b] = ga;
        }
    }
    s->pending_pos = (batch_seeds == nullptr);
    s->epoch += H + 2; s->class_epoch += 2; s->gen += 1; s->last_batches = n_batches;
    AG_CUDA(cudaMemcpyAsync(s->seeds_dev, s->seeds_pinned, (uint64_t)n_batches * s->cap_seeds * 4, cudaMemcpyHostToDevice, st));
    AG_CUDA(cudaMemcpyAsync(s->params_dev, s->params_host, n_batches * sizeof(HParams), cudaMemcpyHostToDevice, st));
    if (want_x) AG_CUDA(cudaMemcpyAsync(s->gather_dev, s->gather_host, G * kMaxNT * sizeof(GatherArgs), cudaMemcpyHostToDevice, st));

    const HParams *pa = s->params_dev;
    const uint32_t nmax = (uint32_t)max_n, nb = n_batches;
    auto tiles_for = [&](uint64_t items) {
        return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((items + kTile - 1) / kTile, std::max<uint64_t>(1, (uint64_t)kSMs * 8 / nb)));
    };
    if (nmax) k_het_insert_seeds<<<dim3((nmax + 255) / 256, nb), 256, 0, st>>>(pa);
    uint64_t f_bound = nmax, items = nmax;
    for (uint32_t stage = 0; stage <= H; ++stage) {
        const bool has_next = stage < H;
        k_het_assign<<<dim3(tiles_for(items), nb), kTile, 0, st>>>(pa, stage, has_next ? 1 : 0);
        if (has_next) {
            const uint32_t blocks = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((f_bound * 32 + kPickThreads - 1) / kPickThreads,
                                                                                      std::max<uint64_t>(1, (uint64_t)kSMs * 16 / nb)));
            k_het_pick<<<dim3(blocks, nb), kPickThreads, 0, st>>>(pa, stage);
            items = f_bound * het_per_node(m, stage);
            f_bound = std::min<uint64_t>(items, s->max_nodes);
        }
    }
    auto ctiles_for = [&](uint64_t n) {
        return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((n + kClassTile - 1) / kClassTile, std::max<uint64_t>(1, (uint64_t)kSMs * 4 / nb)));
    };
    k_class_rank<<<dim3(ctiles_for(s->max_nodes), nb), kClassThreads, 0, st>>>(pa, 0);
    k_class_rank<<<dim3(ctiles_for(s->max_edges), nb), kClassThreads, 0, st>>>(pa, 1);
    {
        const uint64_t work = std::max<uint64_t>(std::max(s->max_edges, s->max_nodes), std::max<uint64_t>(nmax, 1));
        const uint32_t fx = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((work + 255) / 256, std::max<uint64_t>(1, (uint64_t)kSMs * 8 / nb)));
        k_het_scatter<<<dim3(fx, nb), 256, 0, st>>>(pa);
    }
    AG_CUDA(cudaGetLastError());
    if (want_x) {
        for (uint32_t t = 0; t < m.nt; ++t) {
            if (!feats[t]) continue;
            bool any = false, aligned = ((uintptr_t)feats[t]->payload % 16) == 0;
            for (uint32_t b = 0; b < nb; ++b)
                if (bufs[b].x[t]) { any = true; aligned = aligned && ((uintptr_t)bufs[b].x[t] % 16) == 0; }
            if (!any) continue;
            const uint64_t bound = std::min<uint64_t>(s->max_nodes, m.type_nodes[t]);
            AG_CUDA(launch_gather_group(s->gather_dev + (size_t)t * G, nb, (uint32_t)(feats[t]->dim * elem_size(feats[t]->dtype)),
                                        (uint32_t)feats[t]->dim, std::max<uint64_t>(bound / 4, 1), aligned, feats[t]->dtype,
                                        feats[t]->shards != nullptr, st));
        }
    }
    AG_CUDA(cudaMemcpyAsync(s->counts_host, s->counts_dev, nb * sizeof(ag_hetero_counts), cudaMemcpyDeviceToHost, st));
    AG_CUDA(cudaEventRecord(s->done, st));
    s->in_flight = true;
    return AG_OK;
}
}  // namespace

extern "C" int32_t ag_hetero_sample_group_wait(ag_hetero_sampler *s, ag_hetero_counts *counts, int32_t *statuses) {
    if (!s) return fail(AG_ERR_VALUE, "ag_hetero_sample_group_wait: null sampler");
    if (!s->in_flight) return fail(AG_ERR_VALUE, "ag_hetero_sample_group_wait: no batch in flight");
    DeviceGuard guard(s->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const cudaError_t e = cudaEventSynchronize(s->done);
    s->in_flight = false;
    if (e != cudaSuccess) { s->dirty = true; s->pending_pos = false; return fail(AG_ERR_CUDA, "hetero sampling kernels failed: %s", cudaGetErrorString(e)); }
    het_account(s);
    int32_t first = AG_OK;
    for (uint32_t b = 0; b < s->last_batches; ++b) {
        const ag_hetero_counts c = s->counts_host[b];
        if (counts) counts[b] = c;
        int32_t st = AG_OK;
        if (c.error & (kErrSpinTimeout | kErrTableFull)) s->dirty = true;
        if (c.error & kErrBadSeed) st = fail(AG_ERR_SAMPLING, "a seed node is out of range for its node type");
        else if (c.error & kErrCapacity) st = fail(AG_ERR_VALUE, "output buffers too small for the sampled subgraph");
        else if (c.error & kErrBadId) st = fail(AG_ERR_VALUE, "a gathered node id is outside its feature store");
        else if (c.error) st = fail(AG_ERR_WORKER, "hetero sampler kernels reported error bits 0x%x", c.error);
        if (statuses) statuses[b] = st;
        if (st != AG_OK && first == AG_OK) first = st;
    }
    return first;
}

extern "C" int32_t ag_hetero_sample_into(ag_hetero_sampler *s, uint32_t seed_type, const uint32_t *seeds, uint64_t n_seeds,
                                         ag_hetero_buffers *buf, void *stream) {
    return ag_hetero_sample_group_into(s, 1, seed_type, &seeds, &n_seeds, nullptr, nullptr, buf, stream);
}

extern "C" int32_t ag_hetero_sample_wait(ag_hetero_sampler *s, ag_hetero_counts *counts) {
    return ag_hetero_sample_group_wait(s, counts, nullptr);
}

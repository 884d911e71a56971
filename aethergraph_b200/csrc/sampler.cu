// Homogeneous k-hop neighbor sampler with frontier dedup and relabel.
//
// Computes exactly what the reference's NeighborSampler::sample computes
// (crates/aethergraph-core/src/loader/sampler.rs:845-961 with the hop loop at
// :754-842 and the per-node dispatch at :1178-1235), but as a short chain of
// data-parallel kernels instead of one sequential loop.  A batch with H hops
// is 2H + 2 launches:
//
//   insert_seeds   every seed is inserted into a hash table keyed by vertex id
//                  with atomicMin(position): the smallest position that names a
//                  vertex is its first sighting.
//   assign(s)      s = 0 .. H.  The items of stage s are the seeds (s = 0) or
//                  the edges hop s - 1 emitted, in position order.  One
//                  single-pass scan over them turns the first-sighting flags
//                  into local ids (= discovery order, exactly the order the
//                  sequential reference assigns them in) and appends the new
//                  vertices to `nodes`; the same scan carries how many edges and
//                  how many RNG draws each new vertex needs at hop s, so the new
//                  vertices leave the kernel as a frontier with their row
//                  bounds, edge slots and draw offsets attached.
//   pick(s)        s = 0 .. H - 1.  A group of lanes per frontier vertex
//                  reproduces the reference's choice of row positions — take-all
//                  (:1312-1328), Floyd (:1332-1380), with replacement
//                  (:1289-1308) or the weighted Efraimidis-Spirakis keys
//                  (:1418-1469) — writes the edges of hop s at their scanned
//                  slots and inserts the destinations into the table as the
//                  items of stage s + 1.
//                  Every item also learns its vertex's final local id here (its own
//                  if it is the first sighting, else the one the first sighting got,
//                  for which it may have to wait a moment), so dst_local / seed_locals
//                  and the int64 views the Python API exposes are written by the same
//                  kernel; the block that finishes last in the last stage writes the
//                  batch's counts.
//
// The reference draws from one sequential WyRand stream per batch.  WyRand's
// state is an additive counter, so draw d is a pure function of (seed, d); the
// scan of per-vertex draw counts gives every vertex the index of its first
// draw, and the parallel picks are bit-identical to the sequential ones.
//
// Batches are independent, so one launch chain serves a whole GROUP of them:
// every kernel's grid has the batch as its y dimension and each batch brings
// its own parameter block, dedup table, scan descriptors and output buffers.
// A group of 16 batches of 1024 seeds costs the same few launches as one.
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include <sched.h>

#include "common.cuh"
#include "internal.h"
#include "sampler.cuh"

namespace ag {

namespace {

constexpr int kTile = 512;      // threads per block of the assign kernel
// Items per thread of the assign kernel.  The last stage holds no row bounds per item,
// so it can afford twice as many table probes in flight per thread.
template <bool HAS_NEXT> struct AssignShape { static constexpr int kIPT = HAS_NEXT ? 4 : 8; static constexpr int kTileItems = kTile * kIPT; };
constexpr int kPickThreads = 256;
constexpr int kLargeK = 1024;   // largest fanout the k > 32 path keeps in shared memory

enum : int { kModeUniform = 0, kModeReplace = 1, kModeWeighted = 2, kModeWeightedReplace = 3 };
enum : int { kPickSmall = 0, kPickLarge = 1, kPickWeighted = 2 };

// Parameter block of one batch; a group's blocks sit in one device array that
// the kernels index with blockIdx.y.
struct SampleParams {
    const uint64_t *offsets;
    const uint32_t *dst;
    const float *weights;
    uint64_t num_nodes, num_edges;
    DedupTable table;
    BatchState *state;
    TileDesc *tiles;
    uint32_t epoch_base;  // stage s scans under epoch_base + s
    uint32_t n_seeds;
    const uint32_t *seeds;
    uint64_t seed;
    int rng_mode;
    int mode;
    uint64_t start_draw;  // absolute index of the batch's first RNG draw (0 for a freshly seeded batch)
    uint32_t num_hops;
    // outputs
    uint32_t *nodes;
    uint32_t *edge_src, *edge_dst, *src_local, *dst_local, *seed_locals;
    uint64_t *edge_ids;
    uint64_t cap_nodes, cap_edges;
    int64_t *n_id, *edge_index_local, *e_id, *seed_index;
    ag_sample_counts *counts;
    // scratch
    uint32_t *slot_of_seed;
    uint32_t *slot_of_edge;
    FrontierEntry *frontier;
    uint64_t frontier_cap;
    uint32_t *hub_list;   // weighted only: frontier positions of the rows left to k_pick_hubs
    uint32_t *hub_count;
};

// Row bounds with the reference's guard (graph/csr.rs:318-335): an inverted
// pair or one past num_edges is an empty row.
__device__ __forceinline__ void row_bounds(const uint64_t *offsets, uint64_t num_nodes,
                                           uint64_t num_edges, uint32_t id, uint64_t &off,
                                           uint64_t &deg) {
    off = 0; deg = 0;
    if ((uint64_t)id >= num_nodes) return;
    const uint64_t a = __ldg(offsets + id), b = __ldg(offsets + id + 1);
    if (a > b || b > num_edges) return;
    off = a; deg = b - a;
}

// How many edges and draws a row of `deg` asks for at fanout k
// (sampler.rs:1226-1233 uniform, :1289-1308 replace, :1427-1457 weighted).
__device__ __forceinline__ void row_demand(int mode, uint64_t deg, uint32_t k, uint32_t &take,
                                           uint64_t &draws) {
    take = 0; draws = 0;
    if (deg == 0 || k == 0) return;
    if (mode == kModeReplace || mode == kModeWeightedReplace) { take = k; draws = k; return; }
    if ((uint64_t)k >= deg) { take = (uint32_t)deg; return; }
    take = k;
    draws = (mode == kModeWeighted) ? deg : (uint64_t)k;
}

// ------------------------------------------------------------ seed insert --
// Programmatic dependent launch: the kernels of a chain are launched with
// cudaLaunchAttributeProgrammaticStreamSerialization, so the next kernel's blocks
// are scheduled as this one's blocks exit, without waiting for the grid's
// completion to be reported first.  Every kernel starts by waiting for its
// predecessor's results (griddepcontrol.wait; a no-op for a plain launch).  The
// kernels do NOT release their successor early (no griddepcontrol.launch_dependents
// before the work): measured, successor blocks parked in SM slots take those slots
// from the gather of a neighbouring chain and the whole pipeline gets slower.
__device__ __forceinline__ void chain_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__global__ void k_insert_seeds(const SampleParams *__restrict__ pa) {
    chain_sync();
    const SampleParams &p = pa[blockIdx.y];
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.n_seeds) return;
    const uint32_t id = p.seeds[i];
    if ((uint64_t)id >= p.num_nodes) {
        atomicOr(&p.state->error, kErrBadSeed);
        p.slot_of_seed[i] = 0xFFFFFFFFu;
        return;
    }
    p.slot_of_seed[i] = table_insert_min(p.table, id, enc_pending(p.table.gen, 0, i), &p.state->error);
}

// ----------------------------------------------------------------- expand --
__device__ __forceinline__ uint32_t draw_u32(const SampleParams &p, uint32_t hop, uint32_t vertex,
                                             uint64_t dbase, uint32_t slot) {
    if (p.rng_mode == AG_RNG_PHILOX) return philox_u32(p.seed, hop, vertex, slot);
    return (uint32_t)wyrand_at(p.seed, dbase + slot);  // next_u32: genstamp.rs:199-201
}

// Edge t of vertex fe at hop `hop` (= item fe.ebase + t of stage hop + 1), its
// destination d already loaded from CSR position pos.
__device__ __forceinline__ void emit_edge_loaded(const SampleParams &p, uint32_t hop, uint32_t edges_before,
                                                 const FrontierEntry &fe, uint32_t t, uint64_t pos, uint32_t d) {
    const uint32_t e_rel = fe.ebase + t;
    const uint64_t e = (uint64_t)edges_before + e_rel;
    if (e >= p.cap_edges || e_rel >= kMaxPos) { atomicOr(&p.state->error, kErrCapacity); return; }
    if (p.edge_src) p.edge_src[e] = fe.id;
    p.edge_dst[e] = d;
    if (p.edge_ids) p.edge_ids[e] = pos;
    if (p.e_id && p.edge_ids) p.e_id[e] = (int64_t)pos;
    p.src_local[e] = fe.local;
    if ((uint64_t)d >= p.num_nodes) {
        // Only reachable on a graph that skipped validation; the reference drops
        // such an edge (sampler.rs:736-739), which a slot-scanned layout cannot.
        atomicOr(&p.state->error, kErrBadDst);
        p.slot_of_edge[e] = 0xFFFFFFFFu;
        return;
    }
    p.slot_of_edge[e] = table_insert_min(p.table, d, enc_pending(p.table.gen, hop + 1, e_rel), &p.state->error);
}

__device__ __forceinline__ void emit_edge(const SampleParams &p, uint32_t hop, uint32_t edges_before,
                                          const FrontierEntry &fe, uint32_t t, uint64_t pos) {
    const uint32_t e_rel = fe.ebase + t;
    if ((uint64_t)edges_before + e_rel >= p.cap_edges || e_rel >= kMaxPos) { atomicOr(&p.state->error, kErrCapacity); return; }
    emit_edge_loaded(p, hop, edges_before, fe, t, pos, ld_stream_u32(p.dst + pos));
}

__device__ __forceinline__ bool key_less(double ka, uint32_t pa, double kb, uint32_t pb) {
    return ka < kb || (ka == kb && pa < pb);
}

// Fanout <= G <= 32: G lanes per vertex, lane t owns edge slot t.  A lane group works
// on two vertices per round, so the two destination loads (random sectors of the CSR)
// and the table probes behind them are in flight together.
template <int G>
__device__ __forceinline__ void pick_small(const SampleParams &p, uint32_t hop, uint32_t k, uint32_t edges_before,
                                           const FrontierEntry *fes, uint32_t n) {
    constexpr int U = 2;
    const uint32_t t = threadIdx.x % G;
    const uint32_t gshift = (threadIdx.x & 31) & ~(G - 1);
    const uint32_t gmask = (G == 32) ? 0xffffffffu : ((1u << G) - 1u);
    constexpr uint32_t kPerBlock = kPickThreads / G;
    // Grid-stride over the frontier; the loop bound is block-uniform.
    for (uint32_t base = blockIdx.x * kPerBlock * U; base < n; base += gridDim.x * kPerBlock * U) {
        FrontierEntry fe[U];
        uint32_t pick[U];
        bool emit[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t j = base + u * kPerBlock + threadIdx.x / G;
            const bool active = j < n;
            fe[u] = FrontierEntry{};
            if (active) fe[u] = fes[j];
            const uint32_t deg = fe[u].deg;
            const bool sampled = active && p.mode != kModeReplace && deg > k;  // Floyd row
            pick[u] = t;                                                         // take-all: row order
            uint32_t ip = 0;
            if (active && p.mode == kModeReplace && deg > 0 && t < k) {
                // sampler.rs:1298-1300: k independent draws over the whole row
                pick[u] = (uint32_t)(((uint64_t)draw_u32(p, hop, fe[u].id, fe[u].dbase, t) * deg) >> 32);
            } else if (sampled && t < k) {
                // sampler.rs:1345-1346: i runs over deg-k .. deg-1, j = rand_below(i + 1)
                ip = deg - k + t;
                pick[u] = (uint32_t)(((uint64_t)draw_u32(p, hop, fe[u].id, fe[u].dbase, t) * ((uint64_t)ip + 1)) >> 32);
            }
            // Floyd's "already taken?" is sequential in t (sampler.rs:1347-1352):
            // resolve slot s against the finished slots below it, one ballot per s.
            if (__any_sync(0xffffffffu, sampled)) {
                for (uint32_t s = 1; s < k; ++s) {
                    const uint32_t js = __shfl_sync(0xffffffffu, pick[u], s, G);
                    const bool hit = sampled && t < s && pick[u] == js;
                    const uint32_t m = (__ballot_sync(0xffffffffu, hit) >> gshift) & gmask;
                    if (sampled && t == s && m) pick[u] = ip;
                }
            }
            uint32_t take = 0;
            uint64_t draws;
            if (active) row_demand(p.mode, deg, k, take, draws);
            emit[u] = t < take;
        }
        uint32_t d[U];
#pragma unroll
        for (int u = 0; u < U; ++u) d[u] = emit[u] ? ld_stream_u32(p.dst + fe[u].off + pick[u]) : 0u;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (emit[u]) emit_edge_loaded(p, hop, edges_before, fe[u], t, fe[u].off + pick[u], d[u]);
    }
}

// Fanout > 32: one warp per vertex (four warps per block); finished picks live
// in shared memory so later slots can be checked against all earlier ones.
__device__ __forceinline__ void pick_large(const SampleParams &p, uint32_t hop, uint32_t k, uint32_t edges_before,
                                           const FrontierEntry *fes, uint32_t n, uint32_t *s_picks) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint32_t *picks = s_picks + warp * kLargeK;
    for (uint32_t j = blockIdx.x * 4 + warp; j < n; j += gridDim.x * 4) {
        const FrontierEntry fe = fes[j];
        const uint32_t deg = fe.deg;
        uint32_t take;
        uint64_t draws;
        row_demand(p.mode, deg, k, take, draws);
        const bool sampled = p.mode != kModeReplace && deg > k;
        __syncwarp();
        for (uint32_t c = 0; c < take; c += 32) {
            const uint32_t t = c + lane;
            const bool in = t < take;
            uint32_t pick = t, ip = 0;
            bool hit_prev = false;
            if (in && p.mode == kModeReplace) {
                pick = (uint32_t)(((uint64_t)draw_u32(p, hop, fe.id, fe.dbase, t) * deg) >> 32);
            } else if (in && sampled) {
                ip = deg - k + t;
                pick = (uint32_t)(((uint64_t)draw_u32(p, hop, fe.id, fe.dbase, t) * ((uint64_t)ip + 1)) >> 32);
                for (uint32_t q = 0; q < c; ++q) hit_prev |= (picks[q] == pick);
            }
            if (sampled) {
                for (uint32_t s = 0; s < 32; ++s) {
                    const uint32_t js = __shfl_sync(0xffffffffu, pick, s);
                    const bool hit = in && (uint32_t)lane < s && pick == js;
                    const uint32_t m = __ballot_sync(0xffffffffu, hit);
                    if (in && (uint32_t)lane == s && (m || hit_prev)) pick = ip;
                }
                if (in) picks[t] = pick;
                __syncwarp();
            }
            if (in) emit_edge(p, hop, edges_before, fe, t, fe.off + pick);
        }
    }
}

// Weighted sampling without replacement, fanout <= 32, one warp per vertex.
// Selection follows sampler.rs:1418-1469: one 64-bit draw per row position in
// row order, key = -ln(u) / w in f64 with u = ((bits >> 11) + 1) * 2^-53
// (sampler.rs:52-55), +inf for a weight that is not finite and positive; the k
// smallest keys win.  The winners are emitted in ascending (key, position)
// order; the reference's own order comes from Rust's select_nth_unstable_by and
// is not defined by its source tree.  The warp streams the row 32 positions at a
// time and keeps the k best so far sorted across its lanes.
// Weighted picks (sampler.rs:1418-1469): every position of a row with deg > k gets
// the key -ln(u) / w from its own draw; the k smallest (key, position) win and are
// emitted in ascending order.  A warp streams 32 positions at a time and keeps the
// current best k sorted across its lanes.

// Inserts the chunk's candidates (one per lane, cpos == ~0 for none) that beat the
// current k-th best into the sorted lanes.
__device__ __forceinline__ void topk_insert_chunk(double key, uint32_t cpos, double &best_key, uint32_t &best_pos,
                                                  uint32_t k, int lane) {
    for (;;) {
        const double tk = __shfl_sync(0xffffffffu, best_key, k - 1);
        const uint32_t tp = __shfl_sync(0xffffffffu, best_pos, k - 1);
        const uint32_t m = __ballot_sync(0xffffffffu, cpos != 0xFFFFFFFFu && key_less(key, cpos, tk, tp));
        if (!m) break;
        const int src = __ffs(m) - 1;
        const double ck = __shfl_sync(0xffffffffu, key, src);
        const uint32_t cp = __shfl_sync(0xffffffffu, cpos, src);
        // (ck, cp) lands after every entry that is smaller, the rest shift up by one.
        const uint32_t smaller = __ballot_sync(0xffffffffu, key_less(best_key, best_pos, ck, cp));
        const int at = __popc(smaller);
        const double up_k = __shfl_up_sync(0xffffffffu, best_key, 1);
        const uint32_t up_p = __shfl_up_sync(0xffffffffu, best_pos, 1);
        if (lane == at) { best_key = ck; best_pos = cp; }
        else if (lane > at) { best_key = up_k; best_pos = up_p; }
        if (lane == src) cpos = 0xFFFFFFFFu;
    }
}

// Streams positions [begin, end) of the row of `fe` into the warp's sorted best k.
// Exact key of position `pos` of the row (sampler.rs:1440-1452): u from the position's
// own draw, key = -ln(u) / w, +inf for a weight that is not a positive finite number.
__device__ __forceinline__ double weighted_key(const SampleParams &p, uint32_t hop, const FrontierEntry &fe, uint32_t pos) {
    const uint64_t bits = (p.rng_mode == AG_RNG_PHILOX)
        ? (((uint64_t)philox_u32(p.seed, hop, fe.id, 2 * pos) << 32) | philox_u32(p.seed, hop, fe.id, 2 * pos + 1))
        : wyrand_at(p.seed, fe.dbase + pos);
    const double w = (double)__ldg(p.weights + fe.off + pos);
    if (!(isfinite(w) && w > 0.0)) return __longlong_as_double(0x7FF0000000000000ll);
    const double u = ((double)(bits >> 11) + 1.0) * (1.0 / 9007199254740992.0);
    return -log(u) / w;
}

// Streams positions [begin, end) of the row of `fe` into the warp's sorted best k.
//
// Almost every position loses against the k-th best key, and the exact key costs an
// f64 log and divide, so the stream works in two stages.  Stage 1, all lanes, single
// precision: with uf >= u (u's top 24 bits, rounded up) -ln(uf) is a LOWER bound of
// -ln(u); if even that bound, less the error of __logf (< 5e-7 absolute or relative),
// exceeds thr * w (with slack for the f32 product), the exact key cannot be below the
// threshold and the position is dropped.  Survivors are only queued (`buf`, 64 slots
// of the warp's shared memory).  Stage 2, whenever 32 are queued: every lane evaluates
// one queued position exactly and the winners are inserted.  The threshold is the k-th
// best key at the last flush (and, when several warps stream slices of one row,
// `shared_thr`, the lowest k-th best any of them holds; the bit pattern of a
// non-negative float orders like the float).  It is always an upper bound of the
// row's final k-th best key, so stage 1 only ever discards certain losers and the
// winners — and the output — are exactly those of evaluating every position.
__device__ __forceinline__ void topk_stream(const SampleParams &p, uint32_t hop, const FrontierEntry &fe, uint32_t begin,
                                            uint32_t end, uint32_t k, int lane, double &best_key, uint32_t &best_pos,
                                            uint32_t *buf, uint32_t *shared_thr = nullptr) {
    const double inf = __longlong_as_double(0x7FF0000000000000ll);
    uint32_t queued = 0;  // warp-uniform
    float thr = (float)__shfl_sync(0xffffffffu, best_key, k - 1);
    auto flush = [&](uint32_t count) {  // evaluate buf[0 .. count) exactly, one per lane, and insert the winners
        double key = inf;
        uint32_t cpos = 0xFFFFFFFFu;
        if ((uint32_t)lane < count) {
            cpos = buf[lane];
            key = weighted_key(p, hop, fe, cpos);
        }
        topk_insert_chunk(key, cpos, best_key, best_pos, k, lane);
        const double kth = __shfl_sync(0xffffffffu, best_key, k - 1);
        thr = (float)kth;
        if (shared_thr) {
            const float up = __double2float_ru(kth);  // rounded up: still an upper bound
            if (lane == 0 && up < 3.0e38f) atomicMin(shared_thr, __float_as_uint(up));
        }
    };
    for (uint32_t c = begin; c < end; c += 32) {
        const uint32_t pos = c + lane;
        float t = thr;
        if (shared_thr) t = fminf(t, __uint_as_float(*(volatile uint32_t *)shared_thr));
        bool keep = pos < end;
        if (keep && t >= 1.0e-30f) {  // a finite threshold in the normal range: no under- or overflow below
            const uint64_t bits = (p.rng_mode == AG_RNG_PHILOX)
                ? (((uint64_t)philox_u32(p.seed, hop, fe.id, 2 * pos) << 32) | philox_u32(p.seed, hop, fe.id, 2 * pos + 1))
                : wyrand_at(p.seed, fe.dbase + pos);
            const float wf = __ldg(p.weights + fe.off + pos);
            if (wf > 0.0f && wf <= 3.0e38f) {
                const float uf = (float)((uint32_t)(bits >> 40) + 1u) * 5.9604644775390625e-08f;  // 2^-24, exact
                const float lower = -__logf(uf);
                keep = !(lower * 0.999998f - 1.0e-6f > t * wf * 1.00001f + 1.0e-6f);
            }
        }
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (keep) buf[queued + __popc(m & ((1u << lane) - 1u))] = pos;
        queued += __popc(m);
        __syncwarp();
        if (queued >= 32) {
            flush(32);
            __syncwarp();
            const uint32_t rest = queued - 32;  // < 32: move the tail to the front
            const uint32_t moved = (uint32_t)lane < rest ? buf[32 + lane] : 0;
            __syncwarp();
            if ((uint32_t)lane < rest) buf[lane] = moved;
            queued = rest;
            __syncwarp();
        }
    }
    if (queued) { flush(queued); __syncwarp(); }
}

constexpr uint32_t kHubDegree = 4096;  // rows longer than this are left to k_pick_hubs (a whole block per row)
constexpr int kHubThreads = 512;

__device__ __forceinline__ void pick_weighted(const SampleParams &p, uint32_t hop, uint32_t k, uint32_t edges_before,
                                              const FrontierEntry *fes, uint32_t n, uint32_t *queue) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (k == 0) return;
    const double inf = __longlong_as_double(0x7FF0000000000000ll);
    for (uint32_t j = blockIdx.x * (kPickThreads / 32) + warp; j < n; j += gridDim.x * (kPickThreads / 32)) {
        const FrontierEntry fe = fes[j];
        const uint32_t deg = fe.deg;
        if (deg == 0) continue;
        if (k >= deg) {
            for (uint32_t t = lane; t < deg; t += 32) emit_edge(p, hop, edges_before, fe, t, fe.off + t);
            continue;
        }
        if (deg > kHubDegree && p.hub_list) {  // queue the hub for the block-per-row kernel
            if (lane == 0) p.hub_list[atomicAdd(p.hub_count, 1u)] = j;
            continue;
        }
        double best_key = inf;
        uint32_t best_pos = 0xFFFFFFFFu;  // sentinel: sorts after every real (key, position)
        topk_stream(p, hop, fe, 0, deg, k, lane, best_key, best_pos, queue + warp * 64);
        if ((uint32_t)lane < k) emit_edge(p, hop, edges_before, fe, lane, fe.off + best_pos);
    }
}

// One stage: assign local ids to the first sightings among the stage's items
// and (has_next) queue the new vertices, with their row bounds, edge slots and
// draw offsets, as the frontier the pick kernel of hop `stage` expands.  Every
// item also writes the final local id of its vertex (dst_local / seed_locals and
// the int64 views): its own if it is the first sighting, the one already in the
// table if the vertex was registered by an earlier stage, and otherwise the one
// an earlier item of this stage is about to store — a short, bounded wait that is
// taken only after the block has passed its next barrier, so a block never waits
// for a store of its own.
__device__ __forceinline__ StageInfo load_stage_cg(const StageInfo *s) {
    // other blocks of this launch wrote it: read it from L2, not from a stale L1 line
    const uint4 a = __ldcg((const uint4 *)s), b = __ldcg((const uint4 *)s + 1);
    StageInfo r;
    r.n_nodes = a.x; r.n_edges = a.y; r.frontier_n = a.z; r.hop_edges = a.w;
    r.draws = ((uint64_t)b.y << 32) | b.x; r.hop_draws = ((uint64_t)b.w << 32) | b.z;
    return r;
}

__device__ __forceinline__ void write_item_local(const SampleParams &p, uint32_t stage, uint32_t n_edges_before,
                                                 uint32_t item, uint32_t local) {
    if (stage == 0) {
        p.seed_locals[item] = local;
        if (p.seed_index) p.seed_index[item] = (int64_t)local;
    } else {
        const uint64_t e = (uint64_t)n_edges_before + item;
        if (e >= p.cap_edges) return;
        p.dst_local[e] = local;
        if (p.edge_index_local) p.edge_index_local[e] = (int64_t)local;  // row 0: sampled neighbor
    }
}

// Weighted picks with replacement (sampler.rs:1383-1412): the reference sums the row's
// weights in f64 in row order, draws u = next_u64 * (total / u64::MAX) k times and takes,
// for each draw, the first position whose running sum exceeds u.  The running sums must
// be the reference's own, rounding included, so every lane of the warp that owns the row
// adds the weights in the same row order (redundantly: the loads are warp-wide
// broadcasts) — once for the total, once more to place its own draw.  Lane t owns draw t
// of the current round of 32.
__global__ void __launch_bounds__(kPickThreads)
k_pick_weighted_replace(const SampleParams *__restrict__ pa, uint32_t hop, uint32_t k) {
    chain_sync();
    const SampleParams &p = pa[blockIdx.y];
    const StageInfo nx = p.state->stage[hop + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t j = blockIdx.x * (kPickThreads / 32) + warp; j < nx.frontier_n; j += gridDim.x * (kPickThreads / 32)) {
        const FrontierEntry fe = p.frontier[j];
        const uint32_t deg = fe.deg;
        if (deg == 0 || k == 0) continue;
        const float *w = p.weights + fe.off;
        double total = 0.0;
        for (uint32_t i = 0; i < deg; ++i) total += (double)__ldg(w + i);
        const double scale = total / 18446744073709551615.0;  // u64::MAX as f64
        for (uint32_t t0 = 0; t0 < k; t0 += 32) {
            const uint32_t t = t0 + lane;
            const bool mine = t < k;
            const uint64_t bits = (p.rng_mode == AG_RNG_PHILOX)
                ? (((uint64_t)philox_u32(p.seed, hop, fe.id, 2 * t) << 32) | philox_u32(p.seed, hop, fe.id, 2 * t + 1))
                : wyrand_at(p.seed, fe.dbase + t);
            const double u = __ull2double_rn(bits) * scale;
            uint32_t idx = deg - 1;  // partition_point(c <= u) clamped to the last position
            bool placed = !mine;
            double c = 0.0;
            for (uint32_t i = 0; i < deg; ++i) {
                c += (double)__ldg(w + i);
                if (!placed && !(c <= u)) { idx = i; placed = true; }
                if (__all_sync(0xffffffffu, placed)) break;
            }
            if (mine) emit_edge(p, hop, nx.n_edges, fe, t, fe.off + idx);
        }
    }
}

// Weighted picks with a fanout above 32 (up to kLargeK): one block per frontier vertex.
// The block streams the row, every thread evaluating the exact key of one position per
// round (sampler.rs:1440-1452), and collects the positions that beat the current k-th
// best in a shared buffer; when the buffer fills up it is sorted (bitonic, ascending
// (key, position)) and cut back to the best k, which tightens the threshold.  The k
// smallest (key, position) pairs are a property of the row alone, so neither the order
// in which threads append nor the moments of the cuts change the result; the winners
// are emitted in ascending order like the fanout <= 32 path.
constexpr int kWLThreads = 256;
constexpr int kWLBuf = 2048;  // >= kLargeK + kWLThreads

__device__ __forceinline__ void wl_sort(double *key, uint32_t *pos) {  // whole block, kWLBuf entries
    for (uint32_t size = 2; size <= (uint32_t)kWLBuf; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (uint32_t t = threadIdx.x; t < (uint32_t)kWLBuf / 2; t += kWLThreads) {
                const uint32_t lo = 2 * t - (t & (stride - 1));  // index with bit `stride` clear
                const uint32_t hi = lo + stride;
                const bool up = (lo & size) == 0;
                const double ka = key[lo], kb = key[hi];
                const uint32_t pa = pos[lo], pb = pos[hi];
                if (key_less(kb, pb, ka, pa) == up) { key[lo] = kb; pos[lo] = pb; key[hi] = ka; pos[hi] = pa; }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kWLThreads)
k_pick_weighted_large(const SampleParams *__restrict__ pa, uint32_t hop, uint32_t k) {
    __shared__ double s_key[kWLBuf];
    __shared__ uint32_t s_pos[kWLBuf];
    __shared__ uint32_t s_fill;
    chain_sync();
    const SampleParams &p = pa[blockIdx.y];
    const StageInfo nx = p.state->stage[hop + 1];
    const double inf = __longlong_as_double(0x7FF0000000000000ll);
    for (uint32_t j = blockIdx.x; j < nx.frontier_n; j += gridDim.x) {
        const FrontierEntry fe = p.frontier[j];
        const uint32_t deg = fe.deg;
        if (deg == 0 || k == 0) continue;
        if (k >= deg) {  // take-all, row order, no draws
            for (uint32_t t = threadIdx.x; t < deg; t += kWLThreads) emit_edge(p, hop, nx.n_edges, fe, t, fe.off + t);
            continue;
        }
        __syncthreads();
        for (uint32_t t = threadIdx.x; t < (uint32_t)kWLBuf; t += kWLThreads) { s_key[t] = inf; s_pos[t] = 0xFFFFFFFFu; }
        if (threadIdx.x == 0) s_fill = 0;
        __syncthreads();
        double thr_key = inf;            // the k-th best so far (block-uniform)
        uint32_t thr_pos = 0xFFFFFFFFu;
        for (uint32_t c = 0; c < deg; c += kWLThreads) {
            const uint32_t pos = c + threadIdx.x;
            if (pos < deg) {
                const double key = weighted_key(p, hop, fe, pos);
                if (key_less(key, pos, thr_key, thr_pos)) {
                    const uint32_t at = atomicAdd(&s_fill, 1u);  // < kWLBuf: at most k + one round are ever held
                    s_key[at] = key; s_pos[at] = pos;
                }
            }
            __syncthreads();
            if (s_fill + kWLThreads > (uint32_t)kWLBuf || c + kWLThreads >= deg) {
                wl_sort(s_key, s_pos);
                const uint32_t keep = min(s_fill, k);
                for (uint32_t t = keep + threadIdx.x; t < (uint32_t)kWLBuf; t += kWLThreads) { s_key[t] = inf; s_pos[t] = 0xFFFFFFFFu; }
                if (keep == k) { thr_key = s_key[k - 1]; thr_pos = s_pos[k - 1]; }
                __syncthreads();
                if (threadIdx.x == 0) s_fill = keep;
                __syncthreads();
            }
        }
        for (uint32_t t = threadIdx.x; t < k; t += kWLThreads) emit_edge(p, hop, nx.n_edges, fe, t, fe.off + s_pos[t]);
    }
}

// Called by one thread once every block of the batch's last kernel has finished.
__device__ __forceinline__ void publish_counts(const SampleParams &p, BatchState *bs) {
    __threadfence();
    const StageInfo fin = load_stage_cg(&bs->stage[p.num_hops + 1]);
    ag_sample_counts c{};
    c.num_nodes = (uint32_t)min((uint64_t)fin.n_nodes, p.cap_nodes);
    c.num_edges = (uint32_t)min((uint64_t)fin.n_edges, p.cap_edges);
    c.num_seeds = p.n_seeds;
    c.num_hops = p.num_hops;
    for (uint32_t st = 0; st <= p.num_hops; ++st) c.nodes_per_hop[st] = __ldcg(&bs->nodes_per_stage[st]);
    for (uint32_t h = 0; h < p.num_hops; ++h) c.edges_per_hop[h] = load_stage_cg(&bs->stage[h + 1]).hop_edges;
    c.draws = fin.draws - load_stage_cg(&bs->stage[0]).draws;
    c.error = atomicOr(&bs->error, 0u);
    if ((uint64_t)fin.n_nodes > p.cap_nodes || (uint64_t)fin.n_edges > p.cap_edges) c.error |= kErrCapacity;
    *p.counts = c;
    bs->stream_pos = fin.draws;  // a bare sampler keeps consuming the same stream
    bs->error = 0;               // ready for the handle's next batch
    bs->ticket = 0;
    bs->done_blocks = 0;
}

template <bool HAS_NEXT>
__global__ void __launch_bounds__(kTile, 2)
k_assign(const SampleParams *__restrict__ pa, uint32_t stage, uint32_t k) {
    constexpr bool has_next = HAS_NEXT;  // the last stage queues no frontier
    constexpr int kIPT = AssignShape<HAS_NEXT>::kIPT, kTileItems = AssignShape<HAS_NEXT>::kTileItems;
    chain_sync();
    __shared__ uint32_t s_tile;
    __shared__ ScanVal s_warp[kTile / 32];
    __shared__ ScanVal s_prefix;

    const SampleParams &p = pa[blockIdx.y];
    BatchState *bs = p.state;
    StageInfo si = bs->stage[stage];
    if (stage == 0) {
        // A reseeded batch starts its stream at draw 0; otherwise the handle's stream
        // continues where its previous batch stopped (the host keeps that position).
        si = StageInfo{};
        si.draws = p.start_draw;
    }
    const uint32_t count = (stage == 0) ? p.n_seeds : si.hop_edges;
    const uint32_t n_tiles = max(1u, (count + kTileItems - 1) / kTileItems);
    const uint32_t edges_before_next = si.n_edges + ((stage == 0) ? 0u : count);  // where hop `stage` starts
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t gen = p.table.gen;
    const uint32_t *slots_in = (stage == 0) ? p.slot_of_seed : p.slot_of_edge + si.n_edges;

    if (!has_next && p.edge_index_local) {
        // Last stage: every edge of the batch exists, so the row offset of the int64
        // [2, E] local edge index is known.  Row 1 = the expanded vertex's local id.
        const uint64_t total = min((uint64_t)edges_before_next, p.cap_edges);
        for (uint64_t e = (uint64_t)blockIdx.x * kTile + threadIdx.x; e < total; e += (uint64_t)gridDim.x * kTile)
            p.edge_index_local[total + e] = (int64_t)p.src_local[e];
    }

    // The grid is sized for a typical batch, not for the worst case: a block
    // keeps drawing tile tickets until they run out.  Tickets are handed out in
    // order, so the tiles a look-back (or a pending vertex) waits for are always
    // already running.  A thread owns kIPT (4, last stage 8) consecutive items of its tile,
    // so that many table probes (and row-bound loads) are in flight per thread, and the
    // barriers, the ticket and the look-back are paid once per kTile * kIPT items.
    for (;;) {
        if (threadIdx.x == 0) s_tile = atomicAdd(&bs->ticket, 1u);
        __syncthreads();
        const uint32_t tile = s_tile;
        if (tile >= n_tiles) {
            // n_tiles + gridDim.x tickets are drawn in all; the last one resets the counter.
            if (threadIdx.x == 0 && tile == n_tiles + gridDim.x - 1) bs->ticket = 0;
            break;
        }
        const uint32_t item0 = tile * kTileItems + threadIdx.x * kIPT;

        // First sighting?  The table holds the pending mark of the smallest
        // position that named the vertex.
        uint32_t slot[kIPT], id[kIPT], cur32[kIPT];
        bool first[kIPT];
#pragma unroll
        for (int j = 0; j < kIPT; ++j) slot[j] = (item0 + j < count) ? slots_in[item0 + j] : 0xFFFFFFFFu;
#pragma unroll
        for (int j = 0; j < kIPT; ++j) {
            id[j] = 0; cur32[j] = 0; first[j] = false;
            if (slot[j] != 0xFFFFFFFFu) {
                const uint64_t cur = __ldcg((const unsigned long long *)&p.table.slots[slot[j]]);
                cur32[j] = (uint32_t)cur;
                first[j] = (cur32[j] == enc_pending(gen, stage, item0 + j));
                id[j] = (uint32_t)(cur >> 32);
            }
        }
        ScanVal tv{0u, 0u, 0ull};  // this thread's items together
        uint64_t off[kIPT];
        uint32_t deg[kIPT];
#pragma unroll
        for (int j = 0; j < kIPT; ++j) {
            off[j] = 0; deg[j] = 0;
            if (first[j]) {
                tv.flags += 1u;
                if (has_next) {
                    uint64_t d64;
                    row_bounds(p.offsets, p.num_nodes, p.num_edges, id[j], off[j], d64);
                    if (d64 > 0xFFFFFFFFull) { atomicOr(&bs->error, kErrCapacity); d64 = 0; }
                    deg[j] = (uint32_t)d64;
                    uint32_t take; uint64_t draws;
                    row_demand(p.mode, d64, k, take, draws);
                    tv.take += take; tv.draws += draws;
                }
            }
        }

        // Block scan of the threads' totals: warp scans, then the warp totals.
        const ScanVal incl = warp_inclusive_scan(tv, lane);
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
                    // Totals of the stage: hand over to the next one.
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
                    if (p.hub_count) *p.hub_count = 0;  // the hop's hub queue starts empty
                    if (stage == 0) bs->stage[0] = si;  // what the counts measure the draws against
                }
            }
        }
        __syncthreads();
        // exclusive prefix of this thread's first item
        ScanVal run = s_prefix + s_warp[warp];
        run.flags += incl.flags - tv.flags; run.take += incl.take - tv.take; run.draws += incl.draws - tv.draws;
        uint32_t pending = 0;  // bit j: item j's vertex is registered by an earlier item of this stage
#pragma unroll
        for (int j = 0; j < kIPT; ++j) {
            const uint32_t item = item0 + j;
            if (first[j]) {
                const uint32_t local = si.n_nodes + run.flags;
                if ((uint64_t)local >= p.cap_nodes || (uint64_t)local >= kMaxPos ||
                    (has_next && (uint64_t)run.flags >= p.frontier_cap)) {
                    atomicOr(&bs->error, kErrCapacity);
                    if (has_next && (uint64_t)run.flags < p.frontier_cap) p.frontier[run.flags] = FrontierEntry{};
                    // the batch has failed; its other items must still not wait for this vertex
                    p.table.slots[slot[j]] = ((uint64_t)id[j] << 32) | enc_final(gen, local & kPosMask);
                    write_item_local(p, stage, si.n_edges, item, 0xFFFFFFFFu);
                } else {
                    p.nodes[local] = id[j];
                    if (p.n_id) p.n_id[local] = (int64_t)id[j];
                    p.table.slots[slot[j]] = ((uint64_t)id[j] << 32) | enc_final(gen, local);  // readers accept either form
                    write_item_local(p, stage, si.n_edges, item, local);
                    if (has_next) {
                        FrontierEntry fe;
                        fe.off = off[j];
                        fe.dbase = si.draws + run.draws;
                        fe.id = id[j];
                        fe.local = local;
                        fe.deg = deg[j];
                        fe.ebase = run.take;
                        p.frontier[run.flags] = fe;
                    }
                }
                run.flags += 1u;
                if (has_next) {
                    uint32_t take; uint64_t draws;
                    row_demand(p.mode, deg[j], k, take, draws);
                    run.take += take; run.draws += draws;
                }
            } else if (item < count) {
                if (slot[j] == 0xFFFFFFFFu) write_item_local(p, stage, si.n_edges, item, 0xFFFFFFFFu);
                else if (!(cur32[j] & kPendingBit)) write_item_local(p, stage, si.n_edges, item, cur32[j] & kPosMask);  // an earlier stage's vertex
                else pending |= 1u << j;
            }
        }
        // The first sighting of a pending vertex is an earlier item of this stage: in this
        // tile (stored before the barrier below) or in a tile with a smaller ticket, whose
        // block is running and waits for nothing later than itself.
        __syncthreads();
        if (pending) {
#pragma unroll
            for (int j = 0; j < kIPT; ++j) {
                if (!(pending & (1u << j))) continue;
                uint32_t v = (uint32_t)__ldcg((const unsigned long long *)&p.table.slots[slot[j]]), spins = 0;
                while (v & kPendingBit) {
                    if (++spins > kSpinLimit) { atomicOr(&bs->error, kErrSpinTimeout); break; }
                    __nanosleep(40);
                    v = (uint32_t)__ldcg((const unsigned long long *)&p.table.slots[slot[j]]);
                }
                write_item_local(p, stage, si.n_edges, item0 + j, (v & kPendingBit) ? 0xFFFFFFFFu : (v & kPosMask));
            }
        }
    }

    if (has_next) return;
    // Last stage: the block that finishes last publishes the batch's counts (every
    // error bit any block raised is in by then) and leaves the state ready for the
    // handle's next batch.
    __shared__ bool s_last;
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(&bs->done_blocks, 1u) == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last || threadIdx.x != 0) return;
    publish_counts(p, bs);
}

// Hop `hop`: expand the frontier stage `hop` queued (stage[hop + 1] holds its
// size and where the hop's edges start).  The lanes of the whole grid share the
// frontier, so even a hop with few vertices spreads over the GPU.
template <int G, int PICK>
__global__ void __launch_bounds__(PICK == kPickLarge ? 128 : kPickThreads)
k_pick(const SampleParams *__restrict__ pa, uint32_t hop, uint32_t k) {
    __shared__ uint32_t s_picks[PICK == kPickLarge ? 4 : 1][PICK == kPickLarge ? kLargeK : 1];
    __shared__ uint32_t s_queue[PICK == kPickWeighted ? (kPickThreads / 32) * 64 : 1];  // weighted: 64 queued positions per warp
    chain_sync();
    const SampleParams &p = pa[blockIdx.y];
    const StageInfo nx = p.state->stage[hop + 1];
    if constexpr (PICK == kPickWeighted) pick_weighted(p, hop, k, nx.n_edges, p.frontier, nx.frontier_n, s_queue);
    else if constexpr (PICK == kPickLarge) pick_large(p, hop, k, nx.n_edges, p.frontier, nx.frontier_n, &s_picks[0][0]);
    else pick_small<G>(p, hop, k, nx.n_edges, p.frontier, nx.frontier_n);
}

// Hub rows of a weighted hop: one block per queued row.  Every warp streams an
// equal slice of the row into its own best k, the slices' winners meet in shared
// memory and warp 0 merges them; (key, position) is a total order, so the k
// smallest — and their emission order — do not depend on how the row was split.
__global__ void __launch_bounds__(kHubThreads)
k_pick_hubs(const SampleParams *__restrict__ pa, uint32_t hop, uint32_t k) {
    __shared__ double s_key[kHubThreads / 32][32];
    __shared__ uint32_t s_pos[kHubThreads / 32][32];
    __shared__ uint32_t s_thr;  // float bits: lowest k-th best key any warp holds for the current row
    __shared__ uint32_t s_queue[(kHubThreads / 32) * 64];
    chain_sync();
    const SampleParams &p = pa[blockIdx.y];
    const StageInfo nx = p.state->stage[hop + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kWarps = kHubThreads / 32;
    const double inf = __longlong_as_double(0x7FF0000000000000ll);
    const uint32_t hubs = min(*p.hub_count, nx.frontier_n);
    for (uint32_t h = blockIdx.x; h < hubs; h += gridDim.x) {
        const FrontierEntry fe = p.frontier[p.hub_list[h]];
        const uint32_t deg = fe.deg;
        const uint32_t per = ((deg + kWarps - 1) / kWarps + 31) & ~31u;  // slice per warp, whole chunks of 32
        const uint32_t begin = min(deg, (uint32_t)warp * per), end = min(deg, begin + per);
        double best_key = inf;
        uint32_t best_pos = 0xFFFFFFFFu;
        if (threadIdx.x == 0) s_thr = 0x7F800000u;  // +inf
        __syncthreads();
        topk_stream(p, hop, fe, begin, end, k, lane, best_key, best_pos, s_queue + warp * 64, &s_thr);
        s_key[warp][lane] = best_key; s_pos[warp][lane] = best_pos;
        __syncthreads();
        if (warp == 0) {
            for (int w = 1; w < kWarps; ++w) {
                const bool have = (uint32_t)lane < k && s_pos[w][lane] != 0xFFFFFFFFu;
                topk_insert_chunk(have ? s_key[w][lane] : inf, have ? s_pos[w][lane] : 0xFFFFFFFFu, best_key, best_pos, k, lane);
            }
            if ((uint32_t)lane < k) emit_edge(p, hop, nx.n_edges, fe, lane, fe.off + best_pos);
        }
        __syncthreads();
    }
}

// Launches `kern` as a programmatic dependent of the previous kernel on the stream.
template <typename... KArgs, typename... Args>
void launch_chained(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = 0; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

uint64_t next_pow2(uint64_t v) {
    uint64_t p = 1;
    while (p < v) p <<= 1;
    return p;
}

void launch_pick(int mode, uint32_t k, uint64_t frontier_est, uint32_t n_batches, cudaStream_t st,
                 const SampleParams *pa, uint32_t hop) {
    // About two waves of resident blocks over the whole group; the lanes stride beyond.
    auto blocks_for = [&](uint64_t vertices, uint64_t per_block) {
        const uint64_t b = (vertices + per_block - 1) / per_block;
        return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(b, std::max<uint64_t>(1, (uint64_t)kSMs * 16 / n_batches)));
    };
    if (mode == kModeWeightedReplace) {
        launch_chained(k_pick_weighted_replace, dim3(blocks_for(frontier_est, kPickThreads / 32), n_batches), dim3(kPickThreads), st, pa, hop, k);
    } else if (mode == kModeWeighted && k > 32) {
        launch_chained(k_pick_weighted_large, dim3(blocks_for(frontier_est, 1), n_batches), dim3(kWLThreads), st, pa, hop, k);
    } else if (mode == kModeWeighted) {
        launch_chained(k_pick<32, kPickWeighted>, dim3(blocks_for(frontier_est, kPickThreads / 32), n_batches), dim3(kPickThreads), st, pa, hop, k);
        // rows longer than kHubDegree were only queued: one block per queued row
        launch_chained(k_pick_hubs, dim3(std::max<uint32_t>(1, (uint32_t)(kSMs * 2 / n_batches)), n_batches), dim3(kHubThreads), st, pa, hop, k);
    } else if (k > 32) {
        launch_chained(k_pick<32, kPickLarge>, dim3(blocks_for(frontier_est, 4), n_batches), dim3(128), st, pa, hop, k);
    } else {
        const uint32_t G = k <= 4 ? 4 : k <= 8 ? 8 : k <= 16 ? 16 : 32;
        const dim3 grid(blocks_for(frontier_est, 2 * kPickThreads / G), n_batches);  // two vertices per lane group and round
        switch (G) {
            case 4: launch_chained(k_pick<4, kPickSmall>, grid, dim3(kPickThreads), st, pa, hop, k); break;
            case 8: launch_chained(k_pick<8, kPickSmall>, grid, dim3(kPickThreads), st, pa, hop, k); break;
            case 16: launch_chained(k_pick<16, kPickSmall>, grid, dim3(kPickThreads), st, pa, hop, k); break;
            default: launch_chained(k_pick<32, kPickSmall>, grid, dim3(kPickThreads), st, pa, hop, k); break;
        }
    }
}

}  // namespace
}  // namespace ag

using namespace ag;

struct ag_sampler {
    const ag_graph *g = nullptr;
    ag_sampling_config cfg{};
    int device = 0;
    int mode = kModeUniform;
    uint64_t seed = 0;
    // RNG stream position of the handle (draws consumed by earlier batches).  Kept on the
    // host from the counts of every finished continuing batch, so it survives scratch
    // growth and state resets; `pending_pos` marks a launched batch not yet accounted.
    uint64_t stream_pos = 0;
    bool pending_pos = false;
    uint32_t epoch = 0;
    uint32_t gen = 0;    // table generation of the next launch
    uint32_t group = 1;  // batches one launch chain can carry
    // sizing (per batch)
    uint64_t cap_seeds = 0, max_nodes = 0, max_edges = 0, max_hop_edges = 0;
    uint64_t table_cap = 0, n_tiles = 0;
    // scratch (device), each `group` times the per-batch size
    uint64_t *table = nullptr;
    FrontierEntry *frontier = nullptr;
    uint64_t max_frontier = 0;
    uint32_t *slot_of_seed = nullptr, *slot_of_edge = nullptr;
    uint32_t *hub_list = nullptr;  // weighted only: per batch max_frontier queue slots + 1 counter word
    TileDesc *tiles = nullptr;
    BatchState *state = nullptr;
    uint32_t *seeds_dev = nullptr;
    ag_sample_counts *counts_dev = nullptr;
    SampleParams *params_dev = nullptr;
    GatherArgs *gather_dev = nullptr;
    // pinned host
    uint32_t *seeds_pinned = nullptr;
    ag_sample_counts *counts_host = nullptr;
    bool yield_wait = false;  // ag_sample_group_wait polls and yields instead of spinning in the runtime
    SampleParams *params_host = nullptr;
    GatherArgs *gather_host = nullptr;
    cudaEvent_t done = nullptr;
    bool in_flight = false, dirty = true;
    uint32_t in_flight_n = 0;
    // The gather runs on the handle's own low-priority stream, behind an event:
    // sampling kernels of other handles (latency-bound, few resources) then slip
    // in between the short-lived blocks of a running gather (bandwidth-bound).
    cudaStream_t gstream = nullptr;
    cudaEvent_t sampled = nullptr;
    // Sharded stores: the remote part of a chain's rows is fetched by a launch of its own on
    // this stream (between the two priorities), beside the local part on gstream.
    cudaStream_t rstream = nullptr;
    cudaEvent_t remote_done = nullptr;
    uint64_t est_rows_tight = 0;  // rows per batch the last chain produced, with little headroom (sort padding)
    SortScratch sort;  // sharded feature stores: the chain's row ids in address order (gather.cu)
    // The arguments of the chain in flight, kept so that it can be launched once more:
    // the dedup tables are sized from the node counts of earlier chains (small tables stay
    // in L2), and a batch that outgrows its table is sampled again with the full-size one.
    struct Launch {
        uint32_t n_batches = 0;
        std::vector<const uint32_t *> seeds;
        std::vector<uint64_t> n_seeds, batch_seeds;
        bool has_batch_seeds = false;
        int32_t seeds_mem = AG_MEM_HOST;
        const ag_features *feats = nullptr;
        std::vector<ag_subgraph_buffers> bufs;
        cudaStream_t stream = nullptr;
        bool reduced_table = false;
    } last;
    // Grid-size estimates from the last group's real counts (the bounds before
    // the first one); kernels stride past an estimate that turns out too small.
    uint64_t est_nodes = 0;
    uint64_t est_items[AG_MAX_HOPS + 2] = {0};
    // optional per-group device timing
    bool profile = false, gathered = false;
    cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
    // buffers handed out by ag_sample (library-allocated variant)
    std::vector<void *> owned;
};

namespace {

void compute_bounds(const ag_sampler *s, uint64_t n_seeds, uint64_t *max_nodes, uint64_t *max_edges,
                    uint64_t *max_hop_edges) {
    const uint64_t N = s->g->num_nodes;
    uint64_t f = std::min<uint64_t>(n_seeds, N), nodes = f, edges = 0, mhe = 0;
    for (uint32_t h = 0; h < s->cfg.num_hops; ++h) {
        const uint64_t e = f * s->cfg.fanout[h];
        edges += e;
        mhe = std::max(mhe, e);
        f = std::min<uint64_t>(e, N);
        nodes += f;
    }
    if (max_nodes) *max_nodes = std::min<uint64_t>(nodes, N);
    if (max_edges) *max_edges = edges;
    if (max_hop_edges) *max_hop_edges = mhe;
}

void free_scratch(ag_sampler *s) {
    cudaFree(s->table); cudaFree(s->frontier);
    s->frontier = nullptr;
    cudaFree(s->slot_of_seed); cudaFree(s->slot_of_edge); cudaFree(s->tiles);
    cudaFree(s->hub_list); s->hub_list = nullptr;
    cudaFree(s->seeds_dev);
    if (s->seeds_pinned) cudaFreeHost(s->seeds_pinned);
    s->table = nullptr;
    s->slot_of_seed = s->slot_of_edge = nullptr; s->tiles = nullptr;
    s->seeds_dev = nullptr; s->seeds_pinned = nullptr;
}

// A finished continuing batch (no per-batch seed) moves the handle's stream on by
// the draws it consumed; called wherever the host has just waited for the batch.
void account_stream(ag_sampler *s) {
    if (s->pending_pos) s->stream_pos += s->counts_host[0].draws;
    s->pending_pos = false;
}

// Scratch for `group` batches of up to n_seeds seeds each.
int32_t ensure_scratch(ag_sampler *s, uint64_t n_seeds) {
    if (n_seeds <= s->cap_seeds && s->table) return AG_OK;
    if (s->in_flight) { AG_CUDA(cudaEventSynchronize(s->done)); s->in_flight = false; account_stream(s); }
    free_scratch(s);
    s->cap_seeds = 0;
    const uint64_t cap = std::max<uint64_t>(n_seeds, 1), G = s->group;
    compute_bounds(s, cap, &s->max_nodes, &s->max_edges, &s->max_hop_edges);
    if (s->max_nodes >= kMaxPos || s->max_hop_edges >= kMaxPos || cap >= kMaxPos || s->max_edges >= 0xFFFFFFFFull)
        return fail(AG_ERR_VALUE, "batch too large: %llu seeds with this fanout can reach %llu nodes and %llu edges "
                    "in a hop (limit %llu each)", (unsigned long long)n_seeds, (unsigned long long)s->max_nodes,
                    (unsigned long long)s->max_hop_edges, (unsigned long long)kMaxPos - 1);
    s->table_cap = std::max<uint64_t>(1024, next_pow2(2 * s->max_nodes));
    AG_CUDA(cudaMalloc(&s->table, G * s->table_cap * 8));
    // the frontier of a hop holds at most the vertices the previous stage found
    s->max_frontier = std::max<uint64_t>(std::min<uint64_t>(std::max(cap, s->max_hop_edges), s->g->num_nodes), 1);
    AG_CUDA(cudaMalloc(&s->frontier, G * s->max_frontier * sizeof(FrontierEntry)));
    AG_CUDA(cudaMalloc(&s->slot_of_seed, G * cap * 4));
    AG_CUDA(cudaMalloc(&s->slot_of_edge, G * std::max<uint64_t>(s->max_edges, 1) * 4));
    if (s->mode == kModeWeighted) {
        AG_CUDA(cudaMalloc(&s->hub_list, G * (s->max_frontier + 1) * 4));
        AG_CUDA(cudaMemset(s->hub_list, 0, G * (s->max_frontier + 1) * 4));
    }
    s->n_tiles = std::max<uint64_t>(std::max(cap, s->max_hop_edges) / kTile + 2, 2);
    AG_CUDA(cudaMalloc(&s->tiles, G * s->n_tiles * sizeof(TileDesc)));
    AG_CUDA(cudaMemset(s->tiles, 0, G * s->n_tiles * sizeof(TileDesc)));
    AG_CUDA(cudaMalloc(&s->seeds_dev, G * cap * 4));
    AG_CUDA(cudaHostAlloc(&s->seeds_pinned, G * cap * 4, cudaHostAllocDefault));
    s->cap_seeds = cap;
    s->epoch = 0;
    s->dirty = true;
    return AG_OK;
}

}  // namespace

extern "C" int32_t ag_sampler_create_group(const ag_graph *g, const ag_sampling_config *cfg, uint32_t group,
                                           ag_sampler **out) {
    if (!g || !cfg || !out) return fail(AG_ERR_VALUE, "ag_sampler_create: null argument");
    if (group == 0 || group > 256) return fail(AG_ERR_VALUE, "group size must be between 1 and 256 (got %u)", group);
    if (cfg->num_hops == 0 || cfg->num_hops > AG_MAX_HOPS)
        return fail(AG_ERR_VALUE, "num_neighbors must list between 1 and %d hops (got %u)", AG_MAX_HOPS, cfg->num_hops);
    // SamplerConfigError::WeightsMissing (sampler.rs:331-337)
    if (cfg->weighted && !g->weights)
        return fail(AG_ERR_VALUE, "weighted sampling requested, but the graph has no edge weights");
    if (cfg->rng_mode != AG_RNG_WYRAND_EXACT && cfg->rng_mode != AG_RNG_PHILOX)
        return fail(AG_ERR_VALUE, "unknown rng_mode %d", cfg->rng_mode);
    for (uint32_t h = 0; h < cfg->num_hops; ++h) {
        if (cfg->fanout[h] > (uint32_t)kLargeK)
            return fail(AG_ERR_VALUE, "fanout of at most %d per hop is supported (hop %u asks %u)", kLargeK, h, cfg->fanout[h]);
    }
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_sampler *s = new ag_sampler();
    s->g = g;
    s->cfg = *cfg;
    s->device = g->device;
    s->group = group;
    s->mode = cfg->weighted ? (cfg->replace ? kModeWeightedReplace : kModeWeighted) : (cfg->replace ? kModeReplace : kModeUniform);
    s->seed = cfg->seed;
    int32_t st = AG_OK;
    do {
        if (cudaMalloc(&s->state, group * sizeof(BatchState)) != cudaSuccess ||
            cudaMemset(s->state, 0, group * sizeof(BatchState)) != cudaSuccess ||
            cudaMalloc(&s->counts_dev, group * sizeof(ag_sample_counts)) != cudaSuccess ||
            cudaMalloc(&s->params_dev, group * sizeof(SampleParams)) != cudaSuccess ||
            cudaMalloc(&s->gather_dev, group * sizeof(GatherArgs)) != cudaSuccess ||
            cudaHostAlloc(&s->counts_host, group * sizeof(ag_sample_counts), cudaHostAllocDefault) != cudaSuccess ||
            cudaHostAlloc(&s->params_host, group * sizeof(SampleParams), cudaHostAllocDefault) != cudaSuccess ||
            cudaHostAlloc(&s->gather_host, group * sizeof(GatherArgs), cudaHostAllocDefault) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->done, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->sampled, cudaEventDisableTiming) != cudaSuccess) {
            st = fail(AG_ERR_CUDA, "sampler allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);  // lo = least urgent
        // AG_GATHER_PRIORITY=high: the gather streams as urgent as the sampling streams (A/B measurements)
        static const bool gather_high = [] { const char *v = getenv("AG_GATHER_PRIORITY"); return v && v[0] == 'h'; }();
        if (cudaStreamCreateWithPriority(&s->gstream, cudaStreamNonBlocking, gather_high ? hi : lo) != cudaSuccess ||
            cudaStreamCreateWithPriority(&s->rstream, cudaStreamNonBlocking, (lo + hi) / 2) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->remote_done, cudaEventDisableTiming) != cudaSuccess) {
            st = fail(AG_ERR_CUDA, "cudaStreamCreateWithPriority failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        st = ensure_scratch(s, std::max<uint32_t>(cfg->max_seeds, 1));
    } while (0);
    if (st != AG_OK) { ag_sampler_free(s); return st; }
    *out = s;
    return AG_OK;
}

extern "C" int32_t ag_sampler_create(const ag_graph *g, const ag_sampling_config *cfg, ag_sampler **out) {
    return ag_sampler_create_group(g, cfg, 1, out);
}

extern "C" void ag_sampler_free(ag_sampler *s) {
    if (!s) return;
    DeviceGuard guard(s->device);
    if (s->in_flight && s->done) cudaEventSynchronize(s->done);
    free_scratch(s);
    s->sort.release();
    for (void *p : s->owned) cudaFree(p);
    cudaFree(s->state); cudaFree(s->counts_dev); cudaFree(s->params_dev); cudaFree(s->gather_dev);
    if (s->counts_host) cudaFreeHost(s->counts_host);
    if (s->params_host) cudaFreeHost(s->params_host);
    if (s->gather_host) cudaFreeHost(s->gather_host);
    if (s->done) cudaEventDestroy(s->done);
    if (s->sampled) cudaEventDestroy(s->sampled);
    if (s->gstream) cudaStreamDestroy(s->gstream);
    if (s->rstream) cudaStreamDestroy(s->rstream);
    if (s->remote_done) cudaEventDestroy(s->remote_done);
    for (auto &e : s->ev) if (e) cudaEventDestroy(e);
    delete s;
}

extern "C" int32_t ag_sampler_reseed(ag_sampler *s, uint64_t seed) {
    if (!s) return fail(AG_ERR_VALUE, "ag_sampler_reseed: null sampler");
    if (s->in_flight) {  // the batch in flight still belongs to the old stream
        DeviceGuard guard(s->device);
        cudaEventSynchronize(s->done);
    }
    s->seed = seed;
    s->stream_pos = 0;
    s->pending_pos = false;
    return AG_OK;
}

// A loader's worker threads wait for their chains by polling the event and yielding
// the core between polls instead of spinning inside the runtime: with three workers
// per GPU and eight GPUs per host the spinning waits alone would occupy most of the
// host's cores, which the consumer's own thread needs; on an idle core a yield returns
// at once, so nothing is lost when there are cores to spare.  (Sleeping on the event
// — cudaEventBlockingSync — was measured too: -9 % on one GPU, the wake-up is too slow.)
int32_t ag::sampler_set_yielding_wait(ag_sampler *s, bool on) {
    s->yield_wait = on;
    return AG_OK;
}

extern "C" int32_t ag_sampler_set_profiling(ag_sampler *s, int32_t on) {
    if (!s) return fail(AG_ERR_VALUE, "ag_sampler_set_profiling: null sampler");
    DeviceGuard guard(s->device);
    if (!guard.ok) return AG_ERR_CUDA;
    if (on && !s->ev[0])
        for (auto &e : s->ev) AG_CUDA(cudaEventCreate(&e));
    s->profile = on != 0;
    return AG_OK;
}

extern "C" int32_t ag_sampler_bounds(const ag_sampler *s, uint64_t n_seeds, uint64_t *max_nodes, uint64_t *max_edges) {
    if (!s) return fail(AG_ERR_VALUE, "ag_sampler_bounds: null sampler");
    compute_bounds(s, n_seeds, max_nodes, max_edges, nullptr);
    return AG_OK;
}

// One launch chain for `n_batches` independent batches.  batch b uses
// seeds[b] / n_seeds[b] / bufs[b] and, when batch_seeds != NULL, restarts its
// RNG stream at draw 0 of batch_seeds[b]; with batch_seeds == NULL the handle's
// own stream continues (only meaningful for a single batch).
namespace {
int32_t launch_saved(ag_sampler *s, bool relaunch);
}  // namespace

extern "C" int32_t ag_sample_group_into(ag_sampler *s, uint32_t n_batches, const uint32_t *const *seeds,
                                        const uint64_t *n_seeds, int32_t seeds_mem, const uint64_t *batch_seeds,
                                        const ag_features *feats, ag_subgraph_buffers *bufs, void *stream) {
    if (!s || !bufs || !seeds || !n_seeds) return fail(AG_ERR_VALUE, "ag_sample_group_into: null argument");
    if (n_batches == 0 || n_batches > s->group)
        return fail(AG_ERR_VALUE, "group of %u batches does not fit a sampler created for %u", n_batches, s->group);
    const ag_graph *g = s->g;
    uint64_t max_n = 0;
    bool want_x = false;
    for (uint32_t b = 0; b < n_batches; ++b) {
        const ag_subgraph_buffers &B = bufs[b];
        if (!seeds[b] && n_seeds[b]) return fail(AG_ERR_VALUE, "ag_sample_group_into: null seeds");
        if (!B.nodes || !B.edge_dst || !B.src_local || !B.dst_local || !B.seed_locals)
            return fail(AG_ERR_VALUE, "nodes, edge_dst, src_local, dst_local and seed_locals buffers are required");
        if (B.cap_seeds < n_seeds[b]) return fail(AG_ERR_VALUE, "seed_locals capacity %llu < %llu seeds",
                                                  (unsigned long long)B.cap_seeds, (unsigned long long)n_seeds[b]);
        if (n_seeds[b] >= kMaxPos) return fail(AG_ERR_VALUE, "too many seeds");
        max_n = std::max(max_n, n_seeds[b]);
        want_x = want_x || (feats && B.x);
        // Seeds::new (sampler.rs:230-239): name the first id at or past num_nodes.
        if (seeds_mem == AG_MEM_HOST)
            for (uint64_t i = 0; i < n_seeds[b]; ++i)
                if ((uint64_t)seeds[b][i] >= g->num_nodes)
                    return fail(AG_ERR_SAMPLING, "seed node %u (position %llu) is out of range for %llu nodes",
                                seeds[b][i], (unsigned long long)i, (unsigned long long)g->num_nodes);
    }
    if (feats && want_x && feats->row_stride != 1 && !feats->shards)
        return fail(AG_ERR_VALUE, "a cyclic feature shard is read through a sharded view");
    if (feats && want_x && feats->device != s->device)
        return fail(AG_ERR_VALUE, "feature store lives on device %d, sampler on %d", feats->device, s->device);
    DeviceGuard guard(s->device);
    if (!guard.ok) return AG_ERR_CUDA;
    if (s->in_flight) { AG_CUDA(cudaEventSynchronize(s->done)); s->in_flight = false; account_stream(s); }
    ag_sampler::Launch &L = s->last;
    L.n_batches = n_batches;
    L.seeds.assign(seeds, seeds + n_batches);
    L.n_seeds.assign(n_seeds, n_seeds + n_batches);
    L.has_batch_seeds = batch_seeds != nullptr;
    if (batch_seeds) L.batch_seeds.assign(batch_seeds, batch_seeds + n_batches);
    L.seeds_mem = seeds_mem;
    L.feats = feats;
    L.bufs.assign(bufs, bufs + n_batches);
    L.stream = (cudaStream_t)stream;
    return launch_saved(s, false);
}

namespace {
// Time zero of the profiled intervals on a GPU: an event recorded once, on the stream of
// the first profiled launch there.  Called with a null stream it only returns the event.
cudaEvent_t profile_origin(int device, cudaStream_t st) {
    static std::mutex m;
    static cudaEvent_t origin[64] = {nullptr};
    std::lock_guard<std::mutex> lk(m);
    if (device < 0 || device >= 64) return nullptr;
    if (!origin[device] && st) {
        cudaEvent_t e = nullptr;
        if (cudaEventCreate(&e) == cudaSuccess && cudaEventRecord(e, st) == cudaSuccess) origin[device] = e;
        else if (e) cudaEventDestroy(e);
    }
    return origin[device];
}

int32_t launch_saved_impl(ag_sampler *s, bool relaunch);

// Queues the chain described by s->last.  relaunch: the same chain once more with
// full-size dedup tables (host seeds are already in the handle's device copy).
// A failure part way through leaves kernels of the chain queued: wait for them and
// mark the handle's device state unknown, so that the next call clears it instead of
// reusing staging buffers, table generation and batch state under running kernels.
int32_t launch_saved(ag_sampler *s, bool relaunch) {
    const int32_t st = launch_saved_impl(s, relaunch);
    if (st != AG_OK) {
        const std::string msg = ag_last_error();
        cudaStreamSynchronize(s->last.stream);
        if (s->gstream) cudaStreamSynchronize(s->gstream);
        if (s->rstream) cudaStreamSynchronize(s->rstream);
        cudaGetLastError();
        s->dirty = true;
        s->pending_pos = false;
        s->in_flight = false;
        set_error("%s", msg.c_str());
    }
    return st;
}

int32_t launch_saved_impl(ag_sampler *s, bool relaunch) {
    const ag_sampler::Launch &L = s->last;
    const uint32_t n_batches = L.n_batches;
    const uint32_t *const *seeds = L.seeds.data();
    const uint64_t *n_seeds = L.n_seeds.data();
    const uint64_t *batch_seeds = L.has_batch_seeds ? L.batch_seeds.data() : nullptr;
    const int32_t seeds_mem = L.seeds_mem;
    const ag_features *feats = L.feats;
    const ag_subgraph_buffers *bufs = L.bufs.data();
    const ag_graph *g = s->g;
    uint64_t max_n = 0;
    bool want_x = false;
    for (uint32_t b = 0; b < n_batches; ++b) {
        max_n = std::max(max_n, n_seeds[b]);
        want_x = want_x || (feats && bufs[b].x);
    }
    cudaStream_t st = L.stream;
    AG_TRY(ensure_scratch(s, max_n));
    if (s->profile) {
        profile_origin(s->device, st);
        AG_CUDA(cudaEventRecord(s->ev[0], st));
    }
    if (s->dirty || s->gen >= kGens) {
        // Every slot free again.  A launch marks its entries with its generation,
        // so this real clear is only needed once the generations have cycled (or
        // after a failed launch left the table in an unknown state).
        AG_CUDA(cudaMemsetAsync(s->table, 0xFF, (uint64_t)s->group * s->table_cap * 8, st));
        s->gen = 0;
    }
    if (s->dirty) {
        AG_CUDA(cudaMemsetAsync(s->state, 0, s->group * sizeof(BatchState), st));
        s->dirty = false;
    }
    const uint32_t H = s->cfg.num_hops;
    if (s->epoch + (H + 2) > 0x3FFFFF00u) {  // the epoch lives in 30 bits of the tile status
        AG_CUDA(cudaMemsetAsync(s->tiles, 0, (uint64_t)s->group * s->n_tiles * sizeof(TileDesc), st));
        s->epoch = 0;
    }
    // Tables sized for twice the nodes the last chains really produced (with headroom)
    // instead of the worst-case bound: a chain's tables then fit in L2.
    uint64_t used_cap = s->table_cap;
    if (!relaunch && s->est_nodes) used_cap = std::min(s->table_cap, std::max<uint64_t>(1024, next_pow2(2 * s->est_nodes)));
    s->last.reduced_table = used_cap < s->table_cap;
    uint32_t log2cap = 0;
    while ((1ull << log2cap) < used_cap) ++log2cap;
    const uint64_t ecap = std::max<uint64_t>(s->max_edges, 1);

    uint64_t b_nodes = 0;
    for (uint32_t b = 0; b < n_batches; ++b) {
        const ag_subgraph_buffers &B = bufs[b];
        const uint32_t n = (uint32_t)n_seeds[b];
        SampleParams p{};
        p.offsets = g->offsets; p.dst = g->dst; p.weights = g->weights;
        p.num_nodes = g->num_nodes; p.num_edges = g->num_edges;
        p.table = DedupTable{s->table + (uint64_t)b * used_cap, (uint32_t)(used_cap - 1), 32u - log2cap, s->gen};
        p.state = s->state + b;
        p.tiles = s->tiles + (uint64_t)b * s->n_tiles;
        p.epoch_base = s->epoch + 1;
        p.n_seeds = n;
        if (seeds_mem == AG_MEM_HOST) {
            if (n && !relaunch) memcpy(s->seeds_pinned + (uint64_t)b * s->cap_seeds, seeds[b], (size_t)n * 4);
            p.seeds = s->seeds_dev + (uint64_t)b * s->cap_seeds;
        } else {
            p.seeds = seeds[b];
        }
        p.seed = batch_seeds ? batch_seeds[b] : s->seed;
        p.rng_mode = s->cfg.rng_mode; p.mode = s->mode;
        p.start_draw = batch_seeds ? 0ull : s->stream_pos;
        p.num_hops = H;
        p.nodes = B.nodes; p.edge_src = B.edge_src; p.edge_dst = B.edge_dst;
        p.src_local = B.src_local; p.dst_local = B.dst_local; p.seed_locals = B.seed_locals;
        p.edge_ids = s->cfg.track_edge_ids ? B.edge_ids : nullptr;
        p.cap_nodes = B.cap_nodes; p.cap_edges = B.cap_edges;
        p.n_id = B.n_id; p.edge_index_local = B.edge_index_local; p.e_id = B.e_id; p.seed_index = B.seed_index;
        p.counts = s->counts_dev + b;
        p.slot_of_seed = s->slot_of_seed + (uint64_t)b * s->cap_seeds;
        p.slot_of_edge = s->slot_of_edge + (uint64_t)b * ecap;
        p.frontier = s->frontier + (uint64_t)b * s->max_frontier;
        p.frontier_cap = s->max_frontier;
        if (s->hub_list) {
            p.hub_count = s->hub_list + (uint64_t)b * (s->max_frontier + 1);
            p.hub_list = p.hub_count + 1;
        }
        s->params_host[b] = p;
        uint64_t bn, be;
        compute_bounds(s, n, &bn, &be, nullptr);
        b_nodes = std::max(b_nodes, bn);
        if (want_x) {
            GatherArgs ga{};
            if (feats && B.x) {
                set_gather_source(ga, feats);
                ga.ids = B.nodes; ga.ids64 = 0;
                ga.n = std::min<uint64_t>(bn, B.cap_x ? std::min(B.cap_x, B.cap_nodes) : B.cap_nodes);
                // rows to gather = nodes registered by the last stage (read on the device)
                ga.n_dev = &s->state[b].stage[H + 1].n_nodes;
                ga.out = B.x;
            }
            s->gather_host[b] = ga;
        }
    }
    s->pending_pos = (batch_seeds == nullptr);  // a continuing batch advances the handle's stream
    s->epoch += H + 2;
    s->gen += 1;
    if (seeds_mem == AG_MEM_HOST && !relaunch)
        AG_CUDA(cudaMemcpyAsync(s->seeds_dev, s->seeds_pinned, (uint64_t)n_batches * s->cap_seeds * 4, cudaMemcpyHostToDevice, st));
    AG_CUDA(cudaMemcpyAsync(s->params_dev, s->params_host, n_batches * sizeof(SampleParams), cudaMemcpyHostToDevice, st));
    if (want_x)
        AG_CUDA(cudaMemcpyAsync(s->gather_dev, s->gather_host, n_batches * sizeof(GatherArgs), cudaMemcpyHostToDevice, st));

    const SampleParams *pa = s->params_dev;
    const uint32_t nmax = (uint32_t)max_n;
    // Grids cover the worst case only up to about two waves of resident blocks
    // over the whole group; the expand kernel draws tile tickets beyond that, so
    // a batch far below its bound does not pay for thousands of empty blocks.
    auto tiles_for = [&](uint64_t items, bool last) {
        const uint64_t per = last ? AssignShape<false>::kTileItems : AssignShape<true>::kTileItems;
        const uint64_t blocks = (items + per - 1) / per;
        return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(blocks, std::max<uint64_t>(1, (uint64_t)kSMs * 8 / n_batches)));
    };
    if (nmax) k_insert_seeds<<<dim3((nmax + 255) / 256, n_batches), 256, 0, st>>>(pa);
    uint64_t items = nmax;  // bound on the items of the stage being launched
    for (uint32_t stage = 0; stage <= H; ++stage) {
        const bool has_next = stage < H;
        const uint32_t k = has_next ? s->cfg.fanout[stage] : 0;
        const uint64_t expect = (stage && s->est_items[stage]) ? std::min(items, s->est_items[stage]) : items;
        if (has_next) launch_chained(k_assign<true>, dim3(tiles_for(expect, false), n_batches), dim3(kTile), st, pa, stage, k);
        else launch_chained(k_assign<false>, dim3(tiles_for(expect, true), n_batches), dim3(kTile), st, pa, stage, k);
        if (has_next && k) {
            // the new vertices of this stage are at most its items
            launch_pick(s->mode, k, std::min<uint64_t>(expect, g->num_nodes), n_batches, st, pa, stage);
        }
        items = std::min<uint64_t>(items, g->num_nodes) * k;
    }
    AG_CUDA(cudaGetLastError());
    if (s->profile) AG_CUDA(cudaEventRecord(s->ev[1], st));
    AG_CUDA(cudaMemcpyAsync(s->counts_host, s->counts_dev, n_batches * sizeof(ag_sample_counts), cudaMemcpyDeviceToHost, st));
    s->gathered = false;
    if (want_x) {
        bool aligned = ((uintptr_t)feats->payload % 16) == 0;
        for (uint32_t b = 0; b < n_batches; ++b) aligned = aligned && ((uintptr_t)bufs[b].x % 16) == 0;
        const uint64_t rows = s->est_nodes ? std::min(b_nodes, s->est_nodes) : b_nodes;
        const uint32_t row_bytes = (uint32_t)(feats->dim * elem_size(feats->dtype));
        const bool sorted = sorted_gather_applies(feats, row_bytes, aligned);
        // Rows of a sharded store are fetched in address order, each distinct row of the chain
        // once.  Making and sorting the keys is small, latency-bound work like the sampling
        // kernels: it stays on the (high-priority) sampling stream.  (The handle's previous
        // chain has finished — its event was waited for — so the sort scratch is free.)
        const uint64_t sort_rows = s->est_rows_tight ? std::min(rows, s->est_rows_tight) : rows;  // less padding to sort
        if (sorted) AG_CUDA(launch_sort_keys(GatherArgs{}, s->gather_dev, n_batches, sort_rows, feats, s->sort, st));
        // sampling chain -> event -> gather on the low-priority stream -> event -> caller's stream
        AG_CUDA(cudaEventRecord(s->sampled, st));
        AG_CUDA(cudaStreamWaitEvent(s->gstream, s->sampled, 0));
        if (s->profile) AG_CUDA(cudaEventRecord(s->ev[2], s->gstream));
        if (sorted) {
            AG_CUDA(cudaStreamWaitEvent(s->rstream, s->sampled, 0));
            AG_CUDA(launch_sorted_fetch(GatherArgs{}, s->gather_dev, n_batches, sort_rows, row_bytes, (uint32_t)feats->dim,
                                        feats->dtype, feats, s->sort, s->gstream, s->rstream));
            AG_CUDA(cudaEventRecord(s->remote_done, s->rstream));
            AG_CUDA(cudaStreamWaitEvent(s->gstream, s->remote_done, 0));
        } else {
            AG_CUDA(launch_gather_group(s->gather_dev, n_batches, row_bytes, (uint32_t)feats->dim, rows, aligned,
                                        feats->dtype, feats->shards != nullptr, s->gstream));
        }
        if (s->profile) AG_CUDA(cudaEventRecord(s->ev[3], s->gstream));
        AG_CUDA(cudaEventRecord(s->done, s->gstream));
        AG_CUDA(cudaStreamWaitEvent(st, s->done, 0));  // the caller's stream stays ordered behind the gather
        s->gathered = true;
    } else {
        AG_CUDA(cudaEventRecord(s->done, st));
    }
    s->in_flight = true;
    s->in_flight_n = n_batches;
    return AG_OK;
}
}  // namespace

// Waits for the group queued last; counts[b] receives batch b's counts.  Returns
// the first batch error (the other batches' counts are still valid).
extern "C" int32_t ag_sample_group_wait(ag_sampler *s, ag_sample_counts *counts, int32_t *statuses) {
    if (!s) return fail(AG_ERR_VALUE, "ag_sample_wait: null sampler");
    if (!s->in_flight) return fail(AG_ERR_VALUE, "ag_sample_wait: no batch in flight");
    DeviceGuard guard(s->device);
    if (!guard.ok) return AG_ERR_CUDA;
    auto wait_done = [&]() -> cudaError_t {
        if (!s->yield_wait) return cudaEventSynchronize(s->done);
        cudaError_t q;
        while ((q = cudaEventQuery(s->done)) == cudaErrorNotReady) sched_yield();
        return q;
    };
    cudaError_t e = wait_done();
    s->in_flight = false;
    if (e == cudaSuccess && s->last.reduced_table) {
        bool full = false;
        for (uint32_t b = 0; b < s->in_flight_n; ++b) full = full || (s->counts_host[b].error & kErrTableFull);
        if (full) {
            // A batch outgrew the table its chain was given: once more, with the full-size tables.
            s->dirty = true;
            s->est_nodes = 0;
            AG_TRY(launch_saved(s, true));
            e = wait_done();
            s->in_flight = false;
        }
    }
    if (e != cudaSuccess) {
        s->dirty = true;
        s->pending_pos = false;
        return fail(AG_ERR_CUDA, "sampling kernels failed: %s", cudaGetErrorString(e));
    }
    account_stream(s);
    float sample_ms = 0.f, gather_ms = 0.f, gather_begin = 0.f;
    if (s->profile) {
        cudaEventElapsedTime(&sample_ms, s->ev[0], s->ev[1]);
        if (s->gathered) {
            cudaEventElapsedTime(&gather_ms, s->ev[2], s->ev[3]);
            if (cudaEvent_t origin = profile_origin(s->device, nullptr)) cudaEventElapsedTime(&gather_begin, origin, s->ev[2]);
        }
    }
    // Next group's grids follow what this one really produced (with headroom).
    uint64_t mx_nodes = 0, mx_items[AG_MAX_HOPS + 2] = {0};
    for (uint32_t b = 0; b < s->in_flight_n; ++b) {
        const ag_sample_counts &c = s->counts_host[b];
        mx_nodes = std::max<uint64_t>(mx_nodes, c.num_nodes);
        for (uint32_t h = 0; h < c.num_hops && h < AG_MAX_HOPS; ++h)
            mx_items[h + 1] = std::max<uint64_t>(mx_items[h + 1], c.edges_per_hop[h]);
    }
    s->est_nodes = mx_nodes + mx_nodes / 4 + 256;
    s->est_rows_tight = mx_nodes + mx_nodes / 16 + 64;
    for (uint32_t h = 1; h <= s->cfg.num_hops; ++h) s->est_items[h] = mx_items[h] + mx_items[h] / 4 + 512;
    int32_t first = AG_OK;
    for (uint32_t b = 0; b < s->in_flight_n; ++b) {
        ag_sample_counts c = s->counts_host[b];
        c.sample_ms = sample_ms / s->in_flight_n;
        c.gather_ms = gather_ms / s->in_flight_n;
        c.gather_begin_ms = gather_begin;
        c.gather_end_ms = (double)gather_begin + gather_ms;
        if (counts) counts[b] = c;
        int32_t st = AG_OK;
        if (c.error & kErrBadSeed) st = fail(AG_ERR_SAMPLING, "a seed node is out of range for %llu nodes", (unsigned long long)s->g->num_nodes);
        else if (c.error & kErrCapacity) st = fail(AG_ERR_VALUE, "output buffers too small for the sampled subgraph");
        else if (c.error & kErrBadDst) st = fail(AG_ERR_LOAD, "graph holds a destination outside [0, num_nodes); load it with full validation");
        else if (c.error) st = fail(AG_ERR_WORKER, "sampler kernels reported error bits 0x%x", c.error);
        if (st != AG_OK && (c.error & (kErrSpinTimeout | kErrTableFull))) s->dirty = true;
        if (statuses) statuses[b] = st;
        if (st != AG_OK && first == AG_OK) first = st;
    }
    return first;
}

extern "C" int32_t ag_sample_into(ag_sampler *s, const uint32_t *seeds, uint64_t n_seeds, int32_t seeds_mem,
                                  const ag_features *feats, ag_subgraph_buffers *buf, void *stream) {
    if (!s || !buf || (!seeds && n_seeds)) return fail(AG_ERR_VALUE, "ag_sample_into: null argument");
    const uint32_t *sp[1] = {seeds};
    const uint64_t ns[1] = {n_seeds};
    return ag_sample_group_into(s, 1, sp, ns, seeds_mem, nullptr, feats, buf, stream);
}

extern "C" int32_t ag_sample_wait(ag_sampler *s, ag_sample_counts *counts) {
    if (s && s->in_flight && s->in_flight_n != 1) return fail(AG_ERR_VALUE, "ag_sample_wait: a group is in flight; use ag_sample_group_wait");
    return ag_sample_group_wait(s, counts, nullptr);
}

extern "C" int32_t ag_sample(ag_sampler *s, const uint32_t *seeds, uint64_t n_seeds, const ag_features *feats,
                             int32_t want_int64, ag_subgraph_buffers *buf, void *stream) {
    if (!s || !buf) return fail(AG_ERR_VALUE, "ag_sample: null argument");
    DeviceGuard guard(s->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint64_t mn, me;
    compute_bounds(s, n_seeds, &mn, &me, nullptr);
    ag_subgraph_buffers b{};
    b.cap_nodes = std::max<uint64_t>(mn, 1); b.cap_edges = std::max<uint64_t>(me, 1);
    b.cap_seeds = std::max<uint64_t>(n_seeds, 1);
    std::vector<void *> mine;
    auto alloc = [&](void **ptr, uint64_t bytes) -> bool {
        if (cudaMalloc(ptr, bytes) != cudaSuccess) return false;
        mine.push_back(*ptr);
        return true;
    };
    bool ok = alloc((void **)&b.nodes, b.cap_nodes * 4) && alloc((void **)&b.edge_src, b.cap_edges * 4) &&
              alloc((void **)&b.edge_dst, b.cap_edges * 4) && alloc((void **)&b.src_local, b.cap_edges * 4) &&
              alloc((void **)&b.dst_local, b.cap_edges * 4) && alloc((void **)&b.seed_locals, b.cap_seeds * 4);
    if (ok && s->cfg.track_edge_ids) ok = alloc((void **)&b.edge_ids, b.cap_edges * 8);
    if (ok && want_int64) {
        ok = alloc((void **)&b.n_id, b.cap_nodes * 8) && alloc((void **)&b.edge_index_local, b.cap_edges * 16) &&
             alloc((void **)&b.seed_index, b.cap_seeds * 8);
        if (ok && s->cfg.track_edge_ids) ok = alloc((void **)&b.e_id, b.cap_edges * 8);
    }
    if (ok && feats) ok = alloc((void **)&b.x, b.cap_nodes * feats->dim * 4);
    if (!ok) {
        for (void *q : mine) cudaFree(q);
        return fail(AG_ERR_CUDA, "ag_sample: out of device memory: %s", cudaGetErrorString(cudaGetLastError()));
    }
    const int32_t st = ag_sample_into(s, seeds, n_seeds, AG_MEM_HOST, feats, &b, stream);
    if (st != AG_OK) { for (void *q : mine) cudaFree(q); return st; }
    s->owned.insert(s->owned.end(), mine.begin(), mine.end());
    *buf = b;
    return AG_OK;
}

extern "C" int32_t ag_subgraph_release(ag_sampler *s, ag_subgraph_buffers *buf) {
    if (!s || !buf) return fail(AG_ERR_VALUE, "ag_subgraph_release: null argument");
    DeviceGuard guard(s->device);
    if (s->in_flight) { cudaEventSynchronize(s->done); }
    void *ptrs[] = {buf->nodes, buf->edge_src, buf->edge_dst, buf->edge_ids, buf->src_local, buf->dst_local,
                    buf->seed_locals, buf->n_id, buf->edge_index_local, buf->e_id, buf->seed_index, buf->x};
    for (void *q : ptrs) {
        if (!q) continue;
        auto it = std::find(s->owned.begin(), s->owned.end(), q);
        if (it != s->owned.end()) { cudaFree(q); s->owned.erase(it); }
    }
    *buf = ag_subgraph_buffers{};
    return AG_OK;
}

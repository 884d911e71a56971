// Device-side building blocks of the sampling kernels: the dedup table, the
// single-pass scan and the per-batch bookkeeping they share.
#pragma once

#include "common.cuh"

namespace ag {

// A vertex discovered in one stage and expanded in the next: everything the
// picks need, kept in shared memory between the two halves of the expand kernel.
struct __align__(16) FrontierEntry {
    uint64_t off;    // first CSR position of the row
    uint64_t dbase;  // absolute index of the vertex's first RNG draw
    uint32_t id;     // vertex id
    uint32_t local;  // local index assigned at discovery
    uint32_t deg;    // row length
    uint32_t ebase;  // first edge slot of the vertex within its hop
};

// Running totals handed from one stage to the next.  Stage 0 is the seed
// registration, stage h + 1 the edges of hop h.  A stage's kernel only reads
// stage[s] and only the last tile writes stage[s + 1], so nothing is read and
// written concurrently.
struct __align__(16) StageInfo {
    uint32_t n_nodes;     // nodes registered before this stage
    uint32_t n_edges;     // edges emitted before this stage
    uint32_t frontier_n;  // vertices this stage discovered (expanded by the next)
    uint32_t hop_edges;   // items of this stage (edges the previous stage emitted)
    uint64_t draws;       // RNG draws consumed before this stage's picks
    uint64_t hop_draws;   // draws this stage's picks consume
};

struct ScanVal {
    uint32_t flags;
    uint32_t take;
    uint64_t draws;
};
__host__ __device__ __forceinline__ ScanVal operator+(const ScanVal &a, const ScanVal &b) {
    return ScanVal{a.flags + b.flags, a.take + b.take, a.draws + b.draws};
}

// Tile descriptor of the single-pass (decoupled look-back) scan.  `status`
// holds (epoch << 2) | state; a launch uses a fresh epoch, so descriptors never
// need clearing between launches.
struct __align__(16) TileDesc {
    uint32_t status;
    uint32_t pad;
    ScanVal agg;
    ScanVal incl;
};
constexpr uint32_t kTileAgg = 1u, kTileIncl = 2u;

struct BatchState {
    StageInfo stage[AG_MAX_HOPS + 2];
    uint32_t nodes_per_stage[AG_MAX_HOPS + 2];
    uint32_t error;
    uint32_t ticket;
    uint64_t stream_pos;  // draws consumed by earlier batches of this handle
    uint32_t done_blocks; // blocks of the last stage's kernel that have finished
    uint32_t pad;
};

// ------------------------------------------------------------ dedup table --
// Open addressing, linear probing, one 64-bit slot per vertex:
//   key (32) | generation (4) | pending (1) | stage (4) | position (23)
// A pending value says "first named at this position of this stage"; once the
// vertex has its local index the value becomes generation | local.  For one key
// and generation the integer order of the value is exactly the order the
// sequential reference meets the vertex in: assigned < pending of an earlier
// stage < pending of a later stage, then by position.  atomicMin therefore
// keeps the first sighting.  A slot whose generation is not the current one is
// free: a handle bumps the generation per launch instead of clearing the table
// and clears it for real once per 15 launches (generation 15 is the empty mark).
constexpr uint64_t kSlotEmpty = 0xFFFFFFFFFFFFFFFFull;
constexpr uint32_t kGenShift = 28, kPendingBit = 1u << 27, kStageShift = 23;
constexpr uint32_t kPosMask = (1u << 23) - 1u;
constexpr uint32_t kGens = 15;
constexpr uint64_t kMaxPos = 1ull << 23;  // items per stage and nodes per batch

__host__ __device__ __forceinline__ uint32_t enc_pending(uint32_t gen, uint32_t stage, uint32_t pos) {
    return (gen << kGenShift) | kPendingBit | (stage << kStageShift) | pos;
}
__host__ __device__ __forceinline__ uint32_t enc_final(uint32_t gen, uint32_t local) {
    return (gen << kGenShift) | local;
}

// Bounded polling: ~2^20 polls with a short sleep is on the order of 100 ms,
// far beyond any legitimate wait between tiles of one launch.
constexpr uint32_t kSpinLimit = 1u << 20;

#ifdef __CUDACC__

struct DedupTable {
    uint64_t *slots;
    uint32_t mask;
    uint32_t shift;  // 32 - log2(capacity)
    uint32_t gen;
};

__device__ __forceinline__ uint32_t table_hash(uint32_t key, uint32_t shift) {
    return (key * 0x9E3779B1u) >> shift;
}

// Inserts (key, val) keeping the minimum val per key; returns the slot index.
__device__ __forceinline__ uint32_t table_insert_min(const DedupTable &t, uint32_t key,
                                                     uint32_t val, uint32_t *err) {
    const unsigned long long mine = ((unsigned long long)key << 32) | val;
    uint32_t h = table_hash(key, t.shift);
    for (uint32_t probe = 0; probe <= t.mask; ++probe) {
        unsigned long long *slot = (unsigned long long *)&t.slots[h];
        unsigned long long cur = __ldcg(slot);
        // free (never used, or left over from an older generation): claim it
        while (((uint32_t)cur >> kGenShift) != t.gen) {
            const unsigned long long prev = atomicCAS(slot, cur, mine);
            if (prev == cur) return h;
            cur = prev;
        }
        if ((uint32_t)(cur >> 32) == key) {
            if ((uint32_t)cur > val) atomicMin(slot, mine);
            return h;
        }
        h = (h + 1) & t.mask;
    }
    atomicOr(err, kErrTableFull);
    return 0xFFFFFFFFu;
}

__device__ __forceinline__ ScanVal warp_inclusive_scan(ScanVal v, int lane) {
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t f = __shfl_up_sync(0xffffffffu, v.flags, o);
        const uint32_t t = __shfl_up_sync(0xffffffffu, v.take, o);
        const uint64_t d = __shfl_up_sync(0xffffffffu, v.draws, o);
        if (lane >= o) { v.flags += f; v.take += t; v.draws += d; }
    }
    return v;
}

__device__ __forceinline__ ScanVal warp_reduce(ScanVal v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v.flags += __shfl_xor_sync(0xffffffffu, v.flags, o);
        v.take += __shfl_xor_sync(0xffffffffu, v.take, o);
        v.draws += __shfl_xor_sync(0xffffffffu, v.draws, o);
    }
    return v;
}

// Called by warp 0 of a tile once its aggregate is known.  Publishes the
// aggregate, walks back over the predecessors' descriptors 32 at a time until
// an inclusive prefix is found, publishes this tile's inclusive prefix and
// returns the exclusive one.  Tiles get their index from a ticket counter, so
// every predecessor is already running.  Each poll loop is bounded; on timeout
// the error bit is raised and the missing value is treated as zero.
__device__ __forceinline__ ScanVal lookback_exclusive(TileDesc *tiles, uint32_t tile, uint32_t epoch,
                                                      ScanVal agg, int lane, uint32_t *err) {
    ScanVal prefix{0, 0, 0};
    if (tile == 0) {
        if (lane == 0) {
            tiles[0].agg = agg;
            tiles[0].incl = agg;
            st_release_u32(&tiles[0].status, (epoch << 2) | kTileIncl);
        }
        return prefix;
    }
    if (lane == 0) {
        tiles[tile].agg = agg;
        st_release_u32(&tiles[tile].status, (epoch << 2) | kTileAgg);
    }
    int look = (int)tile - 1;
    for (;;) {
        const int t = look - lane;
        uint32_t state = kTileIncl;
        ScanVal v{0, 0, 0};
        if (t >= 0) {
            uint32_t st = 0, spins = 0;
            for (;;) {
                st = ld_acquire_u32(&tiles[t].status);
                if ((st >> 2) == epoch && (st & 3u) != 0) break;
                if (++spins > kSpinLimit) { atomicOr(err, kErrSpinTimeout); st = (epoch << 2) | kTileIncl; break; }
                __nanosleep(32);
            }
            state = st & 3u;
            if (spins <= kSpinLimit) v = (state == kTileIncl) ? tiles[t].incl : tiles[t].agg;
        }
        const uint32_t incl_mask = __ballot_sync(0xffffffffu, state == kTileIncl);
        const int first = __ffs(incl_mask) - 1;  // nearest predecessor holding an inclusive prefix
        if (first >= 0 && lane > first) v = ScanVal{0, 0, 0};
        prefix = prefix + warp_reduce(v);
        if (first >= 0) break;
        look -= 32;
    }
    if (lane == 0) {
        tiles[tile].incl = prefix + agg;
        st_release_u32(&tiles[tile].status, (epoch << 2) | kTileIncl);
    }
    return prefix;
}

#endif  // __CUDACC__

}  // namespace ag

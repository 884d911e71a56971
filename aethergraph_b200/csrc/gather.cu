// Feature-row gather with fused f16/bf16 -> f32 upcast.
//
// Follows FeatureStore::get_batch_into of the reference
// (crates/aethergraph-core/src/features/store.rs:777-838; row decoders
// features/header.rs:110-116, internal/simd.rs:97-101,233-238): output row i is
// the decoded stored row ids[i], in ids order, duplicates re-read.
//
// Shape.  The path is HBM-bound byte movement: per output row it reads
// row_bytes (a whole number of 32-byte sectors when rows are 32-byte aligned)
// and writes dim * 4 bytes.  A row is split into 16-byte vectors; a group of
// LPR lanes (the power of two >= vectors-per-row, at most 32) owns one row, so
// a warp reads 32/LPR rows with fully coalesced 16-byte loads.  Every thread
// issues kInFlight independent row loads before it converts or stores any of
// them, which keeps >= 2 KB per warp in flight — enough to cover HBM latency at
// full occupancy.  Loads bypass L1 (rows are touched once); stores are
// evict-first.  The grid is a whole number of waves of the 148 SMs and strides
// over the rows, so the row count may live on the device (the sampler's node
// count) without a host round trip.
#include <algorithm>

#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "internal.h"

namespace ag {

namespace {

constexpr int kThreads = 256;
constexpr int kInFlight = 4;

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }

// IEEE binary16 -> binary32, exact; a NaN keeps its payload and comes out quiet
// (what the reference's half / F16C converters produce).
__device__ __forceinline__ float f16_to_f32_bits(uint32_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    const uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    if (exp == 0x1Fu) return __uint_as_float(man ? (sign | 0x7FC00000u | (man << 13)) : (sign | 0x7F800000u));
    if (exp == 0) {
        if (man == 0) return __uint_as_float(sign);
        const int shift = __clz(man) - 21;  // bring the top set bit to bit 10
        man = (man << shift) & 0x3FFu;
        return __uint_as_float(sign | ((uint32_t)(113 - shift) << 23) | (man << 13));
    }
    return __uint_as_float(sign | ((exp + 112u) << 23) | (man << 13));
}

template <int DTYPE>
__device__ __forceinline__ void store_decoded(float *dst, uint4 v) {
    if (DTYPE == AG_F32) {
        st_stream_v4(dst, v);
    } else if (DTYPE == AG_BF16) {
        uint4 a, b;
        a.x = v.x << 16; a.y = v.x & 0xFFFF0000u; a.z = v.y << 16; a.w = v.y & 0xFFFF0000u;
        b.x = v.z << 16; b.y = v.z & 0xFFFF0000u; b.z = v.w << 16; b.w = v.w & 0xFFFF0000u;
        st_stream_v4(dst, a);
        st_stream_v4(dst + 4, b);
    } else {
        uint4 a, b;
        a.x = __float_as_uint(f16_to_f32_bits(v.x & 0xFFFFu)); a.y = __float_as_uint(f16_to_f32_bits(v.x >> 16));
        a.z = __float_as_uint(f16_to_f32_bits(v.y & 0xFFFFu)); a.w = __float_as_uint(f16_to_f32_bits(v.y >> 16));
        b.x = __float_as_uint(f16_to_f32_bits(v.z & 0xFFFFu)); b.y = __float_as_uint(f16_to_f32_bits(v.z >> 16));
        b.z = __float_as_uint(f16_to_f32_bits(v.w & 0xFFFFu)); b.w = __float_as_uint(f16_to_f32_bits(v.w >> 16));
        st_stream_v4(dst, a);
        st_stream_v4(dst + 4, b);
    }
}

__device__ __forceinline__ uint64_t load_id(const void *ids, int ids64, uint64_t i) {
    return ids64 ? (uint64_t)((const int64_t *)ids)[i] : (uint64_t)((const uint32_t *)ids)[i];
}

// Feature rows are read once per batch and there are tens of gigabytes of them:
// mark their lines evict-first in L2 as well, so the stream of rows does not push
// out what the sampling kernels of the neighbouring chains keep there (dedup
// tables, scan descriptors, CSR offsets).
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint4 ld_stream_v4_l2ef(const void *p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
    return v;
}

// Plain (coherent) 16-byte load that does not allocate in L1: rows of a peer
// GPU's shard arrive over NVLink through this.
__device__ __forceinline__ uint4 ld_peer_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// Where row `id` of a sharded store lives: shard id / shard_rows, which is this
// GPU's own memory or a peer's (vertex-range shards of equal size).
__device__ __forceinline__ const uint8_t *shard_row(const ag_shard_table *t, uint64_t id, uint32_t row_bytes) {
    if (t->cyclic) {  // rows dealt round-robin: hot vertex ranges spread over all GPUs
        const uint64_t s = id % t->n_shards;
        return t->base[s] + (id / t->n_shards) * row_bytes;
    }
    const uint64_t s = id / t->shard_rows;
    return t->base[s] + (id - s * t->shard_rows) * row_bytes;
}

// Vector path: row_bytes % 16 == 0 and the payload base is 16-byte aligned.
// LPR lanes share a row; vecs = row_bytes / 16.  SHARDED: the store is split by
// vertex range over several GPUs and every row is fetched straight from its
// owner's memory (local HBM or a peer over NVLink), upcast at the reader.
template <int DTYPE, int LPR, bool SHARDED>
__global__ void __launch_bounds__(kThreads)
k_gather_vec(GatherArgs a, const GatherArgs *__restrict__ group, uint64_t first) {
    constexpr int kRowsPerBlock = kThreads / LPR;
    if (group) a = group[blockIdx.y];  // one batch of a group per grid row
    if (!a.payload) return;
    const uint64_t n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;  // a segment of a longer id array
    const int lane = threadIdx.x % LPR;
    const int sub = threadIdx.x / LPR;
    const uint32_t vecs = a.row_bytes >> 4;
    const uint32_t out_per_vec = (DTYPE == AG_F32) ? 4u : 8u;  // floats per 16-byte vector
    // A block owns chunks of kRowsPerBlock * kInFlight consecutive rows.  With a
    // grid of about one chunk per block the blocks are short-lived, so blocks of
    // a concurrent (higher-priority) kernel get SM slots as they retire.
    constexpr uint64_t kChunk = (uint64_t)kRowsPerBlock * kInFlight;
    const uint64_t stride = kRowsPerBlock;
    const uint64_t pol = l2_evict_first_policy();

    // `first`: rows before it are somebody else's (the sorted gather's overflow pass).
    for (uint64_t base = first + (uint64_t)blockIdx.x * kChunk + sub; base < n; base += (uint64_t)gridDim.x * kChunk) {
        for (uint32_t v0 = 0; v0 < vecs; v0 += LPR) {
            const uint32_t v = v0 + lane;
            uint4 val[kInFlight];
            bool ok[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const uint64_t r = base + (uint64_t)u * stride;
                ok[u] = false;
                val[u] = make_uint4(0, 0, 0, 0);
                if (r < n && v < vecs) {
                    const uint64_t id = load_id(a.ids, a.ids64, r);
                    const uint64_t local = id - a.row_begin;
                    ok[u] = true;
                    if (id >= a.row_begin && local < a.rows) {
                        if (SHARDED) val[u] = ld_peer_v4(shard_row(a.shards, id, a.row_bytes) + ((uint64_t)v << 4));
                        else val[u] = ld_stream_v4_l2ef(a.payload + local * a.row_bytes + ((uint64_t)v << 4), pol);
                    } else if (lane == 0) {
                        atomicOr(a.err, kErrBadId);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (ok[u]) {
                    const uint64_t r = base + (uint64_t)u * stride;
                    store_decoded<DTYPE>(a.out + r * a.dim + (uint64_t)v * out_per_vec, val[u]);
                }
            }
        }
    }
}

// Element path for rows that are not a whole number of 16-byte vectors.
template <int DTYPE>
__global__ void __launch_bounds__(kThreads)
k_gather_elem(GatherArgs a, const GatherArgs *__restrict__ group) {
    if (group) a = group[blockIdx.y];
    if (!a.payload) return;
    const uint64_t n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;
    const uint64_t total = n * a.dim;
    for (uint64_t g = (uint64_t)blockIdx.x * kThreads + threadIdx.x; g < total;
         g += (uint64_t)gridDim.x * kThreads) {
        const uint64_t r = g / a.dim;
        const uint32_t j = (uint32_t)(g - r * a.dim);
        const uint64_t id = load_id(a.ids, a.ids64, r);
        const uint64_t local = id - a.row_begin;
        float f = 0.f;
        if (id >= a.row_begin && local < a.rows) {
            if (a.shards) {  // sharded store: plain loads from the owner's memory
                const uint8_t *row = shard_row(a.shards, id, a.row_bytes);
                if (DTYPE == AG_F32) f = __uint_as_float(*(const volatile uint32_t *)(row + 4ull * j));
                else if (DTYPE == AG_BF16) f = bf16lo(*(const volatile uint16_t *)(row + 2ull * j));
                else f = f16_to_f32_bits(*(const volatile uint16_t *)(row + 2ull * j));
            } else {
                const uint8_t *row = a.payload + local * a.row_bytes;
                if (DTYPE == AG_F32) f = __uint_as_float(ld_stream_u32(row + 4ull * j));
                else if (DTYPE == AG_BF16) f = bf16lo(ld_stream_u16(row + 2ull * j));
                else f = f16_to_f32_bits(ld_stream_u16(row + 2ull * j));
            }
        } else if (j == 0) {
            atomicOr(a.err, kErrBadId);
        }
        a.out[g] = f;
    }
}

template <int DTYPE, bool SHARDED>
cudaError_t launch_vec_s(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, dim3 grid, cudaStream_t st,
                         uint64_t first) {
    const uint32_t vecs = row_bytes >> 4;
    if (vecs <= 4) k_gather_vec<DTYPE, 4, SHARDED><<<grid, kThreads, 0, st>>>(a, group, first);
    else if (vecs <= 8) k_gather_vec<DTYPE, 8, SHARDED><<<grid, kThreads, 0, st>>>(a, group, first);
    else if (vecs <= 16) k_gather_vec<DTYPE, 16, SHARDED><<<grid, kThreads, 0, st>>>(a, group, first);
    else k_gather_vec<DTYPE, 32, SHARDED><<<grid, kThreads, 0, st>>>(a, group, first);
    return cudaGetLastError();
}

template <int DTYPE>
cudaError_t launch_vec(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, dim3 grid, bool sharded,
                       cudaStream_t st, uint64_t first = 0) {
    return sharded ? launch_vec_s<DTYPE, true>(a, group, row_bytes, grid, st, first)
                   : launch_vec_s<DTYPE, false>(a, group, row_bytes, grid, st, first);
}

// f32 -> stored dtype, used to build a store from f32 rows on the device.
// bf16: round to nearest even on the dropped 16 bits, NaN -> (bits >> 16) | 0x40
// (reference: features/store.rs:1094-1104).  f16: IEEE RNE (__float2half_rn),
// NaN -> sign | 0x7E00 | (mantissa >> 13) as the reference's half crate does.
__global__ void k_encode(const float *src, uint16_t *dst, uint64_t count, int dtype) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t bits = __float_as_uint(src[i]);
        uint16_t o;
        if (dtype == AG_BF16) {
            if ((bits & 0x7FFFFFFFu) > 0x7F800000u) o = (uint16_t)((bits >> 16) | 0x0040u);
            else o = (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
        } else {
            if ((bits & 0x7FFFFFFFu) > 0x7F800000u)
                o = (uint16_t)(((bits >> 16) & 0x8000u) | 0x7E00u | ((bits & 0x7FFFFFu) >> 13));
            else {
                const uint32_t sign = (bits >> 16) & 0x8000u, exp = (bits >> 23) & 0xFFu;
                uint32_t man = bits & 0x7FFFFFu;
                const int e = (int)exp - 112;
                if (exp == 0xFFu || e >= 0x1F) o = (uint16_t)(sign | 0x7C00u);
                else if (e <= 0) {
                    if (e < -10) o = (uint16_t)sign;
                    else {
                        man |= 0x800000u;
                        const uint32_t shift = (uint32_t)(14 - e);
                        uint32_t hm = man >> shift;
                        const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
                        if (rem > half || (rem == half && (hm & 1u))) hm++;
                        o = (uint16_t)(sign | hm);
                    }
                } else {
                    uint32_t h = ((uint32_t)e << 10) | (man >> 13);
                    const uint32_t rem = man & 0x1FFFu;
                    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
                    o = (uint16_t)(sign | h);
                }
            }
        }
        dst[i] = o;
    }
}


// ------------------------------------------------- address-ordered gather --
// A sharded store's remote rows arrive over NVLink through mappings of the
// peers' memory.  Random rows spread over tens of gigabytes of such mappings
// run far below the link's bandwidth (every row needs an address translation
// that is no longer cached); the same rows requested in address order run at
// the link's bandwidth.  So a launch first turns its row ids into address-order
// keys, sorts them (in local memory) together with the output position of each
// row, and gathers in that order.  The f32 rows are still written at their
// original positions in local HBM, where order costs nothing.
//
// key = row-within-shard * W + owner.  Within one owner the rows ascend, and
// neighbouring keys alternate between the owners, so at any moment a GPU pulls
// from all its peers at once (no owner's links are the only ones busy) while
// each owner is still read in ascending address order.  For round-robin shards
// the key IS the vertex id; for contiguous ranges it is (id % S) * W + id / S.
//
// Sorting has a second use: the batches of one launch chain name many rows more
// than once (hub vertices turn up in most batches of a chain).  Equal keys are
// neighbours after the sort, so a row is loaded once — crosses the link once —
// and written to every batch that asked for it.
constexpr uint32_t kValRowBits = 23;  // value = batch << 23 | row: rows per batch < 2^23, batches per chain <= 256

__device__ __forceinline__ uint32_t addr_key(const ag_shard_table *t, uint64_t id) {
    if (t->cyclic) return (uint32_t)id;
    const uint64_t s = id / t->shard_rows;
    return (uint32_t)((id - s * t->shard_rows) * t->n_shards + s);
}

__global__ void __launch_bounds__(256)
k_make_keys(GatherArgs a, const GatherArgs *__restrict__ group, uint32_t rows_cap, uint32_t sentinel,
            uint32_t *__restrict__ keys, uint32_t *__restrict__ vals) {
    if (group) a = group[blockIdx.y];
    uint64_t n = 0;
    if (a.payload) n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;
    const uint64_t slot0 = (uint64_t)blockIdx.y * rows_cap;
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < rows_cap; r += gridDim.x * blockDim.x) {
        uint32_t key = sentinel;  // slots past the batch's rows sort to the end
        if (r < n) {
            const uint64_t id = load_id(a.ids, a.ids64, r);
            if (id >= a.row_begin && id - a.row_begin < a.rows) key = addr_key(a.shards, id);
            else atomicOr(a.err, kErrBadId);
        }
        keys[slot0 + r] = key;
        vals[slot0 + r] = (blockIdx.y << kValRowBits) | r;
    }
}

template <int DTYPE, int LPR>
__global__ void __launch_bounds__(kThreads)
k_gather_sorted(GatherArgs one, const GatherArgs *__restrict__ group, const ag_shard_table *__restrict__ t,
                const uint32_t *__restrict__ keys, const uint32_t *__restrict__ vals, uint64_t n_items,
                uint32_t sentinel, uint32_t row_bytes, uint32_t dim, unsigned long long *__restrict__ counters) {
    constexpr int kRowsPerBlock = kThreads / LPR;
    uint32_t asked = 0, loaded = 0;  // counted by lane 0 of each row group
    constexpr uint64_t kChunk = (uint64_t)kRowsPerBlock * kInFlight;
    const int lane = threadIdx.x % LPR;
    const int sub = threadIdx.x / LPR;
    const uint32_t vecs = row_bytes >> 4;
    const uint32_t out_per_vec = (DTYPE == AG_F32) ? 4u : 8u;
    const uint32_t W = t->n_shards;
    for (uint64_t chunk0 = (uint64_t)blockIdx.x * kChunk; chunk0 < n_items; chunk0 += (uint64_t)gridDim.x * kChunk) {
        if (keys[chunk0] == sentinel) return;  // sorted: nothing but padding from here on
        const uint64_t base = chunk0 + sub;
        for (uint32_t v0 = 0; v0 < vecs; v0 += LPR) {
            const uint32_t v = v0 + lane;
            uint4 val[kInFlight];
            uint32_t key[kInFlight];
            bool head[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const uint64_t i = base + (uint64_t)u * kRowsPerBlock;
                head[u] = false;
                val[u] = make_uint4(0, 0, 0, 0);
                key[u] = sentinel;
                if (i < n_items && v < vecs) {
                    key[u] = keys[i];
                    // the first of a run of equal keys fetches the row for the whole run
                    head[u] = key[u] != sentinel && (i == 0 || keys[i - 1] != key[u]);
                    if (lane == 0 && v0 == 0) { asked += key[u] != sentinel; loaded += head[u]; }
                    if (head[u]) {
                        const uint32_t owner = key[u] % W;
                        const uint64_t local = key[u] / W;
                        val[u] = ld_peer_v4(t->base[owner] + local * row_bytes + ((uint64_t)v << 4));
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (!head[u]) continue;
                uint64_t j = base + (uint64_t)u * kRowsPerBlock;
                do {
                    const uint32_t pv = vals[j];
                    float *out = group ? group[pv >> kValRowBits].out : one.out;
                    store_decoded<DTYPE>(out + (uint64_t)(pv & ((1u << kValRowBits) - 1u)) * dim + (uint64_t)v * out_per_vec, val[u]);
                    ++j;
                } while (j < n_items && keys[j] == key[u]);
            }
        }
    }
    if (asked) { atomicAdd(counters, (unsigned long long)asked); atomicAdd(counters + 1, (unsigned long long)loaded); }
}

template <int DTYPE>
cudaError_t launch_sorted(const GatherArgs &one, const GatherArgs *group, const ag_shard_table *t, const uint32_t *keys,
                          const uint32_t *vals, uint64_t n_items, uint32_t sentinel, uint32_t row_bytes, uint32_t dim,
                          int blocks, unsigned long long *counters, cudaStream_t st) {
    const uint32_t vecs = row_bytes >> 4;
    if (vecs <= 4) k_gather_sorted<DTYPE, 4><<<blocks, kThreads, 0, st>>>(one, group, t, keys, vals, n_items, sentinel, row_bytes, dim, counters);
    else if (vecs <= 8) k_gather_sorted<DTYPE, 8><<<blocks, kThreads, 0, st>>>(one, group, t, keys, vals, n_items, sentinel, row_bytes, dim, counters);
    else if (vecs <= 16) k_gather_sorted<DTYPE, 16><<<blocks, kThreads, 0, st>>>(one, group, t, keys, vals, n_items, sentinel, row_bytes, dim, counters);
    else k_gather_sorted<DTYPE, 32><<<blocks, kThreads, 0, st>>>(one, group, t, keys, vals, n_items, sentinel, row_bytes, dim, counters);
    return cudaGetLastError();
}

uint32_t bit_width_u64(uint64_t v) {
    uint32_t b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

}  // namespace

int gather_grid_blocks(uint64_t n, uint32_t row_bytes) {
    // One chunk of rows per block, up to 64 blocks per SM's worth of grid; past
    // that the blocks stride over further chunks.
    const uint32_t vecs = row_bytes >> 4;
    const int lpr = vecs <= 4 ? 4 : vecs <= 8 ? 8 : vecs <= 16 ? 16 : 32;
    const uint64_t rows_per_block = (uint64_t)(kThreads / lpr) * kInFlight;
    const uint64_t need = std::max<uint64_t>(1, (n + rows_per_block - 1) / rows_per_block);
    return (int)std::min<uint64_t>(need, (uint64_t)kSMs * 64);
}

cudaError_t launch_gather(const GatherArgs &a, int dtype, cudaStream_t st) {
    if (a.n == 0) return cudaSuccess;
    const bool vec_ok = (a.row_bytes % 16 == 0) && (((uintptr_t)a.payload) % 16 == 0) &&
                        (((uintptr_t)a.out) % 16 == 0);
    if (vec_ok) {
        const dim3 grid(gather_grid_blocks(a.n, a.row_bytes), 1);
        switch (dtype) {
            case AG_F32: return launch_vec<AG_F32>(a, nullptr, a.row_bytes, grid, a.shards != nullptr, st);
            case AG_F16: return launch_vec<AG_F16>(a, nullptr, a.row_bytes, grid, a.shards != nullptr, st);
            default: return launch_vec<AG_BF16>(a, nullptr, a.row_bytes, grid, a.shards != nullptr, st);
        }
    }
    const uint64_t total = a.n * a.dim;
    uint64_t blocks = (total + kThreads - 1) / kThreads;
    if (blocks > (uint64_t)kSMs * 8) blocks = (uint64_t)kSMs * 8;
    switch (dtype) {
        case AG_F32: k_gather_elem<AG_F32><<<(int)blocks, kThreads, 0, st>>>(a, nullptr); break;
        case AG_F16: k_gather_elem<AG_F16><<<(int)blocks, kThreads, 0, st>>>(a, nullptr); break;
        default: k_gather_elem<AG_BF16><<<(int)blocks, kThreads, 0, st>>>(a, nullptr); break;
    }
    return cudaGetLastError();
}

// One launch for a group of batches: grid row b gathers the batch described by
// group_dev[b].  The output buffers come from cudaMalloc / the torch allocator
// (256- / 512-byte aligned) and the payload base is checked by the caller's
// store, so only the row size decides between the vector and the element path.
cudaError_t launch_gather_group(const GatherArgs *group_dev, uint32_t n_batches, uint32_t row_bytes,
                                uint32_t dim, uint64_t n_bound, bool aligned, int dtype, bool sharded,
                                cudaStream_t st) {
    if (n_batches == 0 || n_bound == 0) return cudaSuccess;
    GatherArgs none{};
    if (row_bytes % 16 == 0 && aligned) {
        // n_bound is the caller's estimate of the rows per batch (the true count is
        // read on the device); a batch with more rows strides over extra chunks.
        int per = gather_grid_blocks(n_bound, row_bytes);
        const int cap = std::max(1, (kSMs * 64 + (int)n_batches - 1) / (int)n_batches);
        per = std::min(per, cap);
        const dim3 grid(per, n_batches);
        switch (dtype) {
            case AG_F32: return launch_vec<AG_F32>(none, group_dev, row_bytes, grid, sharded, st);
            case AG_F16: return launch_vec<AG_F16>(none, group_dev, row_bytes, grid, sharded, st);
            default: return launch_vec<AG_BF16>(none, group_dev, row_bytes, grid, sharded, st);
        }
    }
    const uint64_t total = n_bound * dim;
    uint64_t blocks = (total + kThreads - 1) / kThreads;
    blocks = std::max<uint64_t>(1, std::min<uint64_t>(blocks, (uint64_t)kSMs * 8 / n_batches + 1));
    const dim3 grid((uint32_t)blocks, n_batches);
    switch (dtype) {
        case AG_F32: k_gather_elem<AG_F32><<<grid, kThreads, 0, st>>>(none, group_dev); break;
        case AG_F16: k_gather_elem<AG_F16><<<grid, kThreads, 0, st>>>(none, group_dev); break;
        default: k_gather_elem<AG_BF16><<<grid, kThreads, 0, st>>>(none, group_dev); break;
    }
    return cudaGetLastError();
}

// ------------------------------------------------ sorted gather, host side --
void SortScratch::release() {
    cudaFree(keys[0]); cudaFree(keys[1]); cudaFree(vals[0]); cudaFree(vals[1]); cudaFree(temp);
    keys[0] = keys[1] = vals[0] = vals[1] = nullptr; temp = nullptr;
    cap = 0; temp_bytes = 0;
}

cudaError_t SortScratch::ensure(uint64_t items) {
    if (items <= cap) return cudaSuccess;
    release();
    const uint64_t want = items + items / 4 + 1024;  // grow with headroom: the estimate moves from chain to chain
    size_t tb = 0;
    cudaError_t e = cub::DeviceRadixSort::SortPairs(nullptr, tb, (const uint32_t *)nullptr, (uint32_t *)nullptr,
                                                    (const uint32_t *)nullptr, (uint32_t *)nullptr, want, 0, 32, (cudaStream_t)0);
    if (e != cudaSuccess) return e;
    for (int i = 0; i < 2 && e == cudaSuccess; ++i) {
        e = cudaMalloc(&keys[i], want * 4);
        if (e == cudaSuccess) e = cudaMalloc(&vals[i], want * 4);
    }
    if (e == cudaSuccess) e = cudaMalloc(&temp, std::max<size_t>(tb, 16));
    if (e != cudaSuccess) { release(); return e; }
    cap = want; temp_bytes = tb;
    return cudaSuccess;
}

bool sorted_gather_applies(const ag_features *f, uint32_t row_bytes, bool aligned) {
    static const bool enabled = [] {
        const char *v = getenv("AG_GATHER_SORTED");  // "0": keep the unsorted peer-load gather (A/B measurements)
        return !(v && v[0] == '0');
    }();
    if (!enabled || !f || !f->shards || f->n_shards < 2 || !aligned || row_bytes % 16 != 0) return false;
    // keys are 32 bits and one value above the largest key is the padding mark
    return f->shard_rows * f->n_shards < 0xFFFFFFFFull;
}

// The address-ordered gather in two steps, so that a caller can put them on different
// streams (small latency-bound kernels first, the bandwidth-bound fetch behind an event).
// Step 1: keys of rows [0, min(n_b, rows_cap)) of every batch, sorted with their output
// positions.  Step 2: fetch in that order, then rows [rows_cap, n_b) — only present when a
// batch outgrew the caller's estimate — with the unsorted kernel.  `one` / `group_dev` as
// in launch_gather / launch_gather_group.
cudaError_t launch_sort_keys(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                             const ag_features *f, SortScratch &sc, cudaStream_t st) {
    if (n_batches == 0 || rows_cap == 0) return cudaSuccess;
    rows_cap = std::min<uint64_t>(rows_cap, (1ull << kValRowBits) - 1);
    const uint64_t n_items = (uint64_t)n_batches * rows_cap;
    cudaError_t e = sc.ensure(n_items);
    if (e != cudaSuccess) return e;
    const uint64_t max_key = f->shard_rows * f->n_shards;  // one past the largest key
    const uint32_t bits = bit_width_u64(max_key);
    const uint32_t sentinel = bits >= 32 ? 0xFFFFFFFFu : ((1u << bits) - 1u);
    const uint32_t kb = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((rows_cap + 255) / 256, std::max<uint64_t>(1, (uint64_t)kSMs * 8 / n_batches)));
    k_make_keys<<<dim3(kb, n_batches), 256, 0, st>>>(one, group_dev, (uint32_t)rows_cap, sentinel, sc.keys[0], sc.vals[0]);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    size_t tb = sc.temp_bytes;
    return cub::DeviceRadixSort::SortPairs(sc.temp, tb, (const uint32_t *)sc.keys[0], sc.keys[1], (const uint32_t *)sc.vals[0],
                                           sc.vals[1], n_items, 0, (int)bits, st);
}

cudaError_t launch_sorted_fetch(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                                uint32_t row_bytes, uint32_t dim, int dtype, const ag_features *f, SortScratch &sc,
                                cudaStream_t st) {
    if (n_batches == 0 || rows_cap == 0) return cudaSuccess;
    rows_cap = std::min<uint64_t>(rows_cap, (1ull << kValRowBits) - 1);
    const uint64_t n_items = (uint64_t)n_batches * rows_cap;
    const uint32_t bits = bit_width_u64(f->shard_rows * f->n_shards);
    const uint32_t sentinel = bits >= 32 ? 0xFFFFFFFFu : ((1u << bits) - 1u);
    const int blocks = gather_grid_blocks(n_items, row_bytes);
    unsigned long long *counters = (unsigned long long *)((uint8_t *)f->err + 8);
    cudaError_t e;
    switch (dtype) {
        case AG_F32: e = launch_sorted<AG_F32>(one, group_dev, f->shards, sc.keys[1], sc.vals[1], n_items, sentinel, row_bytes, dim, blocks, counters, st); break;
        case AG_F16: e = launch_sorted<AG_F16>(one, group_dev, f->shards, sc.keys[1], sc.vals[1], n_items, sentinel, row_bytes, dim, blocks, counters, st); break;
        default: e = launch_sorted<AG_BF16>(one, group_dev, f->shards, sc.keys[1], sc.vals[1], n_items, sentinel, row_bytes, dim, blocks, counters, st); break;
    }
    if (e != cudaSuccess) return e;
    // Rows past the estimate (rare): a few blocks per batch, which stride; most exit at once.
    const dim3 grid(4, n_batches);
    switch (dtype) {
        case AG_F32: return launch_vec<AG_F32>(one, group_dev, row_bytes, grid, true, st, rows_cap);
        case AG_F16: return launch_vec<AG_F16>(one, group_dev, row_bytes, grid, true, st, rows_cap);
        default: return launch_vec<AG_BF16>(one, group_dev, row_bytes, grid, true, st, rows_cap);
    }
}

cudaError_t launch_gather_sorted(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                                 uint32_t row_bytes, uint32_t dim, int dtype, const ag_features *f, SortScratch &sc,
                                 cudaStream_t st) {
    const cudaError_t e = launch_sort_keys(one, group_dev, n_batches, rows_cap, f, sc, st);
    if (e != cudaSuccess) return e;
    return launch_sorted_fetch(one, group_dev, n_batches, rows_cap, row_bytes, dim, dtype, f, sc, st);
}

cudaError_t launch_encode(const float *src, void *dst, uint64_t count, int dtype, cudaStream_t st) {
    if (count == 0) return cudaSuccess;
    if (dtype == AG_F32) return cudaMemcpyAsync(dst, src, count * 4, cudaMemcpyDeviceToDevice, st);
    uint64_t blocks = (count + 255) / 256;
    if (blocks > (uint64_t)kSMs * 8) blocks = (uint64_t)kSMs * 8;
    k_encode<<<(int)blocks, 256, 0, st>>>(src, (uint16_t *)dst, count, dtype);
    return cudaGetLastError();
}

}  // namespace ag

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
#include <mutex>

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

// Where row `id` of a sharded store lives: the local copy of the hot rows, this GPU's
// own shard or a peer's.  `hot` tells the first case.
__device__ __forceinline__ const uint8_t *shard_row(const ag_shard_table *t, uint64_t id, uint32_t row_bytes, bool &hot) {
    hot = false;
    if (t->hot_slot) {  // a hot row has a copy in this GPU's memory
        const uint32_t h = __ldg(t->hot_slot + id);
        if (h != 0xFFFFFFFFu) { hot = true; return t->base[t->n_shards] + (uint64_t)h * row_bytes; }
    }
    if (t->cyclic) {  // rows dealt round-robin: hot vertex ranges spread over all GPUs
        const uint64_t s = id % t->n_shards;
        return t->base[s] + (id / t->n_shards) * row_bytes;
    }
    const uint64_t s = id / t->shard_rows;
    return t->base[s] + (id - s * t->shard_rows) * row_bytes;
}
__device__ __forceinline__ const uint8_t *shard_row(const ag_shard_table *t, uint64_t id, uint32_t row_bytes) {
    bool hot;
    return shard_row(t, id, row_bytes, hot);
}

// Vector path: row_bytes % 16 == 0 and the payload base is 16-byte aligned.
// LPR lanes share a row; vecs = row_bytes / 16.
template <int DTYPE, int LPR>
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
                        val[u] = ld_stream_v4_l2ef(a.payload + local * a.row_bytes + ((uint64_t)v << 4), pol);
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

// Direct gather over a sharded store: every row is fetched straight from where it
// lives — the local copy of the hot rows, this GPU's shard, or a peer's shard over
// NVLink — and upcast at the reader.
//
// A peer's row takes several times longer to arrive than a local one, and finding
// it takes two dependent loads first (the id, then the hot-row slot).  So the work of
// a block is split: one thread per row resolves the row's address into shared memory,
// for the NEXT set of rows, while all lanes have the loads of the current set in
// flight — kPeerWaves rows per lane group, twice the local kernel's — and a block
// walks through kPeerSets sets instead of retiring after one.
constexpr int kPeerWaves = 8;
constexpr int kPeerSets = 4;

template <int DTYPE, int LPR>
__global__ void __launch_bounds__(kThreads, 3)
k_gather_peer(GatherArgs a, const GatherArgs *__restrict__ group, uint64_t first) {
    constexpr int kRowsPerWave = kThreads / LPR;
    constexpr int kRows = kRowsPerWave * kPeerWaves;  // rows of one set
    __shared__ const uint8_t *s_row[2][kRows];        // where every row of a set starts; null: nothing to fetch
    if (group) a = group[blockIdx.y];  // one batch of a group per grid row
    if (!a.payload) return;
    const uint64_t n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;
    const int lane = threadIdx.x % LPR;
    const int sub = threadIdx.x / LPR;
    const uint32_t vecs = a.row_bytes >> 4;
    const uint32_t out_per_vec = (DTYPE == AG_F32) ? 4u : 8u;
    uint32_t asked = 0, hot_hits = 0;

    // set i covers rows [first + i * kRows, + kRows); a block takes kPeerSets consecutive
    // sets, then the ones a whole grid further on
    auto next_set = [&](uint64_t i) {
        return ((i + 1) % kPeerSets != 0) ? i + 1 : i + 1 + (uint64_t)(gridDim.x - 1) * kPeerSets;
    };
    auto resolve = [&](int buf, uint64_t set) {
        const uint64_t base = first + set * kRows;
        for (int j = threadIdx.x; j < kRows; j += kThreads) {
            const uint64_t r = base + j;
            const uint8_t *p = nullptr;
            if (r < n) {
                const uint64_t id = load_id(a.ids, a.ids64, r);
                if (id >= a.row_begin && id - a.row_begin < a.rows) {
                    bool hot;
                    p = shard_row(a.shards, id, a.row_bytes, hot);
                    ++asked;
                    hot_hits += hot ? 1u : 0u;
                } else {
                    atomicOr(a.err, kErrBadId);
                }
            }
            s_row[buf][j] = p;
        }
    };

    uint64_t set = (uint64_t)blockIdx.x * kPeerSets;
    int buf = 0;
    if (first + set * kRows < n) resolve(0, set);
    __syncthreads();
    while (first + set * kRows < n) {
        const uint64_t base = first + set * kRows;
        const uint64_t following = next_set(set);
        for (uint32_t v0 = 0; v0 < vecs; v0 += LPR) {
            const uint32_t v = v0 + lane;
            uint4 val[kPeerWaves];
            uint32_t ok = 0;  // bit u: row u of this lane group is fetched
            const uint32_t voff = v << 4;
#pragma unroll
            for (int u = 0; u < kPeerWaves; ++u) {
                const uint8_t *p = s_row[buf][u * kRowsPerWave + sub];
                val[u] = make_uint4(0, 0, 0, 0);
                if (p != nullptr && v < vecs) { ok |= 1u << u; val[u] = ld_peer_v4(p + voff); }
            }
            // the addresses of the following set, while this set's rows are on their way
            if (v0 == 0 && first + following * kRows < n) resolve(buf ^ 1, following);
            float *dst = a.out + (base + sub) * a.dim + (uint64_t)v * out_per_vec;
            const uint64_t wave_stride = (uint64_t)kRowsPerWave * a.dim;
#pragma unroll
            for (int u = 0; u < kPeerWaves; ++u) {
                if (ok & (1u << u)) store_decoded<DTYPE>(dst, val[u]);
                dst += wave_stride;
            }
        }
        __syncthreads();  // the following set's addresses are in place, this set's are free to overwrite
        set = following;
        buf ^= 1;
    }
    // the view's counters: rows asked for = rows loaded (nothing is merged), rows served by the hot copy
    for (int o = 16; o > 0; o >>= 1) {
        asked += __shfl_xor_sync(0xffffffffu, asked, o);
        hot_hits += __shfl_xor_sync(0xffffffffu, hot_hits, o);
    }
    if ((threadIdx.x & 31) == 0 && asked) {
        unsigned long long *counters = (unsigned long long *)(a.err + 2);
        atomicAdd(counters, (unsigned long long)asked); atomicAdd(counters + 1, (unsigned long long)asked);
        if (hot_hits) atomicAdd(counters + 2, (unsigned long long)hot_hits);
    }
}

// Block-scaled int8 rows: LPR lanes per row.  A row is a run of 4-byte words (4 codes
// each); lane l of the row's group takes words l, l + LPR, l + 2 LPR, l + 3 LPR, so
// that every load of the group reads LPR consecutive words and every 16-byte store of
// the four decoded floats lands beside its neighbours' (a lane that decoded a whole
// 16-byte vector would write 64 bytes on its own, a quarter of every sector per store
// instruction).  decode = (float)code * scale: one IEEE multiply, the same value the
// reference's BlockScaledI8::decode computes (feature_codec.rs:121-133; its own device
// kernel: crates/aether-stream/src/gpu/kernels/quant/feature_dequant.cu:21-75).
template <int LPR>
__global__ void __launch_bounds__(kThreads)
k_gather_i8(GatherArgs a, const GatherArgs *__restrict__ group, uint64_t first) {
    constexpr int kRowsPerBlock = kThreads / LPR;
    constexpr int kWordsPerLane = 4;
    constexpr int kRowsInFlight = 2;  // x 4 words per lane: eight loads in flight
    if (group) a = group[blockIdx.y];
    if (!a.payload) return;
    const uint64_t n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;
    const int lane = threadIdx.x % LPR;
    const int sub = threadIdx.x / LPR;
    const uint32_t words = a.row_bytes >> 2;                      // 4 codes per word; row_bytes % 16 == 0
    const uint32_t blocks_per_row = (a.dim + kQuantBlock - 1) / kQuantBlock;
    constexpr uint64_t kChunk = (uint64_t)kRowsPerBlock * kInFlight;  // the grid is sized for this many rows per block
    for (uint64_t base = first + (uint64_t)blockIdx.x * kChunk + sub; base < n; base += (uint64_t)gridDim.x * kChunk) {
        for (int u0 = 0; u0 < kInFlight; u0 += kRowsInFlight) {
            for (uint32_t w0 = 0; w0 < words; w0 += LPR * kWordsPerLane) {
                uint32_t val[kRowsInFlight][kWordsPerLane];
                float scale[kRowsInFlight][kWordsPerLane];
                bool ok[kRowsInFlight];
#pragma unroll
                for (int u = 0; u < kRowsInFlight; ++u) {
                    const uint64_t r = base + (uint64_t)(u0 + u) * kRowsPerBlock;
                    ok[u] = false;
                    if (r < n) {
                        const uint64_t id = load_id(a.ids, a.ids64, r);
                        const uint64_t local = id - a.row_begin;
                        if (id >= a.row_begin && local < a.rows) {
                            ok[u] = true;
                            const uint32_t *row = (const uint32_t *)(a.payload + local * a.row_bytes);
                            const float *sc = a.scales + local * blocks_per_row;
#pragma unroll
                            for (int q = 0; q < kWordsPerLane; ++q) {
                                const uint32_t w = w0 + q * LPR + lane;
                                val[u][q] = 0; scale[u][q] = 0.f;
                                if (w < words) {
                                    val[u][q] = __ldg(row + w);
                                    scale[u][q] = __ldg(sc + (w >> 3));  // eight words per 32-element block
                                }
                            }
                        } else if (lane == 0 && w0 == 0) {
                            atomicOr(a.err, kErrBadId);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < kRowsInFlight; ++u) {
                    const uint64_t r = base + (uint64_t)(u0 + u) * kRowsPerBlock;
                    if (r >= n) continue;
                    float *dst = a.out + r * a.dim;
#pragma unroll
                    for (int q = 0; q < kWordsPerLane; ++q) {
                        const uint32_t w = w0 + q * LPR + lane;
                        if (w >= words) continue;
                        uint4 o = make_uint4(0, 0, 0, 0);  // a row outside the store decodes to zeros
                        if (ok[u]) {
                            const uint32_t c = val[u][q];
                            const float sf = scale[u][q];
                            o.x = __float_as_uint((float)(int)(signed char)(c & 0xFFu) * sf);
                            o.y = __float_as_uint((float)(int)(signed char)((c >> 8) & 0xFFu) * sf);
                            o.z = __float_as_uint((float)(int)(signed char)((c >> 16) & 0xFFu) * sf);
                            o.w = __float_as_uint((float)(int)(signed char)(c >> 24) * sf);
                        }
                        st_stream_v4(dst + (uint64_t)w * 4, o);
                    }
                }
            }
        }
    }
}

cudaError_t launch_i8(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, dim3 grid, cudaStream_t st, uint64_t first = 0) {
    const uint32_t vecs = row_bytes >> 4;
    if (vecs <= 4) k_gather_i8<4><<<grid, kThreads, 0, st>>>(a, group, first);
    else if (vecs <= 8) k_gather_i8<8><<<grid, kThreads, 0, st>>>(a, group, first);
    else if (vecs <= 16) k_gather_i8<16><<<grid, kThreads, 0, st>>>(a, group, first);
    else k_gather_i8<32><<<grid, kThreads, 0, st>>>(a, group, first);
    return cudaGetLastError();
}

// f32 -> block-scaled int8 (feature_codec.rs:73-112): a warp per 32-element block.
__global__ void k_encode_i8(const float *__restrict__ src, uint64_t rows, uint64_t dim, int8_t *__restrict__ codes,
                            float *__restrict__ scales, uint32_t *bad) {
    const uint64_t blocks_per_row = (dim + kQuantBlock - 1) / kQuantBlock;
    const uint64_t total = rows * blocks_per_row;
    const int lane = threadIdx.x & 31;
    for (uint64_t b = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < total; b += ((uint64_t)gridDim.x * blockDim.x) >> 5) {
        const uint64_t row = b / blocks_per_row, blk = b - row * blocks_per_row;
        const uint64_t e = blk * kQuantBlock + lane;
        const bool in = e < dim;
        const float v = in ? src[row * dim + e] : 0.f;
        if (in && !isfinite(v)) atomicOr(bad, 1u);
        float peak = fabsf(v);
        for (int o = 16; o > 0; o >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, o));
        const float scale = peak == 0.f ? 0.f : __fdiv_rn(peak, 127.0f);
        if (lane == 0) scales[b] = scale;
        if (in) {
            int q = 0;
            if (scale != 0.f) q = (int)fminf(fmaxf(roundf(__fdiv_rn(v, scale)), -127.0f), 127.0f);  // round half away from zero
            codes[row * dim + e] = (int8_t)q;
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
                else if (DTYPE == AG_I8) f = (float)(int)(signed char)row[j] *
                                             a.scales[local * ((a.dim + kQuantBlock - 1) / kQuantBlock) + j / kQuantBlock];
                else f = f16_to_f32_bits(ld_stream_u16(row + 2ull * j));
            }
        } else if (j == 0) {
            atomicOr(a.err, kErrBadId);
        }
        a.out[g] = f;
    }
}

template <int DTYPE>
cudaError_t launch_vec(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, dim3 grid, bool sharded,
                       cudaStream_t st, uint64_t first = 0) {
    const uint32_t vecs = row_bytes >> 4;
    if (sharded) {
        // `grid.x` counts blocks of kInFlight waves; a block of the peer kernel takes kPeerSets sets of kPeerWaves
        constexpr unsigned kFold = (unsigned)(kPeerWaves / kInFlight * kPeerSets);
        grid.x = std::max(1u, (grid.x + kFold - 1) / kFold);
        if (vecs <= 4) k_gather_peer<DTYPE, 4><<<grid, kThreads, 0, st>>>(a, group, first);
        else if (vecs <= 8) k_gather_peer<DTYPE, 8><<<grid, kThreads, 0, st>>>(a, group, first);
        else if (vecs <= 16) k_gather_peer<DTYPE, 16><<<grid, kThreads, 0, st>>>(a, group, first);
        else k_gather_peer<DTYPE, 32><<<grid, kThreads, 0, st>>>(a, group, first);
        return cudaGetLastError();
    }
    if (vecs <= 4) k_gather_vec<DTYPE, 4><<<grid, kThreads, 0, st>>>(a, group, first);
    else if (vecs <= 8) k_gather_vec<DTYPE, 8><<<grid, kThreads, 0, st>>>(a, group, first);
    else if (vecs <= 16) k_gather_vec<DTYPE, 16><<<grid, kThreads, 0, st>>>(a, group, first);
    else k_gather_vec<DTYPE, 32><<<grid, kThreads, 0, st>>>(a, group, first);
    return cudaGetLastError();
}

// Staged gather: the rows of a set travel global -> shared memory as bulk asynchronous
// copies (cp.async.bulk, one per row, issued by one warp, completion counted in bytes
// on an mbarrier), and the block's warps convert and store a set that has landed while
// the copies of the next sets are in flight.  The bytes in flight are held by shared
// memory instead of registers: a block is 128 threads and ~5 K registers for up to
// 48 KiB in flight, so the latency-bound sampling kernels of the other chains find
// room on the SM beside it — the register version needs 12 K registers per 16 KiB.
// Source and destination of every copy are 16-byte aligned and the size is a multiple
// of 16 (row_bytes % 16 == 0, aligned payload; the shared rows are packed at row_bytes).
constexpr int kBulkThreads = 128;
constexpr int kBulkRows = 32;     // rows per set: one copy per lane of the issuing warp
constexpr int kBulkStages = 4;    // sets in shared memory (three in flight while one is converted)
constexpr long long kBulkWaitCycles = 2000000000ll;  // about a second of SM clock: then the kernel gives up on a set

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Polls the barrier's phase; false when it has not completed within kBulkWaitCycles.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if ((i & 63u) == 63u) {
            if (clock64() - t0 > kBulkWaitCycles) return false;
            __nanosleep(32);
        }
    }
}

template <int DTYPE>
__global__ void __launch_bounds__(kBulkThreads)
k_gather_bulk(GatherArgs a, const GatherArgs *__restrict__ group, uint64_t first) {
    extern __shared__ __align__(128) uint8_t s_rows[];           // kBulkStages sets of kBulkRows rows
    __shared__ __align__(8) unsigned long long s_bar[kBulkStages];
    __shared__ uint32_t s_ok[kBulkStages];                        // bit r: row r of the set was copied
    if (group) a = group[blockIdx.y];
    if (!a.payload) return;
    const uint64_t n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;
    const uint32_t row_bytes = a.row_bytes;
    const uint32_t set_bytes = (uint32_t)kBulkRows * row_bytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int st = 0; st < kBulkStages; ++st)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&s_bar[st])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const uint64_t pol = l2_evict_first_policy();
    const uint64_t sets = n > first ? (n - first + kBulkRows - 1) / kBulkRows : 0;
    // this block's sets: blockIdx.x, blockIdx.x + gridDim.x, ...
    const uint64_t mine = sets > blockIdx.x ? (sets - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    // warp 0 issues the copies of this block's k-th set into stage k % kBulkStages
    auto issue = [&](uint64_t k) {
        const int st = (int)(k % kBulkStages);
        const uint64_t r = first + (blockIdx.x + k * gridDim.x) * kBulkRows + lane;
        bool ok = false;
        const uint8_t *src = nullptr;
        if (r < n) {
            const uint64_t id = load_id(a.ids, a.ids64, r);
            const uint64_t local = id - a.row_begin;
            if (id >= a.row_begin && local < a.rows) { ok = true; src = a.payload + local * row_bytes; }
            else atomicOr(a.err, kErrBadId);
        }
        const uint32_t okmask = __ballot_sync(0xffffffffu, ok);
        const uint32_t bar = smem_u32(&s_bar[st]);
        if (lane == 0) {  // the one arrival of the phase, with the bytes the copies below will deliver
            s_ok[st] = okmask;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;"
                         :: "r"(bar), "r"((uint32_t)__popc(okmask) * row_bytes) : "memory");
        }
        __syncwarp();
        if (ok) {
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                         :: "r"(smem_u32(s_rows + (size_t)st * set_bytes + (size_t)lane * row_bytes)), "l"(src), "r"(row_bytes),
                            "r"(bar), "l"(pol) : "memory");
        }
    };

    if (warp == 0)
        for (uint64_t k = 0; k < mine && k < (uint64_t)(kBulkStages - 1); ++k) issue(k);
    const uint32_t vecs = row_bytes >> 4;
    const uint32_t out_per_vec = (DTYPE == AG_F32) ? 4u : 8u;
    constexpr int kWarps = kBulkThreads / 32;
    bool failed = false;
    for (uint64_t k = 0; k < mine; ++k) {
        const int st = (int)(k % kBulkStages);
        // the stage of set k + kBulkStages - 1 held set k - 1: every warp finished reading it before the barrier below
        if (warp == 0 && k + kBulkStages - 1 < mine) issue(k + kBulkStages - 1);
        // A set that never arrives is reported and skipped; every thread still reaches the
        // block barrier of every set, and the polls are bounded, so the kernel always ends.
        if (!failed && !mbar_wait(smem_u32(&s_bar[st]), (uint32_t)((k / kBulkStages) & 1))) {
            failed = true;
            atomicOr(a.err, kErrSpinTimeout);
        }
        if (!failed) {
            const uint32_t okmask = s_ok[st];
            const uint64_t r0 = first + (blockIdx.x + k * gridDim.x) * kBulkRows;
            const uint8_t *set = s_rows + (size_t)st * set_bytes;
            for (int rr = warp; rr < kBulkRows; rr += kWarps) {
                const uint64_t r = r0 + rr;
                if (r >= n) break;
                float *dst = a.out + r * a.dim;
                const bool ok = (okmask >> rr) & 1u;
                for (uint32_t v = lane; v < vecs; v += 32) {
                    uint4 val = make_uint4(0, 0, 0, 0);  // a row outside the store decodes to zeros
                    if (ok) val = *(const uint4 *)(set + (size_t)rr * row_bytes + ((size_t)v << 4));
                    store_decoded<DTYPE>(dst + (uint64_t)v * out_per_vec, val);
                }
            }
        }
        __syncthreads();
    }
}

template <int DTYPE>
cudaError_t launch_bulk(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, uint64_t rows_per_batch,
                        uint32_t n_batches, cudaStream_t st, uint64_t first = 0) {
    const size_t smem = (size_t)kBulkStages * kBulkRows * row_bytes;
    // per device, so set on every launch (cheap next to the launch itself)
    const cudaError_t ae = cudaFuncSetAttribute(k_gather_bulk<DTYPE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (ae != cudaSuccess) return ae;
    // a block walks many sets, so that its pipeline fills once per few hundred rows
    static const uint64_t per_block = [] { const char *v = getenv("AG_BULK_SETS"); return v ? (uint64_t)std::max(1, atoi(v)) : 16ull; }();
    const uint64_t sets = std::max<uint64_t>(1, (rows_per_batch + kBulkRows - 1) / kBulkRows);
    const uint64_t cap = std::max<uint64_t>(1, ((uint64_t)kSMs * 32 + n_batches - 1) / n_batches);
    const dim3 grid((unsigned)std::max<uint64_t>(1, std::min<uint64_t>((sets + per_block - 1) / per_block, cap)), n_batches);
    k_gather_bulk<DTYPE><<<grid, kBulkThreads, smem, st>>>(a, group, first);
    return cudaGetLastError();
}

// AG_GATHER_BULK=1: the replicated gather goes through shared memory (A/B measurements).
bool bulk_gather_enabled(uint32_t row_bytes) {
    static const bool on = [] { const char *v = getenv("AG_GATHER_BULK"); return v && v[0] == '1'; }();
    return on && row_bytes >= 64 && (size_t)kBulkStages * kBulkRows * row_bytes <= 200 * 1024;
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
// the link's bandwidth.  So a launch first turns its row ids into keys, sorts
// them (in local memory) together with the output position of each row, and
// gathers in that order.  The f32 rows are still written at their original
// positions in local HBM, where order costs nothing.
//
// key = remote << B | turn << R | row-within-source, the sources being the W shards
// and, when the view holds a copy of the hot rows, that copy as source W (S = W or
// W + 1); 2^R >= the rows of the largest source; `remote` says the source is another
// GPU's memory; `turn` = (source - self - 1) mod S, the source's place in this
// reader's order.
//   * Local rows sort before remote ones, and the two parts are fetched by two
//     launches that can run side by side: the local part streams at HBM speed,
//     the remote part waits on NVLink round trips, and neither holds the other up.
//   * The remote part walks one peer after the other, each in ascending address
//     order, starting with the peer after the reader: ranks that run in step read
//     from different owners.  (Interleaving the peers row by row — every peer at the
//     same offset at the same time — was measured at 4 GPUs and collapses to
//     ~50 GB/s: the mappings of the peers' shards collide in the address translation.)
// The batches of one launch chain name many rows more than once (hub vertices turn
// up in most batches of a chain: three rows in ten of a 64-batch chain on the
// R-MAT benchmark graph are repeats).  Equal keys are neighbours after the sort, so
// such a row is loaded once and written to every batch that asked for it.  (Sorting
// only the upper bits of the key would be enough for the address translation and
// save two of the four radix passes, but it loses the repeats: measured, the extra
// row loads cost three times what the passes do.)
constexpr uint32_t kValRowBits = 23;  // value = batch << 23 | row: rows per batch < 2^23, batches per chain <= 256
constexpr uint32_t kSortedBits = 32;  // key bits the radix sort orders, counted from the top: all of them
constexpr int kPartLocal = 0, kPartRemote = 1, kPartAll = 2;

struct SortedKeys {
    uint32_t addr_bits;   // B
    uint32_t row_bits;    // R
    uint32_t sentinel;    // padding mark: above every key
    int begin_bit, end_bit;
};

__device__ __forceinline__ uint32_t addr_key(const ag_shard_table *t, uint64_t id, uint32_t addr_bits, uint32_t row_bits) {
    const uint32_t S = t->n_sources;  // the shards, and the local copy of the hot rows as one more source
    uint32_t source, local;
    bool hot = false;
    if (t->hot_slot) {
        const uint32_t h = __ldg(t->hot_slot + id);
        if (h != 0xFFFFFFFFu) { source = t->n_shards; local = h; hot = true; }
    }
    if (!hot) {
        if (t->cyclic) { source = (uint32_t)(id % t->n_shards); local = (uint32_t)(id / t->n_shards); }
        else { source = (uint32_t)(id / t->shard_rows); local = (uint32_t)(id - (uint64_t)source * t->shard_rows); }
    }
    uint32_t turn = source + S - t->self - 1;  // the reader's own shard comes last, the peer after it first
    if (turn >= S) turn -= S;
    const uint32_t remote = (!hot && source != t->self) ? 1u : 0u;
    return (remote << addr_bits) | (turn << row_bits) | local;
}

// counts[0] / counts[1] receive the number of keys of local / remote rows (local ones sort to the front).
__global__ void __launch_bounds__(256)
k_make_keys(GatherArgs a, const GatherArgs *__restrict__ group, uint32_t rows_cap, uint32_t addr_bits, uint32_t row_bits,
            uint32_t sentinel, uint32_t *__restrict__ keys, uint32_t *__restrict__ vals, uint32_t *__restrict__ counts) {
    if (group) a = group[blockIdx.y];
    uint64_t n = 0;
    if (a.payload) n = a.n_dev ? min((uint64_t)*a.n_dev, a.n) : a.n;
    if (a.ids_off) a.ids = (const uint32_t *)a.ids + *a.ids_off;
    const uint64_t slot0 = (uint64_t)blockIdx.y * rows_cap;
    uint32_t local_rows = 0, remote_rows = 0;
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < rows_cap; r += gridDim.x * blockDim.x) {
        uint32_t key = sentinel;  // slots past the batch's rows sort to the end
        if (r < n) {
            const uint64_t id = load_id(a.ids, a.ids64, r);
            if (id >= a.row_begin && id - a.row_begin < a.rows) {
                key = addr_key(a.shards, id, addr_bits, row_bits);
                if ((key >> addr_bits) == 0) ++local_rows; else ++remote_rows;
            } else {
                atomicOr(a.err, kErrBadId);
            }
        }
        keys[slot0 + r] = key;
        vals[slot0 + r] = (blockIdx.y << kValRowBits) | r;
    }
    // one atomic per warp and counter
    for (int o = 16; o > 0; o >>= 1) {
        local_rows += __shfl_xor_sync(0xffffffffu, local_rows, o);
        remote_rows += __shfl_xor_sync(0xffffffffu, remote_rows, o);
    }
    if ((threadIdx.x & 31) == 0) {
        if (local_rows) atomicAdd(counts, local_rows);
        if (remote_rows) atomicAdd(counts + 1, remote_rows);
    }
}

// The fetch.  Entry i of the sorted list fetches its row when it starts a run of
// equal keys or sits at a multiple of kRunCap; it then writes the row to every entry
// up to the next fetcher.  Repeats are loaded once per kRunCap entries at most, and
// no lane group is ever left writing a long run on its own.
constexpr int kRunCap = 4;

// address part of a key -> (source, row within source): shifts and one conditional
// subtraction, no division (two divisions per row and lane by the run-time number of
// sources were measured to saturate the special-function pipe).
__device__ __forceinline__ void split_key(uint32_t ak, uint32_t S, uint32_t self, uint32_t row_bits, uint32_t &src,
                                          uint32_t &local) {
    local = ak & ((1u << row_bits) - 1u);
    src = (ak >> row_bits) + self + 1;
    if (src >= S) src -= S;
}

template <int DTYPE, int LPR>
__global__ void __launch_bounds__(kThreads, 4)
k_gather_sorted(GatherArgs one, const GatherArgs *__restrict__ group, uint32_t n_batches,
                const ag_shard_table *__restrict__ t, const uint32_t *__restrict__ keys,
                const uint32_t *__restrict__ vals, uint64_t n_items, uint32_t addr_bits, uint32_t row_bits,
                uint32_t sentinel, uint32_t row_bytes, uint32_t dim, int part, const uint32_t *__restrict__ counts,
                unsigned long long *__restrict__ counters) {
    constexpr int kRowsPerBlock = kThreads / LPR;
    constexpr uint32_t kChunk = (uint32_t)kRowsPerBlock * kInFlight;
    __shared__ float *s_out[256];       // output base of every batch of the chain
    __shared__ const uint8_t *s_base[9];  // where every source's rows start
    if (group) { for (uint32_t b = threadIdx.x; b < n_batches; b += kThreads) s_out[b] = group[b].out; }
    else if (threadIdx.x == 0) s_out[0] = one.out;
    const uint32_t S = t->n_sources, W = t->n_shards, self = t->self;
    if (threadIdx.x < 9) s_base[threadIdx.x] = threadIdx.x < S ? t->base[threadIdx.x] : nullptr;
    __syncthreads();
    const int lane = threadIdx.x % LPR;
    const int sub = threadIdx.x / LPR;
    const uint32_t vecs = row_bytes >> 4;
    const uint32_t out_per_vec = (DTYPE == AG_F32) ? 4u : 8u;
    const uint32_t addr_mask = (1u << addr_bits) - 1u;
    constexpr uint32_t kRowMask = (1u << kValRowBits) - 1u;
    // this launch's part of the list: the local rows, the remote rows, or all of them
    // (32-bit positions: the host keeps a list below 2^31 entries)
    const uint32_t n_all = (uint32_t)n_items;
    const uint32_t n_local = min(counts[0], n_all);
    const uint32_t n_valid = (uint32_t)min((uint64_t)n_local + counts[1], (uint64_t)n_all);
    const uint32_t begin = (part == kPartRemote) ? n_local : 0u;
    const uint32_t end = (part == kPartLocal) ? n_local : n_valid;
    constexpr uint32_t kNoFetch = 0xFFFFFFFFu;  // never an address: the remote bit sits below bit 31
    uint32_t asked = 0, loaded = 0, local_hits = 0;  // counted by lane 0 of each row group
    // Every block takes one contiguous stretch of the list, so the blocks of a launch
    // work on gridDim.x distant address ranges at once.  Walking the list chunk by
    // chunk across the grid keeps all in-flight loads on the same few pages, and each
    // first touch of a 2 MB page of peer memory then stalls the whole launch for a
    // page walk: ~0.5 us per page, 10 ms for one pass over 38 GB of peer shards,
    // whatever the number of rows (measured on 4 GPUs).
    const uint32_t n_chunks = end > begin ? (end - begin + kChunk - 1) / kChunk : 0u;
    const uint32_t per_block = (n_chunks + gridDim.x - 1) / gridDim.x;
    const uint32_t first_chunk = blockIdx.x * per_block;
    const uint32_t last_chunk = min(first_chunk + per_block, n_chunks);
    for (uint32_t chunk = first_chunk; chunk < last_chunk; ++chunk) {
        const uint32_t chunk0 = begin + chunk * (uint32_t)kChunk;
        const uint32_t base = chunk0 + sub;
        uint32_t ak[kInFlight];   // address part of a fetching entry's key, or kNoFetch
        uint32_t val[kInFlight];
#pragma unroll
        for (int u = 0; u < kInFlight; ++u) {
            const uint32_t i = base + u * kRowsPerBlock;
            ak[u] = kNoFetch; val[u] = 0;
            if (i < end) {
                const uint32_t key = keys[i];
                val[u] = vals[i];
                const uint32_t prev = i > begin ? keys[i - 1] : sentinel;
                const bool fetch = prev != key || (i % kRunCap) == 0;
                if (fetch) ak[u] = key & addr_mask;
                if (lane == 0) { ++asked; loaded += fetch; }
            }
        }
        for (uint32_t v0 = 0; v0 < vecs; v0 += LPR) {
            const uint32_t v = v0 + lane;
            uint4 row[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                row[u] = make_uint4(0, 0, 0, 0);
                if (ak[u] != kNoFetch && v < vecs) {
                    uint32_t src, local;
                    split_key(ak[u], S, self, row_bits, src, local);
                    if (lane == 0 && v0 == 0) local_hits += (S > W && src == W);
                    row[u] = ld_peer_v4(s_base[src] + (uint64_t)local * row_bytes + (v << 4));
                }
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (ak[u] == kNoFetch || v >= vecs) continue;
                store_decoded<DTYPE>(s_out[val[u] >> kValRowBits] + (uint64_t)(val[u] & kRowMask) * dim + v * out_per_vec, row[u]);
                // the rest of the run, up to the next fetcher
                const uint32_t i = base + u * kRowsPerBlock;
                for (uint32_t j = i + 1; j < end && (j % kRunCap) != 0 && keys[j] == keys[i]; ++j) {
                    const uint32_t pv = vals[j];
                    store_decoded<DTYPE>(s_out[pv >> kValRowBits] + (uint64_t)(pv & kRowMask) * dim + v * out_per_vec, row[u]);
                }
            }
        }
    }
    if (lane == 0 && asked) {
        atomicAdd(counters, (unsigned long long)asked); atomicAdd(counters + 1, (unsigned long long)loaded);
        if (local_hits) atomicAdd(counters + 2, (unsigned long long)local_hits);
    }
}

template <int DTYPE>
cudaError_t launch_sorted(const GatherArgs &one, const GatherArgs *group, uint32_t n_batches, const ag_shard_table *t,
                          const uint32_t *keys, const uint32_t *vals, uint64_t n_items, const SortedKeys &sk, uint32_t row_bytes,
                          uint32_t dim, int part, const uint32_t *counts, unsigned long long *counters, cudaStream_t st) {
    // a few chunks per block: the block's tables of output and source bases are set up once
    const int blocks = std::max(1, std::min(gather_grid_blocks(n_items, row_bytes), kSMs * 16));
    const uint32_t vecs = row_bytes >> 4;
#define AG_LAUNCH_SORTED(L) k_gather_sorted<DTYPE, L><<<blocks, kThreads, 0, st>>>(one, group, n_batches, t, keys, vals, n_items, \
                                sk.addr_bits, sk.row_bits, sk.sentinel, row_bytes, dim, part, counts, counters)
    if (vecs <= 4) AG_LAUNCH_SORTED(4);
    else if (vecs <= 8) AG_LAUNCH_SORTED(8);
    else if (vecs <= 16) AG_LAUNCH_SORTED(16);
    else AG_LAUNCH_SORTED(32);
#undef AG_LAUNCH_SORTED
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
            case AG_I8: return launch_i8(a, nullptr, a.row_bytes, grid, st);
            case AG_F32: return launch_vec<AG_F32>(a, nullptr, a.row_bytes, grid, a.shards != nullptr, st);
            case AG_F16: return launch_vec<AG_F16>(a, nullptr, a.row_bytes, grid, a.shards != nullptr, st);
            default: return launch_vec<AG_BF16>(a, nullptr, a.row_bytes, grid, a.shards != nullptr, st);
        }
    }
    const uint64_t total = a.n * a.dim;
    uint64_t blocks = (total + kThreads - 1) / kThreads;
    if (blocks > (uint64_t)kSMs * 8) blocks = (uint64_t)kSMs * 8;
    switch (dtype) {
        case AG_I8: k_gather_elem<AG_I8><<<(int)blocks, kThreads, 0, st>>>(a, nullptr); break;
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
        // AG_GATHER_BLOCKS_PER_SM: grid cap of a chain's gather in blocks per SM (A/B measurements)
        static const int per_sm = [] { const char *v = getenv("AG_GATHER_BLOCKS_PER_SM"); return v ? std::max(1, atoi(v)) : 64; }();
        const int cap = std::max(1, (kSMs * per_sm + (int)n_batches - 1) / (int)n_batches);
        per = std::min(per, cap);
        const dim3 grid(per, n_batches);
        if (!sharded && dtype != AG_I8 && bulk_gather_enabled(row_bytes)) {
            switch (dtype) {
                case AG_F32: return launch_bulk<AG_F32>(none, group_dev, row_bytes, n_bound, n_batches, st);
                case AG_F16: return launch_bulk<AG_F16>(none, group_dev, row_bytes, n_bound, n_batches, st);
                default: return launch_bulk<AG_BF16>(none, group_dev, row_bytes, n_bound, n_batches, st);
            }
        }
        switch (dtype) {
            case AG_I8: return launch_i8(none, group_dev, row_bytes, grid, st);
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
        case AG_I8: k_gather_elem<AG_I8><<<grid, kThreads, 0, st>>>(none, group_dev); break;
        case AG_F32: k_gather_elem<AG_F32><<<grid, kThreads, 0, st>>>(none, group_dev); break;
        case AG_F16: k_gather_elem<AG_F16><<<grid, kThreads, 0, st>>>(none, group_dev); break;
        default: k_gather_elem<AG_BF16><<<grid, kThreads, 0, st>>>(none, group_dev); break;
    }
    return cudaGetLastError();
}

// ------------------------------------------------ sorted gather, host side --
void SortScratch::release() {
    cudaFree(keys[0]); cudaFree(keys[1]); cudaFree(vals[0]); cudaFree(vals[1]); cudaFree(temp); cudaFree(counts);
    keys[0] = keys[1] = vals[0] = vals[1] = nullptr; temp = nullptr; counts = nullptr;
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
    if (e == cudaSuccess) e = cudaMalloc(&counts, 16);
    if (e != cudaSuccess) { release(); return e; }
    cap = want; temp_bytes = tb;
    return cudaSuccess;
}

// Bits of the row-within-source field: 2^R >= the rows of the largest source.
uint32_t sorted_row_bits(const ag_features *f) {
    return std::max<uint32_t>(1, bit_width_u64(std::max<uint64_t>(std::max<uint64_t>(f->shard_rows, f->hot_n), 2) - 1));
}
// One past the largest turn << R | row of the view.
uint64_t sorted_key_bound(const ag_features *f) {
    const uint64_t sources = f->n_shards + (f->hot_n ? 1 : 0);
    return sources << sorted_row_bits(f);
}

namespace {
SortedKeys sorted_keys_of(const ag_features *f) {
    SortedKeys k{};
    k.row_bits = sorted_row_bits(f);
    k.addr_bits = bit_width_u64(sorted_key_bound(f));          // B: every address part is below 2^B
    k.sentinel = (uint32_t)((1ull << (k.addr_bits + 2)) - 1);   // above remote << B | anything
    k.end_bit = (int)k.addr_bits + 2;
    k.begin_bit = std::max(0, k.end_bit - (int)kSortedBits);
    return k;
}
}  // namespace

bool sorted_gather_applies(const ag_features *f, uint32_t row_bytes, bool aligned) {
    // AG_GATHER_SORTED=0 / 1 overrides every view's setting (A/B measurements)
    static const int forced = [] {
        const char *v = getenv("AG_GATHER_SORTED");
        return !v ? -1 : (v[0] == '0' ? 0 : 1);
    }();
    if (!f || !f->shards || f->n_shards < 2 || !aligned || row_bytes % 16 != 0) return false;
    if (bit_width_u64(sorted_key_bound(f)) > 30) return false;  // 32-bit keys: address part, the remote bit, the padding mark above
    if (forced >= 0) return forced == 1;
    if (f->gather_order == AG_GATHER_ORDERED) return true;
    if (f->gather_order == AG_GATHER_DIRECT) return false;
    // Peers mapped with large pages serve random rows at link speed: sorting only adds
    // work (measured at 8 GPUs, 100M x 256 bf16: 17.4 G edges/s direct, 13.8 G ordered).
    // A legacy IPC mapping is an order of magnitude slower at random than in address order.
    return f->legacy_peer;
}

// The address-ordered gather in two steps, so that a caller can put them on different
// streams (small latency-bound kernels first, the fetch behind an event).
// Step 1: keys of rows [0, min(n_b, rows_cap)) of every batch, sorted with their output
// positions.  Step 2: fetch in that order — the local part on st_local, the remote part
// on st_remote (the same stream: one after the other) — then rows [rows_cap, n_b), only
// present when a batch outgrew the caller's estimate, with the unsorted kernel.
// `one` / `group_dev` as in launch_gather / launch_gather_group.
cudaError_t launch_sort_keys(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                             const ag_features *f, SortScratch &sc, cudaStream_t st) {
    if (n_batches == 0 || rows_cap == 0) return cudaSuccess;
    rows_cap = std::min<uint64_t>(rows_cap, (1ull << kValRowBits) - 1);
    const uint64_t n_items = (uint64_t)n_batches * rows_cap;
    cudaError_t e = sc.ensure(n_items);
    if (e != cudaSuccess) return e;
    const SortedKeys sk = sorted_keys_of(f);
    if ((e = cudaMemsetAsync(sc.counts, 0, 16, st)) != cudaSuccess) return e;
    const uint32_t kb = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((rows_cap + 255) / 256, std::max<uint64_t>(1, (uint64_t)kSMs * 8 / n_batches)));
    k_make_keys<<<dim3(kb, n_batches), 256, 0, st>>>(one, group_dev, (uint32_t)rows_cap, sk.addr_bits, sk.row_bits, sk.sentinel, sc.keys[0],
                                                    sc.vals[0], sc.counts);
    if ((e = cudaGetLastError()) != cudaSuccess) return e;
    size_t tb = sc.temp_bytes;
    return cub::DeviceRadixSort::SortPairs(sc.temp, tb, (const uint32_t *)sc.keys[0], sc.keys[1], (const uint32_t *)sc.vals[0],
                                           sc.vals[1], n_items, sk.begin_bit, sk.end_bit, st);
}

cudaError_t launch_sorted_fetch(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                                uint32_t row_bytes, uint32_t dim, int dtype, const ag_features *f, SortScratch &sc,
                                cudaStream_t st_local, cudaStream_t st_remote) {
    if (n_batches == 0 || rows_cap == 0) return cudaSuccess;
    rows_cap = std::min<uint64_t>(rows_cap, (1ull << kValRowBits) - 1);
    const uint64_t n_items = (uint64_t)n_batches * rows_cap;
    const SortedKeys sk = sorted_keys_of(f);
    unsigned long long *counters = (unsigned long long *)((uint8_t *)f->err + 8);
    auto fetch = [&](int part, cudaStream_t st) {
        switch (dtype) {
            case AG_F32: return launch_sorted<AG_F32>(one, group_dev, n_batches, f->shards, sc.keys[1], sc.vals[1], n_items, sk, row_bytes, dim, part, sc.counts, counters, st);
            case AG_F16: return launch_sorted<AG_F16>(one, group_dev, n_batches, f->shards, sc.keys[1], sc.vals[1], n_items, sk, row_bytes, dim, part, sc.counts, counters, st);
            default: return launch_sorted<AG_BF16>(one, group_dev, n_batches, f->shards, sc.keys[1], sc.vals[1], n_items, sk, row_bytes, dim, part, sc.counts, counters, st);
        }
    };
    cudaError_t e = fetch(kPartRemote, st_remote);
    if (e == cudaSuccess) e = fetch(kPartLocal, st_local);
    if (e != cudaSuccess) return e;
    // Rows past the estimate (rare): a few blocks per batch, which stride; most exit at once.
    const dim3 grid(4, n_batches);
    switch (dtype) {
        case AG_F32: return launch_vec<AG_F32>(one, group_dev, row_bytes, grid, true, st_local, rows_cap);
        case AG_F16: return launch_vec<AG_F16>(one, group_dev, row_bytes, grid, true, st_local, rows_cap);
        default: return launch_vec<AG_BF16>(one, group_dev, row_bytes, grid, true, st_local, rows_cap);
    }
}

cudaError_t launch_gather_sorted(const GatherArgs &one, const GatherArgs *group_dev, uint32_t n_batches, uint64_t rows_cap,
                                 uint32_t row_bytes, uint32_t dim, int dtype, const ag_features *f, SortScratch &sc,
                                 cudaStream_t st) {
    const cudaError_t e = launch_sort_keys(one, group_dev, n_batches, rows_cap, f, sc, st);
    if (e != cudaSuccess) return e;
    return launch_sorted_fetch(one, group_dev, n_batches, rows_cap, row_bytes, dim, dtype, f, sc, st, st);
}

cudaError_t launch_encode_i8(const float *src, uint64_t rows, uint64_t dim, int8_t *codes, float *scales, uint32_t *bad_dev,
                             cudaStream_t st) {
    const uint64_t blocks = rows * ((dim + kQuantBlock - 1) / kQuantBlock);
    if (blocks == 0) return cudaSuccess;
    const uint64_t grid = std::max<uint64_t>(1, std::min<uint64_t>((blocks * 32 + 255) / 256, (uint64_t)kSMs * 16));
    k_encode_i8<<<(int)grid, 256, 0, st>>>(src, rows, dim, codes, scales, bad_dev);
    return cudaGetLastError();
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

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
k_gather_vec(GatherArgs a, const GatherArgs *__restrict__ group) {
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

    for (uint64_t base = (uint64_t)blockIdx.x * kChunk + sub; base < n; base += (uint64_t)gridDim.x * kChunk) {
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
cudaError_t launch_vec_s(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, dim3 grid, cudaStream_t st) {
    const uint32_t vecs = row_bytes >> 4;
    if (vecs <= 4) k_gather_vec<DTYPE, 4, SHARDED><<<grid, kThreads, 0, st>>>(a, group);
    else if (vecs <= 8) k_gather_vec<DTYPE, 8, SHARDED><<<grid, kThreads, 0, st>>>(a, group);
    else if (vecs <= 16) k_gather_vec<DTYPE, 16, SHARDED><<<grid, kThreads, 0, st>>>(a, group);
    else k_gather_vec<DTYPE, 32, SHARDED><<<grid, kThreads, 0, st>>>(a, group);
    return cudaGetLastError();
}

template <int DTYPE>
cudaError_t launch_vec(const GatherArgs &a, const GatherArgs *group, uint32_t row_bytes, dim3 grid, bool sharded,
                       cudaStream_t st) {
    return sharded ? launch_vec_s<DTYPE, true>(a, group, row_bytes, grid, st)
                   : launch_vec_s<DTYPE, false>(a, group, row_bytes, grid, st);
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

cudaError_t launch_encode(const float *src, void *dst, uint64_t count, int dtype, cudaStream_t st) {
    if (count == 0) return cudaSuccess;
    if (dtype == AG_F32) return cudaMemcpyAsync(dst, src, count * 4, cudaMemcpyDeviceToDevice, st);
    uint64_t blocks = (count + 255) / 256;
    if (blocks > (uint64_t)kSMs * 8) blocks = (uint64_t)kSMs * 8;
    k_encode<<<(int)blocks, 256, 0, st>>>(src, (uint16_t *)dst, count, dtype);
    return cudaGetLastError();
}

}  // namespace ag

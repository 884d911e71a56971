// Seeded synthetic inputs generated directly in HBM: R-MAT graphs, bipartite
// relations and N(0,1)-like feature tables.  They stand in for datasets: the
// reference's own benchmarks also run on seeded synthetic graphs
// (crates/aethergraph-core/benches/sampling_scale.rs:29-49).
//
// Everything is a pure function of (seed, index) built from the SplitMix64
// finalizer and integer arithmetic, so any other implementation of the same
// recipe (the CPU twin used by the CPU baseline) produces identical bits:
//   mix(x)        = SplitMix64 finalizer of x + 0x9E3779B97F4A7C15
//   edge i        : base = mix(seed ^ mix(i)); attempt t: st = mix(base + t * G1);
//                   word w = mix(st + (w + 1) * G2); level l takes 16 bits
//                   u = (word[l / 4] >> 16 * (l % 4)) & 0xFFFF and picks the
//                   quadrant u < A -> (0,0), < AB -> (0,1), < ABC -> (1,0), else (1,1)
//                   (first bit to the source id, second to the destination);
//                   an endpoint past the vertex count is redrawn with t + 1.
//   rows          : sorted by (source, destination); duplicates and self-loops kept.
//   feature (v,j) : e = v * dim + j; r0 = mix(seed ^ mix(e)); r1 = mix(r0 + G1);
//                   s = sum of the eight 16-bit fields of r0, r1 (Irwin-Hall, 8 terms);
//                   value = float(s - 262140) * kScale, then encoded to the store dtype.
//   weight at CSR position p: exp(sigma * z(seed, p)) with z as for features.
#include <cub/device/device_radix_sort.cuh>

#include "common.cuh"
#include "internal.h"

namespace ag {
namespace {

constexpr uint64_t G1 = 0x9E3779B97F4A7C15ull, G2 = 0xD6E8FEB86659FD93ull;
// 1 / sqrt(8 * (65536^2 - 1) / 12): unit variance for the 8-term sum of 16-bit uniforms.
constexpr float kScale = 1.8688173e-05f;

__host__ __device__ __forceinline__ uint64_t mix(uint64_t x) {
    uint64_t z = x + G1;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ float unit_normal(uint64_t seed, uint64_t e) {
    const uint64_t r0 = mix(seed ^ mix(e)), r1 = mix(r0 + G1);
    uint32_t s = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) s += (uint32_t)((r0 >> (16 * k)) & 0xFFFF) + (uint32_t)((r1 >> (16 * k)) & 0xFFFF);
    return (float)((int)s - 262140) * kScale;
}

struct RmatParams {
    uint64_t num_src, num_dst, num_edges, seed;
    uint32_t bits_src, bits_dst, a16, ab16, abc16;
};

__device__ __forceinline__ void rmat_edge(const RmatParams &p, uint64_t i, uint32_t &s, uint32_t &d) {
    const uint64_t base = mix(p.seed ^ mix(i));
    const uint32_t levels = max(p.bits_src, p.bits_dst);
    for (uint32_t t = 0;; ++t) {
        const uint64_t st = mix(base + (uint64_t)t * G1);
        uint64_t src = 0, dst = 0, word = 0;
        for (uint32_t l = 0; l < levels; ++l) {
            if ((l & 3u) == 0) word = mix(st + (uint64_t)(l / 4 + 1) * G2);
            const uint32_t u = (uint32_t)(word >> (16 * (l & 3u))) & 0xFFFFu;
            const uint32_t sb = u >= p.ab16 ? 1u : 0u;
            const uint32_t db = ((u >= p.a16 && u < p.ab16) || u >= p.abc16) ? 1u : 0u;
            // a side with fewer levels than the other ignores the leading ones
            if (l + p.bits_src >= levels) src = (src << 1) | sb;
            if (l + p.bits_dst >= levels) dst = (dst << 1) | db;
        }
        if (src < p.num_src && dst < p.num_dst) { s = (uint32_t)src; d = (uint32_t)dst; return; }
        if (t == 63) { s = (uint32_t)(src % p.num_src); d = (uint32_t)(dst % p.num_dst); return; }
    }
}

__global__ void k_rmat_keys(RmatParams p, uint64_t *keys) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.num_edges;
         i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t s, d;
        rmat_edge(p, i, s, d);
        keys[i] = ((uint64_t)s << 32) | d;
    }
}

// Graphs whose edge keys (16 bytes per edge while they are sorted) do not fit the
// free device memory are built in partitions of the source id range: a first pass
// counts the edges per bin of source ids, bins are grouped into contiguous ranges
// that fit, and every range is generated (all edges are drawn again, the ones
// whose source falls in the range are kept), sorted and written on its own.  The
// result is the same CSR — rows are sorted by (source, destination) either way.
constexpr int kHistBits = 12;

__global__ void k_rmat_hist(RmatParams p, uint32_t shift, unsigned long long *hist) {
    __shared__ uint32_t s_hist[1 << kHistBits];
    for (int i = threadIdx.x; i < (1 << kHistBits); i += blockDim.x) s_hist[i] = 0;
    __syncthreads();
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < p.num_edges;
         i += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t s, d;
        rmat_edge(p, i, s, d);
        atomicAdd(&s_hist[s >> shift], 1u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (1 << kHistBits); i += blockDim.x)
        if (s_hist[i]) atomicAdd(&hist[i], (unsigned long long)s_hist[i]);
}

// Keeps the edges whose source lies in [row_lo, row_hi); order does not matter (they are sorted next).
__global__ void k_rmat_keys_range(RmatParams p, uint64_t row_lo, uint64_t row_hi, uint64_t *keys,
                                  unsigned long long *count, uint64_t cap) {
    for (uint64_t i0 = (uint64_t)blockIdx.x * blockDim.x; i0 < p.num_edges; i0 += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t i = i0 + threadIdx.x;
        uint32_t s = 0, d = 0;
        bool keep = false;
        if (i < p.num_edges) {
            rmat_edge(p, i, s, d);
            keep = s >= row_lo && s < row_hi;
        }
        const uint32_t m = __ballot_sync(0xffffffffu, keep);
        if (!m) continue;
        const int lane = threadIdx.x & 31, leader = __ffs(m) - 1;
        unsigned long long base = 0;
        if (lane == leader) base = atomicAdd(count, (unsigned long long)__popc(m));
        base = __shfl_sync(0xffffffffu, base, leader);
        const uint64_t at = base + __popc(m & ((1u << lane) - 1u));
        if (keep && at < cap) keys[at] = ((uint64_t)s << 32) | d;
    }
}

// One partition's sorted keys -> its slice of dst and the offsets of rows [row_lo, row_hi).
__global__ void k_keys_to_csr_part(const uint64_t *keys, uint64_t e, uint64_t base, uint64_t row_lo, uint64_t row_hi,
                                   uint64_t *offsets, uint32_t *dst) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += stride) {
        const uint64_t k = keys[i];
        dst[base + i] = (uint32_t)k;
        const uint64_t s = k >> 32;
        const uint64_t prev = i ? (keys[i - 1] >> 32) + 1 : row_lo;
        for (uint64_t v = prev; v <= s; ++v) offsets[v] = base + i;
        if (i == e - 1) for (uint64_t v = s + 1; v < row_hi; ++v) offsets[v] = base + e;
    }
    if (e == 0)
        for (uint64_t v = row_lo + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; v < row_hi; v += stride) offsets[v] = base;
}

// From keys sorted by (src, dst): dst array and CSR offsets.
__global__ void k_keys_to_csr(const uint64_t *keys, uint64_t e, uint64_t n, uint64_t *offsets, uint32_t *dst) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += stride) {
        const uint64_t k = keys[i];
        dst[i] = (uint32_t)k;
        const uint64_t s = k >> 32;
        const uint64_t prev = i ? (keys[i - 1] >> 32) + 1 : 0;  // first row that starts at or before i
        for (uint64_t v = prev; v <= s; ++v) offsets[v] = i;
        if (i == e - 1) for (uint64_t v = s + 1; v <= n; ++v) offsets[v] = e;
    }
    if (e == 0)
        for (uint64_t v = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; v <= n; v += stride) offsets[v] = 0;
}

__global__ void k_weights(float *w, uint64_t e, uint64_t seed, float sigma) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += (uint64_t)gridDim.x * blockDim.x)
        w[i] = expf(sigma * unit_normal(seed, i));
}

// One source -> exactly `k` destinations: dst = mix(seed ^ mix(v * k + j)) % num_dst, row-sorted not required.
__global__ void k_fixed_degree(uint64_t num_src, uint64_t num_dst, uint32_t k, uint64_t seed, uint64_t *offsets,
                               uint32_t *dst) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t v = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; v <= num_src; v += stride) {
        offsets[v] = v * k;
        if (v < num_src)
            for (uint32_t j = 0; j < k; ++j) dst[v * k + j] = (uint32_t)(mix(seed ^ mix(v * k + j)) % num_dst);
    }
}

__device__ __forceinline__ uint16_t enc_bf16(float v) {
    const uint32_t bits = __float_as_uint(v);
    return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);  // values are finite
}

// Held row i is row row_begin + i * row_stride of the whole table; a value depends
// only on (seed, row, column), so any shard of the table has the whole table's bits.
__global__ void k_features(uint8_t *payload, uint64_t row_begin, uint64_t row_stride, uint64_t rows, uint64_t dim,
                           int dtype, uint64_t seed) {
    const uint64_t total = rows * dim;
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < total;
         g += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t index = row_begin * dim + g;
        if (row_stride != 1) {
            const uint64_t i = g / dim;
            index = (row_begin + i * row_stride) * dim + (g - i * dim);
        }
        const float f = unit_normal(seed, index);
        if (dtype == AG_F32) ((float *)payload)[g] = f;
        else if (dtype == AG_BF16) ((uint16_t *)payload)[g] = enc_bf16(f);
        else ((uint16_t *)payload)[g] = __half_as_ushort(__float2half_rn(f));
    }
}

uint32_t bits_for(uint64_t n) {
    uint32_t b = 0;
    while ((1ull << b) < n) ++b;
    return b;
}

int grid_for(uint64_t n) {
    const uint64_t b = (n + 255) / 256;
    return (int)std::max<uint64_t>(1, std::min<uint64_t>(b, (uint64_t)kSMs * 16));
}

int32_t build_relation_partitioned(const RmatParams &p, float weight_sigma, uint64_t budget_edges,
                                   uint64_t **offsets_out, uint32_t **dst_out, float **w_out);

int32_t build_relation(uint64_t num_src, uint64_t num_dst, uint64_t num_edges, const float abc[3], uint64_t seed,
                       float weight_sigma, int device, uint64_t **offsets_out, uint32_t **dst_out, float **w_out) {
    if (num_src == 0 || num_dst == 0 || num_src > 0xFFFFFFFFull || num_dst > 0xFFFFFFFFull)
        return fail(AG_ERR_VALUE, "vertex counts must be in [1, 2^32)");
    RmatParams p{};
    p.num_src = num_src; p.num_dst = num_dst; p.num_edges = num_edges; p.seed = seed;
    p.bits_src = bits_for(num_src); p.bits_dst = bits_for(num_dst);
    p.a16 = (uint32_t)(abc[0] * 65536.0f);
    p.ab16 = (uint32_t)((abc[0] + abc[1]) * 65536.0f);
    p.abc16 = (uint32_t)((abc[0] + abc[1] + abc[2]) * 65536.0f);
    {
        // All keys at once need 16 bytes per edge (two sort buffers) beside the result;
        // otherwise build the rows a range of sources at a time.
        size_t free_b = 0, total_b = 0;
        if (cudaMemGetInfo(&free_b, &total_b) == cudaSuccess) {
            const uint64_t result = (num_src + 1) * 8 + num_edges * (weight_sigma > 0.f ? 8 : 4);
            const uint64_t spare = (uint64_t)(0.92 * (double)free_b);
            const char *force = getenv("AG_SYNTH_PARTITION_EDGES");  // tests: force the partitioned build
            if (force || num_edges * 16 + num_edges * 4 + (num_src + 1) * 8 + (64ull << 20) > spare) {
                if (spare < result + (1ull << 30)) return fail(AG_ERR_CUDA, "graph of %llu edges does not fit the free device memory",
                                                                (unsigned long long)num_edges);
                uint64_t budget = (spare - result - (256ull << 20)) / 17;  // two key buffers + sort scratch
                if (force) budget = std::max<uint64_t>(1, strtoull(force, nullptr, 10));
                return build_relation_partitioned(p, weight_sigma, budget, offsets_out, dst_out, w_out);
            }
        }
    }
    uint64_t *keys_a = nullptr, *keys_b = nullptr, *offsets = nullptr;
    uint32_t *dst = nullptr;
    float *w = nullptr;
    void *temp = nullptr;
    int32_t st = AG_OK;
    auto cuda_ok = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == AG_OK) st = fail(AG_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
        return e == cudaSuccess;
    };
    do {
        const uint64_t kb = std::max<uint64_t>(num_edges, 1) * 8;
        if (!cuda_ok(cudaMalloc(&keys_a, kb), "cudaMalloc(keys)")) break;
        if (!cuda_ok(cudaMalloc(&keys_b, kb), "cudaMalloc(keys)")) break;
        k_rmat_keys<<<grid_for(num_edges), 256>>>(p, keys_a);
        if (!cuda_ok(cudaGetLastError(), "k_rmat_keys")) break;
        cub::DoubleBuffer<uint64_t> buf(keys_a, keys_b);
        size_t temp_bytes = 0;
        const int end_bit = 32 + (int)p.bits_src;
        if (!cuda_ok(cub::DeviceRadixSort::SortKeys(nullptr, temp_bytes, buf, (uint64_t)num_edges, 0, end_bit), "sort sizing")) break;
        if (!cuda_ok(cudaMalloc(&temp, std::max<size_t>(temp_bytes, 16)), "cudaMalloc(sort temp)")) break;
        if (!cuda_ok(cub::DeviceRadixSort::SortKeys(temp, temp_bytes, buf, (uint64_t)num_edges, 0, end_bit), "radix sort")) break;
        if (!cuda_ok(cudaDeviceSynchronize(), "radix sort")) break;
        cudaFree(temp); temp = nullptr;
        // keep only the sorted buffer
        uint64_t *sorted = buf.Current();
        if (sorted == keys_a) { cudaFree(keys_b); keys_b = nullptr; } else { cudaFree(keys_a); keys_a = nullptr; }
        if (!cuda_ok(cudaMalloc(&offsets, (num_src + 1) * 8), "cudaMalloc(offsets)")) break;
        if (!cuda_ok(cudaMalloc(&dst, std::max<uint64_t>(num_edges, 1) * 4), "cudaMalloc(dst)")) break;
        k_keys_to_csr<<<grid_for(std::max<uint64_t>(num_edges, num_src + 1)), 256>>>(sorted, num_edges, num_src, offsets, dst);
        if (!cuda_ok(cudaGetLastError(), "k_keys_to_csr")) break;
        if (weight_sigma > 0.f) {
            if (!cuda_ok(cudaMalloc(&w, std::max<uint64_t>(num_edges, 1) * 4), "cudaMalloc(weights)")) break;
            k_weights<<<grid_for(num_edges), 256>>>(w, num_edges, mix(seed ^ 0x77656967687473ull), weight_sigma);
            if (!cuda_ok(cudaGetLastError(), "k_weights")) break;
        }
        cuda_ok(cudaDeviceSynchronize(), "graph generation");
    } while (0);
    cudaFree(keys_a); cudaFree(keys_b); cudaFree(temp);
    if (st != AG_OK) { cudaFree(offsets); cudaFree(dst); cudaFree(w); return st; }
    *offsets_out = offsets; *dst_out = dst; *w_out = w;
    return AG_OK;
}

int32_t build_relation_partitioned(const RmatParams &p, float weight_sigma, uint64_t budget_edges,
                                   uint64_t **offsets_out, uint32_t **dst_out, float **w_out) {
    const uint64_t num_src = p.num_src, num_edges = p.num_edges;
    const uint32_t hist_bits = std::min<uint32_t>(kHistBits, p.bits_src);
    const uint32_t shift = p.bits_src - hist_bits;
    const uint32_t bins = 1u << hist_bits;
    uint64_t *keys_a = nullptr, *keys_b = nullptr, *offsets = nullptr;
    unsigned long long *hist_dev = nullptr, *count_dev = nullptr;
    uint32_t *dst = nullptr;
    float *w = nullptr;
    void *temp = nullptr;
    int32_t st = AG_OK;
    auto cuda_ok = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == AG_OK) st = fail(AG_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
        return e == cudaSuccess;
    };
    do {
        if (!cuda_ok(cudaMalloc(&offsets, (num_src + 1) * 8), "cudaMalloc(offsets)")) break;
        if (!cuda_ok(cudaMalloc(&dst, std::max<uint64_t>(num_edges, 1) * 4), "cudaMalloc(dst)")) break;
        if (!cuda_ok(cudaMalloc(&hist_dev, (bins + 1) * 8), "cudaMalloc(histogram)")) break;
        if (!cuda_ok(cudaMemset(hist_dev, 0, (bins + 1) * 8), "cudaMemset")) break;
        count_dev = hist_dev + bins;
        k_rmat_hist<<<grid_for(num_edges), 256>>>(p, shift, hist_dev);
        std::vector<unsigned long long> hist(bins);
        if (!cuda_ok(cudaMemcpy(hist.data(), hist_dev, bins * 8, cudaMemcpyDeviceToHost), "edge histogram")) break;
        // contiguous groups of bins with at most budget_edges edges each (a single bin may exceed it)
        struct Part { uint32_t lo, hi; uint64_t edges; };
        std::vector<Part> parts;
        uint64_t biggest = 0;
        for (uint32_t b = 0; b < bins;) {
            Part q{b, b, 0};
            while (q.hi < bins && (q.hi == q.lo || q.edges + hist[q.hi] <= budget_edges)) q.edges += hist[q.hi++];
            parts.push_back(q);
            biggest = std::max(biggest, q.edges);
            b = q.hi;
        }
        const uint64_t kb = std::max<uint64_t>(biggest, 1) * 8;
        if (!cuda_ok(cudaMalloc(&keys_a, kb), "cudaMalloc(keys)")) break;
        if (!cuda_ok(cudaMalloc(&keys_b, kb), "cudaMalloc(keys)")) break;
        size_t temp_bytes = 0;
        const int end_bit = 32 + (int)p.bits_src;
        {
            cub::DoubleBuffer<uint64_t> probe(keys_a, keys_b);
            if (!cuda_ok(cub::DeviceRadixSort::SortKeys(nullptr, temp_bytes, probe, biggest, 0, end_bit), "sort sizing")) break;
        }
        if (!cuda_ok(cudaMalloc(&temp, std::max<size_t>(temp_bytes, 16)), "cudaMalloc(sort temp)")) break;
        uint64_t base = 0;
        for (const Part &q : parts) {
            const uint64_t row_lo = std::min<uint64_t>((uint64_t)q.lo << shift, num_src);
            const uint64_t row_hi = std::min<uint64_t>((uint64_t)q.hi << shift, num_src);
            if (!cuda_ok(cudaMemset(count_dev, 0, 8), "cudaMemset")) break;
            if (q.edges) k_rmat_keys_range<<<grid_for(num_edges), 256>>>(p, row_lo, row_hi, keys_a, count_dev, biggest);
            unsigned long long got = 0;
            if (!cuda_ok(cudaMemcpy(&got, count_dev, 8, cudaMemcpyDeviceToHost), "k_rmat_keys_range")) break;
            if (got != q.edges) { st = fail(AG_ERR_CUDA, "partitioned graph build: a range produced %llu edges, its bins hold %llu", got, (unsigned long long)q.edges); break; }
            cub::DoubleBuffer<uint64_t> buf(keys_a, keys_b);
            if (q.edges && !cuda_ok(cub::DeviceRadixSort::SortKeys(temp, temp_bytes, buf, (uint64_t)q.edges, 0, end_bit), "radix sort")) break;
            k_keys_to_csr_part<<<grid_for(std::max<uint64_t>(q.edges, row_hi - row_lo + 1)), 256>>>(buf.Current(), q.edges, base, row_lo,
                                                                                                   row_hi, offsets, dst);
            if (!cuda_ok(cudaDeviceSynchronize(), "k_keys_to_csr_part")) break;
            base += q.edges;
        }
        if (st != AG_OK) break;
        if (base != num_edges) { st = fail(AG_ERR_CUDA, "partitioned graph build lost edges (%llu of %llu)", (unsigned long long)base, (unsigned long long)num_edges); break; }
        if (!cuda_ok(cudaMemcpy(offsets + num_src, &num_edges, 8, cudaMemcpyHostToDevice), "offsets tail")) break;
        cudaFree(keys_a); cudaFree(keys_b); cudaFree(temp);
        keys_a = keys_b = nullptr; temp = nullptr;
        if (weight_sigma > 0.f) {
            if (!cuda_ok(cudaMalloc(&w, std::max<uint64_t>(num_edges, 1) * 4), "cudaMalloc(weights)")) break;
            k_weights<<<grid_for(num_edges), 256>>>(w, num_edges, mix(p.seed ^ 0x77656967687473ull), weight_sigma);
            if (!cuda_ok(cudaGetLastError(), "k_weights")) break;
        }
        cuda_ok(cudaDeviceSynchronize(), "graph generation");
    } while (0);
    cudaFree(keys_a); cudaFree(keys_b); cudaFree(temp); cudaFree(hist_dev);
    if (st != AG_OK) { cudaFree(offsets); cudaFree(dst); cudaFree(w); return st; }
    *offsets_out = offsets; *dst_out = dst; *w_out = w;
    return AG_OK;
}

}  // namespace

// Sorts `n` 64-bit keys (row << 32 | value) by their low `32 + bits_row` bits and
// turns them into a CSR over `num_rows` rows: offsets[num_rows + 1] and the values
// in sorted order.  keys is consumed (freed); offsets / vals are cudaMalloc'ed.
int32_t keys_to_sorted_csr(uint64_t *keys, uint64_t n, uint64_t num_rows, uint64_t **offsets_out, uint32_t **vals_out) {
    uint64_t *alt = nullptr, *offsets = nullptr;
    uint32_t *vals = nullptr;
    void *temp = nullptr;
    int32_t st = AG_OK;
    auto ok = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == AG_OK) st = fail(AG_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
        return e == cudaSuccess;
    };
    uint64_t *sorted = keys;
    do {
        if (n) {
            if (!ok(cudaMalloc(&alt, n * 8), "cudaMalloc(sort buffer)")) break;
            cub::DoubleBuffer<uint64_t> buf(keys, alt);
            size_t temp_bytes = 0;
            const int end_bit = 32 + (int)bits_for(std::max<uint64_t>(num_rows, 2));
            if (!ok(cub::DeviceRadixSort::SortKeys(nullptr, temp_bytes, buf, n, 0, end_bit), "sort sizing")) break;
            if (!ok(cudaMalloc(&temp, std::max<size_t>(temp_bytes, 16)), "cudaMalloc(sort temp)")) break;
            if (!ok(cub::DeviceRadixSort::SortKeys(temp, temp_bytes, buf, n, 0, end_bit), "radix sort")) break;
            if (!ok(cudaDeviceSynchronize(), "radix sort")) break;
            sorted = buf.Current();
            cudaFree(temp); temp = nullptr;
            if (sorted == keys) { cudaFree(alt); alt = nullptr; } else { cudaFree(keys); keys = nullptr; }
        }
        if (!ok(cudaMalloc(&offsets, (num_rows + 1) * 8), "cudaMalloc(offsets)")) break;
        if (!ok(cudaMalloc(&vals, std::max<uint64_t>(n, 1) * 4), "cudaMalloc(values)")) break;
        k_keys_to_csr<<<grid_for(std::max<uint64_t>(n, num_rows + 1)), 256>>>(sorted, n, num_rows, offsets, vals);
        if (!ok(cudaGetLastError(), "k_keys_to_csr")) break;
        ok(cudaDeviceSynchronize(), "k_keys_to_csr");
    } while (0);
    cudaFree(temp); cudaFree(keys); cudaFree(alt);
    if (st != AG_OK) { cudaFree(offsets); cudaFree(vals); return st; }
    *offsets_out = offsets; *vals_out = vals;
    return AG_OK;
}

}  // namespace ag

using namespace ag;

extern "C" int32_t ag_synth_rmat_csr(uint64_t num_src, uint64_t num_dst, uint64_t num_edges, float a, float b, float c,
                                     uint64_t seed, float weight_sigma, int32_t device, uint64_t **offsets_dev,
                                     uint32_t **dst_dev, float **weights_dev) {
    if (!offsets_dev || !dst_dev || !weights_dev) return fail(AG_ERR_VALUE, "ag_synth_rmat_csr: null argument");
    if (!(a > 0.f && b >= 0.f && c >= 0.f && a + b + c < 1.f)) return fail(AG_ERR_VALUE, "R-MAT needs a > 0, b, c >= 0, a + b + c < 1");
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    const float abc[3] = {a, b, c};
    return build_relation(num_src, num_dst, num_edges, abc, seed, weight_sigma, device, offsets_dev, dst_dev, weights_dev);
}

extern "C" int32_t ag_synth_rmat_graph(uint64_t num_nodes, uint64_t num_edges, float a, float b, float c,
                                       uint64_t seed, float weight_sigma, int32_t device, ag_graph **out) {
    if (!out) return fail(AG_ERR_VALUE, "ag_synth_rmat_graph: null argument");
    uint64_t *off = nullptr;
    uint32_t *dst = nullptr;
    float *w = nullptr;
    AG_TRY(ag_synth_rmat_csr(num_nodes, num_nodes, num_edges, a, b, c, seed, weight_sigma, device, &off, &dst, &w));
    const int32_t st = ag_graph_adopt_device_csr(num_nodes, num_edges, off, dst, w, device, out);
    if (st != AG_OK) { DeviceGuard guard(device); cudaFree(off); cudaFree(dst); cudaFree(w); }
    return st;
}

extern "C" int32_t ag_synth_fixed_degree_csr(uint64_t num_src, uint64_t num_dst, uint32_t degree, uint64_t seed,
                                             int32_t device, uint64_t **offsets_dev, uint32_t **dst_dev) {
    if (!offsets_dev || !dst_dev || num_dst == 0) return fail(AG_ERR_VALUE, "ag_synth_fixed_degree_csr: bad argument");
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint64_t *off = nullptr;
    uint32_t *dst = nullptr;
    AG_CUDA(cudaMalloc(&off, (num_src + 1) * 8));
    if (cudaMalloc(&dst, std::max<uint64_t>(num_src * degree, 1) * 4) != cudaSuccess) {
        cudaFree(off);
        return fail(AG_ERR_CUDA, "out of device memory");
    }
    k_fixed_degree<<<grid_for(num_src + 1), 256>>>(num_src, num_dst, degree, seed, off, dst);
    const cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaFree(off); cudaFree(dst); return fail(AG_ERR_CUDA, "k_fixed_degree: %s", cudaGetErrorString(e)); }
    *offsets_dev = off; *dst_dev = dst;
    return AG_OK;
}

extern "C" int32_t ag_synth_free_device(void *ptr, int32_t device) {
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    cudaFree(ptr);
    return AG_OK;
}

namespace {
int32_t synth_feature_rows(uint64_t num_nodes, uint64_t dim, int32_t dtype, uint64_t seed, int32_t device,
                           uint64_t row_begin, uint64_t row_stride, uint64_t rows, ag_features **out) {
    if (!out) return fail(AG_ERR_VALUE, "ag_synth_features: null argument");
    if (dtype < 0 || dtype > AG_I8) return fail(AG_ERR_VALUE, "unknown feature dtype tag: %d", dtype);
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    if (dtype == AG_I8) {
        // the same values as the f32 table, quantised block by block: generated and encoded a slab of rows at a time
        if (row_stride != 1 || dim == 0) return fail(AG_ERR_VALUE, "the int8 payload is generated for contiguous rows of a non-zero dim");
        const uint64_t bpr = (dim + kQuantBlock - 1) / kQuantBlock;
        int8_t *codes = nullptr;
        float *scales = nullptr, *slab = nullptr;
        uint32_t *bad = nullptr;
        const uint64_t slab_rows = std::max<uint64_t>(1, std::min<uint64_t>(rows, (256ull << 20) / (dim * 4)));
        cudaError_t e = cudaMalloc(&codes, std::max<uint64_t>(rows * dim, 16));
        if (e == cudaSuccess) e = cudaMalloc(&scales, std::max<uint64_t>(rows * bpr * 4, 16));
        if (e == cudaSuccess) e = cudaMalloc(&slab, slab_rows * dim * 4);
        if (e == cudaSuccess) e = cudaMalloc(&bad, 4);
        if (e == cudaSuccess) e = cudaMemset(bad, 0, 4);
        for (uint64_t r0 = 0; r0 < rows && e == cudaSuccess; r0 += slab_rows) {
            const uint64_t m = std::min(slab_rows, rows - r0);
            k_features<<<grid_for(m * dim), 256>>>((uint8_t *)slab, row_begin + r0, 1, m, dim, AG_F32, seed);
            e = launch_encode_i8(slab, m, dim, codes + r0 * dim, scales + r0 * bpr, bad, 0);
        }
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        cudaFree(slab); cudaFree(bad);
        ag_features *f = nullptr;
        int32_t st = e == cudaSuccess ? ag_features_adopt_device(codes, rows, dim, AG_I8, device, &f)
                                      : fail(AG_ERR_CUDA, "int8 feature generation failed: %s", cudaGetErrorString(e));
        if (st != AG_OK) { cudaFree(codes); cudaFree(scales); return st; }
        f->num_nodes = num_nodes; f->row_begin = row_begin; f->rows = rows; f->owns_payload = true; f->scales = scales;
        *out = f;
        return AG_OK;
    }
    PeerBlock *block = nullptr;  // peers can map it with large pages when the store becomes a shard
    uint8_t *payload = nullptr;
    AG_TRY(alloc_feature_payload(device, std::max<uint64_t>(rows * dim * elem_size(dtype), 16), &payload, &block));
    k_features<<<grid_for(rows * dim), 256>>>(payload, row_begin, row_stride, rows, dim, dtype, seed);
    const cudaError_t e = cudaDeviceSynchronize();
    auto drop = [&] { if (block) peer_block_free(block); else cudaFree(payload); };
    if (e != cudaSuccess) { drop(); return fail(AG_ERR_CUDA, "k_features: %s", cudaGetErrorString(e)); }
    ag_features *f = nullptr;
    const int32_t st = ag_features_adopt_device(payload, rows, dim, dtype, device, &f);
    if (st != AG_OK) { drop(); return st; }
    f->block = block;
    f->num_nodes = num_nodes; f->row_begin = row_begin; f->rows = rows; f->row_stride = row_stride; f->owns_payload = true;
    *out = f;
    return AG_OK;
}
}  // namespace

extern "C" int32_t ag_synth_features(uint64_t num_nodes, uint64_t dim, int32_t dtype, uint64_t seed, int32_t device,
                                     uint64_t row_begin, uint64_t row_end, ag_features **out) {
    row_end = std::min(row_end, num_nodes);
    row_begin = std::min(row_begin, row_end);
    return synth_feature_rows(num_nodes, dim, dtype, seed, device, row_begin, 1, row_end - row_begin, out);
}

extern "C" int32_t ag_synth_features_shard(uint64_t num_nodes, uint64_t dim, int32_t dtype, uint64_t seed, int32_t device,
                                           uint32_t rank, uint32_t world, int32_t layout, ag_features **out) {
    if (world == 0 || rank >= world) return fail(AG_ERR_VALUE, "ag_synth_features_shard: bad rank %u of %u", rank, world);
    if (layout == AG_SHARD_CYCLIC && world > 1) {
        const uint64_t rows = num_nodes > rank ? (num_nodes - rank + world - 1) / world : 0;
        return synth_feature_rows(num_nodes, dim, dtype, seed, device, rank, world, rows, out);
    }
    if (layout != AG_SHARD_RANGE && layout != AG_SHARD_CYCLIC) return fail(AG_ERR_VALUE, "unknown shard layout %d", layout);
    const uint64_t per = (num_nodes + world - 1) / world;
    const uint64_t begin = std::min<uint64_t>((uint64_t)rank * per, num_nodes), end = std::min<uint64_t>(begin + per, num_nodes);
    return synth_feature_rows(num_nodes, dim, dtype, seed, device, begin, 1, end - begin, out);
}

// A copy of the hottest feature rows on every GPU of a sharded store.
//
// On a skewed graph most gathered rows belong to few vertices: the rows a
// minibatch gathers are the destinations of sampled edges, so a vertex is asked
// for in proportion to its in-degree, and in a power-law graph a percent of the
// vertices holds most of the in-degree (R-MAT a=.57 b=c=.19 on 2^27 vertices: 1 %
// of the vertices are the destination of 69 % of the edges).  A sharded store
// therefore keeps, beside its 1/W of the table, a copy of the K rows with the
// highest in-degree; a gather serves those from local HBM and only the cold rest
// crosses NVLink.  The copy is a cache of rows that never change, so there is
// nothing to keep coherent, and the gathered values are the same bits.
//
// The reference's counterpart is the GPU-resident hot tier of its feature cache,
// in which the hottest nodes are pinned when frequencies are known
// (crates/aethergraph-core/src/features/cache/mod.rs:1-20), in front of its
// sharded remote gather (crates/aether-stream/src/rdma/sharded.rs:1-33).
#include <cub/device/device_radix_sort.cuh>

#include <algorithm>

#include "common.cuh"
#include "internal.h"

using namespace ag;

namespace {

__global__ void k_in_degree(const uint32_t *__restrict__ dst, uint64_t e, uint64_t n, uint32_t *cnt) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t d = ld_stream_u32(dst + i);
        if (d < n) atomicAdd(cnt + d, 1u);
    }
}

// key = ~in-degree (ascending sort = hottest first), value = vertex id
__global__ void k_degree_keys(const uint32_t *cnt, uint64_t n, uint32_t *keys, uint32_t *vals) {
    for (uint64_t v = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; v < n; v += (uint64_t)gridDim.x * blockDim.x) {
        keys[v] = ~cnt[v];
        vals[v] = (uint32_t)v;
    }
}

__global__ void k_set_slots(const uint32_t *ids, uint64_t n, uint64_t num_nodes, uint32_t *slot, uint32_t *err) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t v = ids[i];
        if (v < num_nodes) slot[v] = (uint32_t)i; else atomicOr(err, kErrBadId);
    }
}

int grid_of(uint64_t n) { return (int)std::max<uint64_t>(1, std::min<uint64_t>((n + 255) / 256, (uint64_t)kSMs * 16)); }

}  // namespace

// The `max_rows` vertices with the highest in-degree, hottest first, as a device
// array the caller frees with ag_synth_free_device.  Vertices nobody points at are
// never returned, so *n_out may be smaller than max_rows.
extern "C" int32_t ag_graph_hot_vertices(const ag_graph *g, uint64_t max_rows, uint32_t **ids_dev, uint64_t *n_out) {
    if (!g || !ids_dev || !n_out) return fail(AG_ERR_VALUE, "ag_graph_hot_vertices: null argument");
    *ids_dev = nullptr; *n_out = 0;
    const uint64_t n = g->num_nodes;
    if (n == 0 || max_rows == 0 || g->num_edges == 0) return AG_OK;
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint32_t *cnt = nullptr, *keys[2] = {nullptr, nullptr}, *vals[2] = {nullptr, nullptr}, *out = nullptr;
    void *temp = nullptr;
    int32_t st = AG_OK;
    auto ok = [&](cudaError_t e, const char *what) {
        if (e != cudaSuccess && st == AG_OK) st = fail(AG_ERR_CUDA, "%s failed: %s", what, cudaGetErrorString(e));
        return e == cudaSuccess;
    };
    do {
        if (!ok(cudaMalloc(&cnt, n * 4), "cudaMalloc(in-degrees)") || !ok(cudaMemset(cnt, 0, n * 4), "cudaMemset")) break;
        k_in_degree<<<grid_of(g->num_edges), 256>>>(g->dst, g->num_edges, n, cnt);
        for (int i = 0; i < 2; ++i)
            if (!ok(cudaMalloc(&keys[i], n * 4), "cudaMalloc(sort keys)") || !ok(cudaMalloc(&vals[i], n * 4), "cudaMalloc(sort values)")) break;
        if (st != AG_OK) break;
        k_degree_keys<<<grid_of(n), 256>>>(cnt, n, keys[0], vals[0]);
        size_t tb = 0;
        if (!ok(cub::DeviceRadixSort::SortPairs(nullptr, tb, (const uint32_t *)keys[0], keys[1], (const uint32_t *)vals[0], vals[1], n), "sort sizing")) break;
        if (!ok(cudaMalloc(&temp, std::max<size_t>(tb, 16)), "cudaMalloc(sort temp)")) break;
        if (!ok(cub::DeviceRadixSort::SortPairs(temp, tb, (const uint32_t *)keys[0], keys[1], (const uint32_t *)vals[0], vals[1], n), "radix sort")) break;
        // drop the tail of vertices with in-degree 0 (key 0xFFFFFFFF): find how many of the first max_rows have one
        uint64_t take = std::min<uint64_t>(max_rows, n);
        uint32_t last_key = 0;
        if (!ok(cudaMemcpy(&last_key, keys[1] + (take - 1), 4, cudaMemcpyDeviceToHost), "read back")) break;
        if (last_key == 0xFFFFFFFFu) {
            // binary search for the first zero-degree vertex among the sorted keys
            uint64_t lo = 0, hi = take;  // keys[lo-1] != ~0, keys[hi-1] == ~0
            while (lo < hi) {
                const uint64_t mid = (lo + hi) / 2;
                uint32_t km = 0;
                if (!ok(cudaMemcpy(&km, keys[1] + mid, 4, cudaMemcpyDeviceToHost), "read back")) break;
                if (km == 0xFFFFFFFFu) hi = mid; else lo = mid + 1;
            }
            if (st != AG_OK) break;
            take = lo;
        }
        if (take == 0) break;
        if (!ok(cudaMalloc(&out, take * 4), "cudaMalloc(hot ids)")) break;
        if (!ok(cudaMemcpy(out, vals[1], take * 4, cudaMemcpyDeviceToDevice), "copy")) break;
        *ids_dev = out; *n_out = take;
        out = nullptr;
    } while (0);
    cudaFree(cnt); cudaFree(keys[0]); cudaFree(keys[1]); cudaFree(vals[0]); cudaFree(vals[1]); cudaFree(temp); cudaFree(out);
    return st;
}

// Copies the stored rows of `ids_dev` (device, n vertex ids, no repeats) into this
// GPU's memory and makes the sharded view serve them from there.  Replaces an
// earlier copy.  No gather over the view may be running or be started meanwhile.
extern "C" int32_t ag_features_cache_rows(ag_features *view, const uint32_t *ids_dev, uint64_t n) {
    if (!view || (!ids_dev && n)) return fail(AG_ERR_VALUE, "ag_features_cache_rows: null argument");
    if (!view->shards || view->n_shards == 0) return fail(AG_ERR_VALUE, "ag_features_cache_rows: the store is not a sharded view");
    const uint64_t row_bytes = view->dim * elem_size(view->dtype);
    if (row_bytes == 0 || row_bytes % 4 != 0) return fail(AG_ERR_VALUE, "ag_features_cache_rows: rows must be a whole number of 4-byte words");
    if (n >= 0xFFFFFFFFull) return fail(AG_ERR_VALUE, "ag_features_cache_rows: too many rows");
    DeviceGuard guard(view->device);
    if (!guard.ok) return AG_ERR_CUDA;
    AG_CUDA(cudaDeviceSynchronize());
    ag_shard_table t{};
    AG_CUDA(cudaMemcpy(&t, view->shards, sizeof(t), cudaMemcpyDeviceToHost));
    // back to the plain view first: the rows are fetched through it
    t.base[t.n_shards] = nullptr; t.n_sources = t.n_shards; t.hot_slot = nullptr;
    AG_CUDA(cudaMemcpy(view->shards, &t, sizeof(t), cudaMemcpyHostToDevice));
    cudaFree(view->hot_rows); cudaFree(view->hot_slot);
    view->hot_rows = nullptr; view->hot_slot = nullptr; view->hot_n = 0;
    AG_CUDA(cudaMemset((uint8_t *)view->err + 8, 0, 24));  // the counters start over
    if (n == 0) return AG_OK;
    uint8_t *rows = nullptr;
    uint32_t *slot = nullptr;
    int32_t st = AG_OK;
    do {
        if (cudaMalloc(&rows, n * row_bytes) != cudaSuccess || cudaMalloc(&slot, view->num_nodes * 4) != cudaSuccess ||
            cudaMemset(slot, 0xFF, view->num_nodes * 4) != cudaSuccess) {
            st = fail(AG_ERR_CUDA, "ag_features_cache_rows: out of device memory for %llu rows: %s", (unsigned long long)n,
                      cudaGetErrorString(cudaGetLastError()));
            break;
        }
        // A gather of raw rows: the stored row seen as row_bytes / 4 words of f32 is copied bit for bit.
        const bool vec = row_bytes % 16 == 0 && ((uintptr_t)rows % 16) == 0;
        const uint64_t chunk = 4ull << 20;  // rows per launch (the address-ordered gather takes < 2^23)
        for (uint64_t done = 0; done < n && st == AG_OK; done += chunk) {
            const uint64_t m = std::min(chunk, n - done);
            GatherArgs a{};
            set_gather_source(a, view);
            a.dim = (uint32_t)(row_bytes / 4);
            a.ids = ids_dev + done; a.ids64 = 0; a.n = m; a.n_dev = nullptr;
            a.out = (float *)(rows + done * row_bytes);
            cudaError_t e;
            if (view->sort && vec && sorted_gather_applies(view, (uint32_t)row_bytes, true))
                e = launch_gather_sorted(a, nullptr, 1, m, (uint32_t)row_bytes, a.dim, AG_F32, view, view->sort->scratch, 0);
            else
                e = launch_gather(a, AG_F32, 0);
            if (e == cudaSuccess) e = cudaDeviceSynchronize();
            if (e != cudaSuccess) st = fail(AG_ERR_CUDA, "ag_features_cache_rows: copying the rows failed: %s", cudaGetErrorString(e));
        }
        if (st != AG_OK) break;
        k_set_slots<<<grid_of(n), 256>>>(ids_dev, n, view->num_nodes, slot, view->err);
        if (cudaDeviceSynchronize() != cudaSuccess) { st = fail(AG_ERR_CUDA, "ag_features_cache_rows: %s", cudaGetErrorString(cudaGetLastError())); break; }
        uint32_t errbits = 0;
        cudaMemcpy(&errbits, view->err, 4, cudaMemcpyDeviceToHost);
        if (errbits) { cudaMemset(view->err, 0, 4); st = fail(AG_ERR_VALUE, "ag_features_cache_rows: a vertex id is out of bounds (num_nodes=%llu)", (unsigned long long)view->num_nodes); break; }
        t.base[t.n_shards] = rows; t.n_sources = t.n_shards + 1; t.hot_slot = slot;
        if (cudaMemcpy(view->shards, &t, sizeof(t), cudaMemcpyHostToDevice) != cudaSuccess) { st = fail(AG_ERR_CUDA, "ag_features_cache_rows: table update failed"); break; }
        view->hot_rows = rows; view->hot_slot = slot; view->hot_n = n;
        cudaMemset((uint8_t *)view->err + 8, 0, 24);  // the counters start over
        return AG_OK;
    } while (0);
    cudaFree(rows); cudaFree(slot);
    return st;
}

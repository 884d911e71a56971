// Subgraph rewrites applied after a sampling pass
// (crates/aethergraph-core/src/loader/sampler.rs:964-1040 apply_subgraph_type):
//   mirror  (bidirectional): the sampled edges stay, then the reverse of edge i is
//           appended, in the order of i, unless its (src_local, dst_local) pair is
//           already among the sampled edges or an earlier appended reverse;
//   induce  (induced): the edges become every stored edge between two sampled
//           nodes, ordered by the expanded node's local index, then row position.
// Both are exact restatements for parallel hardware: "first in order wins" is an
// atomicMin over edge positions in a hash table of pairs, "in order" is a prefix
// sum over keep flags.  Hash probes are bounded by the table size.
#include <cub/device/device_scan.cuh>

#include "common.cuh"
#include "internal.h"

using namespace ag;

namespace {

constexpr uint64_t kEmptyKey = ~0ull;

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
    x ^= x >> 33; x *= 0xff51afd7ed558ccdull; x ^= x >> 33; x *= 0xc4ceb9fe1a85ec53ull; x ^= x >> 33;
    return x;
}

// Finds `key` or claims an empty slot for it; returns the slot, or ~0 when the
// table is full (cannot happen at load <= 1/2; the caller records it).
__device__ __forceinline__ uint64_t find_or_insert(unsigned long long *keys, uint64_t mask, uint64_t key) {
    uint64_t slot = mix64(key) & mask;
    for (uint64_t probe = 0; probe <= mask; ++probe) {
        const unsigned long long cur = keys[slot];
        if (cur == key) return slot;
        if (cur == kEmptyKey) {
            const unsigned long long prev = atomicCAS(&keys[slot], (unsigned long long)kEmptyKey, (unsigned long long)key);
            if (prev == kEmptyKey || prev == key) return slot;
        }
        slot = (slot + 1) & mask;
    }
    return ~0ull;
}

__device__ __forceinline__ uint64_t find(const unsigned long long *keys, uint64_t mask, uint64_t key) {
    uint64_t slot = mix64(key) & mask;
    for (uint64_t probe = 0; probe <= mask; ++probe) {
        const unsigned long long cur = keys[slot];
        if (cur == key) return slot;
        if (cur == kEmptyKey) return ~0ull;
        slot = (slot + 1) & mask;
    }
    return ~0ull;
}

__device__ __forceinline__ uint64_t pair_key(uint32_t a, uint32_t b) { return ((uint64_t)a << 32) | b; }

// Phase 1: every sampled pair enters the table with value 0 ("forward").
__global__ void k_mirror_forward(const uint32_t *__restrict__ sl, const uint32_t *__restrict__ dl, uint64_t n,
                                 unsigned long long *keys, uint32_t *vals, uint64_t mask, uint32_t *err) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t slot = find_or_insert(keys, mask, pair_key(sl[i], dl[i]));
        if (slot == ~0ull) { atomicOr(err, 1u); continue; }
        atomicMin(&vals[slot], 0u);
    }
}

// Phase 2: the reverse pair of edge i competes with value i + 1; a pair that is a
// forward pair keeps 0, otherwise the smallest i wins.
__global__ void k_mirror_reverse(const uint32_t *__restrict__ sl, const uint32_t *__restrict__ dl, uint64_t n,
                                 unsigned long long *keys, uint32_t *vals, uint64_t mask, uint32_t *err) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t slot = find_or_insert(keys, mask, pair_key(dl[i], sl[i]));
        if (slot == ~0ull) { atomicOr(err, 1u); continue; }
        atomicMin(&vals[slot], (uint32_t)(i + 1));
    }
}

__global__ void k_mirror_flags(const uint32_t *__restrict__ sl, const uint32_t *__restrict__ dl, uint64_t n,
                               const unsigned long long *keys, const uint32_t *vals, uint64_t mask, uint32_t *flags) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t slot = find(keys, mask, pair_key(dl[i], sl[i]));
        flags[i] = (slot != ~0ull && vals[slot] == (uint32_t)(i + 1)) ? 1u : 0u;
    }
}

// Appends the winners behind the n sampled edges.  rank = exclusive prefix of flags.
__global__ void k_mirror_append(uint32_t *edge_src, uint32_t *edge_dst, uint32_t *sl, uint32_t *dl, uint64_t *edge_ids,
                                uint64_t n, const uint32_t *__restrict__ flags, const uint32_t *__restrict__ rank) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        if (!flags[i]) continue;
        const uint64_t o = n + rank[i];
        edge_src[o] = edge_dst[i]; edge_dst[o] = edge_src[i];
        sl[o] = dl[i]; dl[o] = sl[i];
        if (edge_ids) edge_ids[o] = edge_ids[i];
    }
}

// int64 [2, e]: row 0 the neighbor's local index, row 1 the expanded node's.
__global__ void k_edge_index_local(const uint32_t *__restrict__ sl, const uint32_t *__restrict__ dl, uint64_t e, int64_t *out) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < e; i += (uint64_t)gridDim.x * blockDim.x) {
        out[i] = (int64_t)dl[i];
        out[e + i] = (int64_t)sl[i];
    }
}

uint64_t pow2_at_least(uint64_t v) {
    uint64_t p = 1024;
    while (p < v) p <<= 1;
    return p;
}

uint32_t grid_for(uint64_t n) { return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((n + 255) / 256, (uint64_t)kSMs * 8)); }

struct Scratch {
    void *p[6] = {};
    ~Scratch() { for (void *q : p) if (q) cudaFree(q); }
};

}  // namespace

// In place on the device arrays of one sampled subgraph.  The four u32 edge arrays
// (and edge_ids when given) hold n_edges entries and room for 2 * n_edges;
// edge_index_local (optional) has room for [2, 2 * n_edges] and is rewritten for the
// new edge count.  *n_edges_out (host) receives the new count.  Synchronous.
extern "C" int32_t ag_subgraph_mirror(int32_t device, uint64_t n_edges, uint64_t cap_edges, uint32_t *edge_src,
                                      uint32_t *edge_dst, uint32_t *src_local, uint32_t *dst_local, uint64_t *edge_ids,
                                      int64_t *edge_index_local, uint64_t *n_edges_out, void *stream) {
    if (!n_edges_out) return fail(AG_ERR_VALUE, "ag_subgraph_mirror: null argument");
    *n_edges_out = n_edges;
    if (n_edges == 0) return AG_OK;
    if (!edge_src || !edge_dst || !src_local || !dst_local) return fail(AG_ERR_VALUE, "ag_subgraph_mirror: null edge array");
    if (cap_edges < 2 * n_edges) return fail(AG_ERR_VALUE, "ag_subgraph_mirror: capacity %llu < 2 x %llu edges",
                                             (unsigned long long)cap_edges, (unsigned long long)n_edges);
    if (n_edges >= 0x7FFFFFFFull) return fail(AG_ERR_VALUE, "ag_subgraph_mirror: too many edges");
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    const uint64_t cap = pow2_at_least(4 * n_edges), mask = cap - 1;  // <= 2n keys: load <= 1/2
    Scratch sc;
    unsigned long long *keys = nullptr; uint32_t *vals = nullptr, *flags = nullptr, *rank = nullptr, *err = nullptr;
    AG_CUDA(cudaMalloc(&sc.p[0], cap * 8)); keys = (unsigned long long *)sc.p[0];
    AG_CUDA(cudaMalloc(&sc.p[1], cap * 4)); vals = (uint32_t *)sc.p[1];
    AG_CUDA(cudaMalloc(&sc.p[2], (n_edges + 1) * 4)); flags = (uint32_t *)sc.p[2];
    AG_CUDA(cudaMalloc(&sc.p[3], (n_edges + 1) * 4)); rank = (uint32_t *)sc.p[3];
    AG_CUDA(cudaMalloc(&sc.p[4], 4)); err = (uint32_t *)sc.p[4];
    AG_CUDA(cudaMemsetAsync(keys, 0xFF, cap * 8, st));
    AG_CUDA(cudaMemsetAsync(vals, 0xFF, cap * 4, st));
    AG_CUDA(cudaMemsetAsync(err, 0, 4, st));
    AG_CUDA(cudaMemsetAsync(flags + n_edges, 0, 4, st));
    const uint32_t grid = grid_for(n_edges);
    k_mirror_forward<<<grid, 256, 0, st>>>(src_local, dst_local, n_edges, keys, vals, mask, err);
    k_mirror_reverse<<<grid, 256, 0, st>>>(src_local, dst_local, n_edges, keys, vals, mask, err);
    k_mirror_flags<<<grid, 256, 0, st>>>(src_local, dst_local, n_edges, keys, vals, mask, flags);
    size_t temp_bytes = 0;
    AG_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, flags, rank, (int)(n_edges + 1), st));
    AG_CUDA(cudaMalloc(&sc.p[5], std::max<size_t>(temp_bytes, 16)));
    AG_CUDA(cub::DeviceScan::ExclusiveSum(sc.p[5], temp_bytes, flags, rank, (int)(n_edges + 1), st));
    k_mirror_append<<<grid, 256, 0, st>>>(edge_src, edge_dst, src_local, dst_local, edge_ids, n_edges, flags, rank);
    uint32_t added = 0, herr = 0;
    AG_CUDA(cudaMemcpyAsync(&added, rank + n_edges, 4, cudaMemcpyDeviceToHost, st));
    AG_CUDA(cudaMemcpyAsync(&herr, err, 4, cudaMemcpyDeviceToHost, st));
    AG_CUDA(cudaStreamSynchronize(st));
    if (herr) return fail(AG_ERR_WORKER, "ag_subgraph_mirror: pair table overflow");
    const uint64_t total = n_edges + added;
    if (edge_index_local) {
        k_edge_index_local<<<grid_for(total), 256, 0, st>>>(src_local, dst_local, total, edge_index_local);
        AG_CUDA(cudaStreamSynchronize(st));
    }
    AG_CUDA(cudaGetLastError());
    *n_edges_out = total;
    return AG_OK;
}

// ------------------------------------------------------------------ induce --
namespace {

constexpr uint32_t kEmptyNode = 0xFFFFFFFFu;

__device__ __forceinline__ uint32_t node_slot(uint32_t v, uint32_t mask) { return (uint32_t)(mix64(v) & mask); }

// The sampled nodes are distinct: node -> local index.
__global__ void k_induce_insert(const uint32_t *__restrict__ nodes, uint64_t n, uint32_t *keys, uint32_t *vals, uint32_t mask,
                                uint32_t *err) {
    for (uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t v = nodes[i];
        uint32_t slot = node_slot(v, mask);
        bool done = false;
        for (uint32_t probe = 0; probe <= mask && !done; ++probe) {
            const uint32_t prev = atomicCAS(&keys[slot], kEmptyNode, v);
            if (prev == kEmptyNode || prev == v) { vals[slot] = (uint32_t)i; done = true; }
            else slot = (slot + 1) & mask;
        }
        if (!done) atomicOr(err, 1u);
    }
}

__device__ __forceinline__ uint32_t node_lookup(const uint32_t *__restrict__ keys, const uint32_t *__restrict__ vals,
                                                uint32_t mask, uint32_t v) {
    uint32_t slot = node_slot(v, mask);
    for (uint32_t probe = 0; probe <= mask; ++probe) {
        const uint32_t k = keys[slot];
        if (k == v) return vals[slot];
        if (k == kEmptyNode) return kEmptyNode;
        slot = (slot + 1) & mask;
    }
    return kEmptyNode;
}

// One warp per sampled node: walks the node's row 32 neighbours at a time.  With
// FILL the hits are written in row order behind row_start[u_local]; without, they
// are counted.
template <bool FILL>
__global__ void k_induce_rows(const uint64_t *__restrict__ offsets, const uint32_t *__restrict__ dst, uint64_t num_graph_nodes,
                              const uint32_t *__restrict__ nodes, uint64_t n, const uint32_t *__restrict__ keys,
                              const uint32_t *__restrict__ vals, uint32_t mask, uint64_t *row_count,
                              const uint64_t *__restrict__ row_start, uint32_t *edge_src, uint32_t *edge_dst, uint32_t *sl,
                              uint32_t *dl, uint64_t *edge_ids) {
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t u_local = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; u_local < n; u_local += warps) {
        const uint32_t u = nodes[u_local];
        uint64_t lo = 0, hi = 0;
        if ((uint64_t)u < num_graph_nodes) { lo = offsets[u]; hi = offsets[(uint64_t)u + 1]; }
        uint64_t out = FILL ? row_start[u_local] : 0, count = 0;
        for (uint64_t base = lo; base < hi; base += 32) {
            const uint64_t pos = base + lane;
            uint32_t w = 0, w_local = kEmptyNode;
            if (pos < hi) { w = dst[pos]; w_local = node_lookup(keys, vals, mask, w); }
            const uint32_t hits = __ballot_sync(0xFFFFFFFFu, w_local != kEmptyNode);
            if (FILL) {
                if (w_local != kEmptyNode) {
                    const uint64_t o = out + __popc(hits & ((1u << lane) - 1));
                    edge_src[o] = u; edge_dst[o] = w; sl[o] = (uint32_t)u_local; dl[o] = w_local;
                    if (edge_ids) edge_ids[o] = pos;
                }
                out += __popc(hits);
            } else {
                count += __popc(hits);
            }
        }
        if (!FILL && lane == 0) row_count[u_local] = count;
    }
}

}  // namespace

struct ag_induce_plan {
    int device = 0;
    const ag_graph *g = nullptr;
    const uint32_t *nodes = nullptr;
    uint64_t n_nodes = 0, n_edges = 0;
    uint32_t *keys = nullptr, *vals = nullptr, mask = 0;
    uint64_t *row_count = nullptr, *row_start = nullptr;
};

extern "C" void ag_subgraph_induce_free(ag_induce_plan *p) {
    if (!p) return;
    DeviceGuard guard(p->device);
    cudaFree(p->keys); cudaFree(p->vals); cudaFree(p->row_count); cudaFree(p->row_start);
    delete p;
}

// Step 1 of the induced rewrite: indexes the n_nodes sampled nodes (device u32 ids,
// distinct) and counts the stored edges between them; *n_edges_out (host) sizes the
// arrays for step 2.  `nodes_dev` must stay valid until the plan is freed.  Synchronous.
extern "C" int32_t ag_subgraph_induce_plan(const ag_graph *g, const uint32_t *nodes_dev, uint64_t n_nodes, void *stream,
                                           ag_induce_plan **out, uint64_t *n_edges_out) {
    if (!g || !out || !n_edges_out || (!nodes_dev && n_nodes)) return fail(AG_ERR_VALUE, "ag_subgraph_induce_plan: null argument");
    if (n_nodes >= 0x40000000ull) return fail(AG_ERR_VALUE, "ag_subgraph_induce_plan: too many nodes");
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    ag_induce_plan *p = new ag_induce_plan();
    p->device = g->device; p->g = g; p->nodes = nodes_dev; p->n_nodes = n_nodes;
    *out = nullptr; *n_edges_out = 0;
    if (n_nodes == 0) { *out = p; return AG_OK; }
    const uint64_t cap = pow2_at_least(2 * n_nodes);
    p->mask = (uint32_t)(cap - 1);
    void *temp = nullptr; uint32_t *err = nullptr;
    auto bail = [&](int32_t rc) { cudaFree(temp); cudaFree(err); ag_subgraph_induce_free(p); return rc; };
#define AG_PLAN_CUDA(expr) do { const cudaError_t e_ = (expr); if (e_ != cudaSuccess) \
        return bail(fail(AG_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_))); } while (0)
    AG_PLAN_CUDA(cudaMalloc(&p->keys, cap * 4));
    AG_PLAN_CUDA(cudaMalloc(&p->vals, cap * 4));
    AG_PLAN_CUDA(cudaMalloc(&p->row_count, (n_nodes + 1) * 8));
    AG_PLAN_CUDA(cudaMalloc(&p->row_start, (n_nodes + 1) * 8));
    AG_PLAN_CUDA(cudaMalloc(&err, 4));
    AG_PLAN_CUDA(cudaMemsetAsync(p->keys, 0xFF, cap * 4, st));
    AG_PLAN_CUDA(cudaMemsetAsync(err, 0, 4, st));
    AG_PLAN_CUDA(cudaMemsetAsync(p->row_count + n_nodes, 0, 8, st));
    k_induce_insert<<<grid_for(n_nodes), 256, 0, st>>>(nodes_dev, n_nodes, p->keys, p->vals, p->mask, err);
    const uint32_t grid = grid_for(n_nodes * 32);
    k_induce_rows<false><<<grid, 256, 0, st>>>(g->offsets, g->dst, g->num_nodes, nodes_dev, n_nodes, p->keys, p->vals, p->mask,
                                               p->row_count, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr);
    size_t temp_bytes = 0;
    AG_PLAN_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, p->row_count, p->row_start, (int)(n_nodes + 1), st));
    AG_PLAN_CUDA(cudaMalloc(&temp, std::max<size_t>(temp_bytes, 16)));
    AG_PLAN_CUDA(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, p->row_count, p->row_start, (int)(n_nodes + 1), st));
    uint64_t total = 0; uint32_t herr = 0;
    AG_PLAN_CUDA(cudaMemcpyAsync(&total, p->row_start + n_nodes, 8, cudaMemcpyDeviceToHost, st));
    AG_PLAN_CUDA(cudaMemcpyAsync(&herr, err, 4, cudaMemcpyDeviceToHost, st));
    AG_PLAN_CUDA(cudaStreamSynchronize(st));
    AG_PLAN_CUDA(cudaGetLastError());
#undef AG_PLAN_CUDA
    cudaFree(temp); cudaFree(err);
    if (herr) { ag_subgraph_induce_free(p); return fail(AG_ERR_WORKER, "ag_subgraph_induce_plan: node table overflow"); }
    p->n_edges = total;
    *n_edges_out = total;
    *out = p;
    return AG_OK;
}

// Step 2: writes the plan's edges (cap_edges >= the planned count).  edge_ids and
// edge_index_local ([2, n_edges] int64) are optional.  Synchronous.
extern "C" int32_t ag_subgraph_induce_fill(ag_induce_plan *p, uint64_t cap_edges, uint32_t *edge_src, uint32_t *edge_dst,
                                           uint32_t *src_local, uint32_t *dst_local, uint64_t *edge_ids,
                                           int64_t *edge_index_local, void *stream) {
    if (!p) return fail(AG_ERR_VALUE, "ag_subgraph_induce_fill: null plan");
    if (p->n_edges == 0) return AG_OK;
    if (!edge_src || !edge_dst || !src_local || !dst_local) return fail(AG_ERR_VALUE, "ag_subgraph_induce_fill: null edge array");
    if (cap_edges < p->n_edges) return fail(AG_ERR_VALUE, "ag_subgraph_induce_fill: capacity %llu < %llu edges",
                                            (unsigned long long)cap_edges, (unsigned long long)p->n_edges);
    DeviceGuard guard(p->device);
    if (!guard.ok) return AG_ERR_CUDA;
    cudaStream_t st = (cudaStream_t)stream;
    k_induce_rows<true><<<grid_for(p->n_nodes * 32), 256, 0, st>>>(p->g->offsets, p->g->dst, p->g->num_nodes, p->nodes, p->n_nodes,
                                                                   p->keys, p->vals, p->mask, nullptr, p->row_start, edge_src,
                                                                   edge_dst, src_local, dst_local, edge_ids);
    if (edge_index_local)
        k_edge_index_local<<<grid_for(p->n_edges), 256, 0, st>>>(src_local, dst_local, p->n_edges, edge_index_local);
    AG_CUDA(cudaGetLastError());
    AG_CUDA(cudaStreamSynchronize(st));
    return AG_OK;
}

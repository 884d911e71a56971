// Locality reordering: Rabbit Order communities and the relabelled graph.
//
// reference: crates/aethergraph-core/src/graph/reorder.rs
//   :142-262  rabbit_dendrogram — modularity-driven incremental aggregation
//   :46-105   Dendrogram::root / permutation / partitions
//   :297-383  Graph::permute
//
// The community detection is a sequential, deterministic merge in the reference
// (one vertex after the other in ascending degree order, exact integer gains), and it
// is one here: it runs on the host over a copy of the CSR, as a preprocessing step.
// What is parallel — applying a permutation to the graph — runs on the GPU: the
// inverse permutation with its duplicate check, the new row lengths, their scan, and
// one thread per edge that finds its new row by bisection and relabels its endpoint.
#include <cub/device/device_scan.cuh>

#include <algorithm>
#include <numeric>
#include <vector>

#include "common.cuh"
#include "internal.h"

using namespace ag;

namespace {

constexpr uint32_t kNone = 0xFFFFFFFFu;  // reorder.rs:30

// Blocks of 256 threads for n items, a whole number of waves at most: the kernels stride.
int grid_for(uint64_t n) {
    const uint64_t want = (n + 255) / 256;
    return (int)std::max<uint64_t>(1, std::min<uint64_t>(want, (uint64_t)kSMs * 16));
}

uint32_t find_root(std::vector<uint32_t> &parent, uint32_t v) {  // reorder.rs:46-59
    uint32_t r = v;
    while (parent[r] != r) r = parent[r];
    uint32_t x = v;
    while (parent[x] != r) {
        const uint32_t next = parent[x];
        parent[x] = r;
        x = next;
    }
    return r;
}

// flag bits: 1 an entry of perm is out of range, 2 a vertex appears twice
__global__ void k_invert_perm(const uint32_t *__restrict__ perm, uint64_t n, uint32_t *inv, uint32_t *flag) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t old_id = perm[i];
        if (old_id >= n) { atomicOr(flag, 1u); continue; }
        if (atomicCAS(&inv[old_id], kNone, (uint32_t)i) != kNone) atomicOr(flag, 2u);
    }
}

__global__ void k_new_row_lengths(const uint64_t *__restrict__ offsets, const uint32_t *__restrict__ perm, uint64_t n,
                                  uint64_t *__restrict__ lengths) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= n; i += (uint64_t)gridDim.x * blockDim.x)
        lengths[i] = i < n ? offsets[perm[i] + 1ull] - offsets[perm[i]] : 0ull;  // entry n: receives the total
}

// Edge e of the new graph: its row is the last new_offsets entry <= e; it is the
// (e - row start)-th edge of the old row perm[row], endpoint relabelled.
__global__ void k_fill_permuted(const uint64_t *__restrict__ old_offsets, const uint32_t *__restrict__ old_dst,
                                const float *__restrict__ old_w, const uint32_t *__restrict__ perm,
                                const uint32_t *__restrict__ inv, const uint64_t *__restrict__ new_offsets, uint64_t n,
                                uint64_t e_total, uint32_t *__restrict__ new_dst, float *__restrict__ new_w) {
    for (uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; e < e_total; e += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t lo = 0, hi = n;  // invariant: new_offsets[lo] <= e < new_offsets[hi]
        while (hi - lo > 1) {
            const uint64_t mid = (lo + hi) >> 1;
            if (new_offsets[mid] <= e) lo = mid; else hi = mid;
        }
        const uint64_t src = old_offsets[perm[lo]] + (e - new_offsets[lo]);
        new_dst[e] = inv[old_dst[src]];
        if (new_w) new_w[e] = old_w[src];
    }
}

struct Dev {
    void *p = nullptr;
    ~Dev() { cudaFree(p); }
    cudaError_t alloc(uint64_t bytes) { return cudaMalloc(&p, std::max<uint64_t>(bytes, 16)); }
    template <typename T> T *as() { return (T *)p; }
    void *release() { void *q = p; p = nullptr; return q; }
};

}  // namespace

extern "C" int32_t ag_graph_rabbit_order(const ag_graph *g, uint32_t *perm_out, uint32_t *partitions_out) {
    if (!g || (!perm_out && !partitions_out)) return fail(AG_ERR_VALUE, "ag_graph_rabbit_order: null argument");
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint64_t n = g->num_nodes, m = g->num_edges;
    std::vector<uint64_t> off(n + 1);
    std::vector<uint32_t> dst(m);
    AG_CUDA(cudaMemcpy(off.data(), g->offsets, (n + 1) * 8, cudaMemcpyDeviceToHost));
    if (m) AG_CUDA(cudaMemcpy(dst.data(), g->dst, m * 4, cudaMemcpyDeviceToHost));
    std::vector<uint32_t> parent(n), first_child(n, kNone), next_sibling(n, kNone);
    std::iota(parent.begin(), parent.end(), 0u);
    if (n > 1 && m > 0) {
        // in-edge transpose, sources ascending within a row (reorder.rs:111-136)
        std::vector<uint64_t> in_off(n + 1, 0);
        for (uint64_t e = 0; e < m; ++e) in_off[(uint64_t)dst[e] + 1]++;
        for (uint64_t v = 0; v < n; ++v) in_off[v + 1] += in_off[v];
        std::vector<uint32_t> in_src(m);
        {
            std::vector<uint64_t> cursor(in_off.begin(), in_off.end() - 1);
            for (uint64_t u = 0; u < n; ++u)
                for (uint64_t e = off[u]; e < off[u + 1]; ++e) in_src[cursor[dst[e]]++] = (uint32_t)u;
        }
        // undirected degree without self-loops; becomes the community degree (reorder.rs:169-183)
        std::vector<uint64_t> degree(n);
        uint64_t two_m = 0;
        for (uint64_t v = 0; v < n; ++v) {
            uint64_t d = 0;
            for (uint64_t e = off[v]; e < off[v + 1]; ++e) d += dst[e] != v;
            for (uint64_t e = in_off[v]; e < in_off[v + 1]; ++e) d += in_src[e] != v;
            degree[v] = d;
            two_m += d;
        }
        if (two_m != 0) {
            std::vector<uint32_t> order(n);
            std::iota(order.begin(), order.end(), 0u);
            std::sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) {
                return degree[a] != degree[b] ? degree[a] < degree[b] : a < b;  // (degree, v): a total order
            });
            std::vector<std::vector<std::pair<uint32_t, uint64_t>>> carried(n);
            std::vector<uint8_t> has_carried(n, 0), visited(n, 0);
            std::vector<uint64_t> weight_to(n, 0);
            std::vector<uint32_t> touched;
            for (const uint32_t u : order) {
                touched.clear();
                auto add = [&](uint32_t c, uint64_t w) {
                    c = find_root(parent, c);
                    if (c == u) return;
                    if (weight_to[c] == 0) touched.push_back(c);
                    weight_to[c] += w;
                };
                for (uint64_t e = off[u]; e < off[u + 1]; ++e) add(dst[e], 1);
                for (uint64_t e = in_off[u]; e < in_off[u + 1]; ++e) add(in_src[e], 1);
                for (uint32_t child = first_child[u]; child != kNone; child = next_sibling[child]) {
                    if (has_carried[child]) {
                        has_carried[child] = 0;
                        std::vector<std::pair<uint32_t, uint64_t>> list;
                        list.swap(carried[child]);
                        for (const auto &cw : list) add(cw.first, cw.second);
                    }
                }
                // gain of joining c, scaled by 2m^2: 2m w(u,c) - d(u) d(c), exact (reorder.rs:218-232)
                const __int128 du = (__int128)degree[u];
                bool have = false;
                __int128 best_gain = 0;
                uint32_t best = 0;
                for (const uint32_t c : touched) {
                    const __int128 gain = (__int128)two_m * (__int128)weight_to[c] - du * (__int128)degree[c];
                    const bool better = !have ? gain > 0 : (gain > best_gain || (gain == best_gain && c < best));
                    if (better) { have = true; best_gain = gain; best = c; }
                }
                if (have) {
                    parent[u] = best;
                    degree[best] += degree[u];
                    next_sibling[u] = first_child[best];  // prepend: most recent child first
                    first_child[best] = u;
                    if (!visited[best]) {
                        has_carried[u] = 1;
                        carried[u].reserve(touched.size());
                        for (const uint32_t t : touched) carried[u].emplace_back(t, weight_to[t]);
                    }
                }
                for (const uint32_t t : touched) weight_to[t] = 0;
                visited[u] = 1;
            }
        }
    }
    if (perm_out) {  // pre-order walk of every tree, roots in id order (reorder.rs:64-87)
        uint64_t at = 0;
        std::vector<uint32_t> stack;
        for (uint64_t root = 0; root < n; ++root) {
            if (parent[root] != root) continue;
            perm_out[at++] = (uint32_t)root;
            stack.push_back(first_child[root]);
            while (!stack.empty()) {
                const uint32_t c = stack.back();
                if (c == kNone) { stack.pop_back(); continue; }
                stack.back() = next_sibling[c];
                perm_out[at++] = c;
                stack.push_back(first_child[c]);
            }
        }
        if (at != n) return fail(AG_ERR_WORKER, "rabbit order: the dendrogram walk visited %llu of %llu vertices", (unsigned long long)at, (unsigned long long)n);
    }
    if (partitions_out) {  // dense ids by each community's first vertex (reorder.rs:90-104)
        std::vector<uint32_t> id_of_root(n, kNone);
        uint32_t next = 0;
        for (uint64_t v = 0; v < n; ++v) {
            const uint32_t r = find_root(parent, (uint32_t)v);
            if (id_of_root[r] == kNone) id_of_root[r] = next++;
            partitions_out[v] = id_of_root[r];
        }
    }
    return AG_OK;
}

extern "C" int32_t ag_graph_permute(const ag_graph *g, const uint32_t *perm, uint64_t perm_len, ag_graph **out) {
    if (!g || !out || (!perm && perm_len)) return fail(AG_ERR_VALUE, "ag_graph_permute: null argument");
    const uint64_t n = g->num_nodes, m = g->num_edges;
    if (perm_len != n) return fail(AG_ERR_VALUE, "permutation length mismatch: %llu entries for %llu nodes", (unsigned long long)perm_len, (unsigned long long)n);
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    Dev perm_d, inv, lengths, new_dst, new_w, flag, temp;
    if (perm_d.alloc(n * 4) != cudaSuccess || inv.alloc(n * 4) != cudaSuccess || lengths.alloc((n + 1) * 8) != cudaSuccess ||
        new_dst.alloc(m * 4) != cudaSuccess || (g->weights && new_w.alloc(m * 4) != cudaSuccess) || flag.alloc(4) != cudaSuccess)
        return fail(AG_ERR_CUDA, "out of device memory for the permuted graph: %s", cudaGetErrorString(cudaGetLastError()));
    if (n) AG_CUDA(cudaMemcpy(perm_d.p, perm, n * 4, cudaMemcpyHostToDevice));
    AG_CUDA(cudaMemset(inv.p, 0xFF, std::max<uint64_t>(n * 4, 4)));
    AG_CUDA(cudaMemset(flag.p, 0, 4));
    if (n) k_invert_perm<<<grid_for(n), 256>>>(perm_d.as<uint32_t>(), n, inv.as<uint32_t>(), flag.as<uint32_t>());
    uint32_t bad = 0;
    AG_CUDA(cudaMemcpy(&bad, flag.p, 4, cudaMemcpyDeviceToHost));
    if (bad & 1u) return fail(AG_ERR_VALUE, "the permutation names an out-of-range node");
    if (bad & 2u) return fail(AG_ERR_VALUE, "the permutation names a node twice (duplicate node)");
    k_new_row_lengths<<<grid_for(n + 1), 256>>>(g->offsets, perm_d.as<uint32_t>(), n, lengths.as<uint64_t>());
    size_t temp_bytes = 0;
    AG_CUDA(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, lengths.as<uint64_t>(), lengths.as<uint64_t>(), (size_t)(n + 1)));
    if (temp.alloc(temp_bytes) != cudaSuccess) return fail(AG_ERR_CUDA, "out of device memory for the scan");
    AG_CUDA(cub::DeviceScan::ExclusiveSum(temp.p, temp_bytes, lengths.as<uint64_t>(), lengths.as<uint64_t>(), (size_t)(n + 1)));
    uint64_t total = 0;
    AG_CUDA(cudaMemcpy(&total, lengths.as<uint64_t>() + n, 8, cudaMemcpyDeviceToHost));
    if (total != m) return fail(AG_ERR_LOAD, "permuted rows hold %llu edges, graph has %llu", (unsigned long long)total, (unsigned long long)m);
    if (m)
        k_fill_permuted<<<grid_for(m), 256>>>(g->offsets, g->dst, g->weights, perm_d.as<uint32_t>(), inv.as<uint32_t>(),
                                             lengths.as<uint64_t>(), n, m, new_dst.as<uint32_t>(),
                                             g->weights ? new_w.as<float>() : nullptr);
    AG_CUDA(cudaDeviceSynchronize());
    ag_graph *p = new ag_graph();
    p->device = g->device; p->num_nodes = n; p->num_edges = m;
    p->offsets = (uint64_t *)lengths.release();
    p->dst = (uint32_t *)new_dst.release();
    p->weights = g->weights ? (float *)new_w.release() : nullptr;
    *out = p;
    return AG_OK;
}

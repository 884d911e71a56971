// Feature stores sharded over the GPUs of one node.
//
// The reference scales past one machine's memory by partitioning the feature
// matrix across workers and fetching remote rows over the fabric
// (python/aethergraph/ray/datasource.py:6-10 keeps the topology replicated and
// the features partitioned; crates/aether-stream's RDMA gather is its transport).
// On one NVSwitch node the transport is a plain load: every GPU maps its peers'
// shards and the gather kernel reads row v straight out of the owner's HBM.  A
// payload the library allocated is a shareable block (peer_block.cu) that peers map
// with 2 MB pages, across processes or inside one; a payload adopted from the caller
// falls back to a legacy CUDA IPC handle, whose mapping is an order of magnitude
// slower to read at random once tens of GB are mapped.  The stored
// (bf16 / f16) row crosses NVLink; the upcast happens at the reader.  There is no
// staging buffer, no collective, and nothing here uses TMA.
//
// Two layouts.  AG_SHARD_RANGE is the reference's: contiguous vertex ranges,
// owner(v) = v / ceil(N / G).  On skewed graphs the low vertex ids are the hubs,
// so most sampled rows live in shard 0 and that GPU's NVLink egress becomes the
// bottleneck of all the others.  AG_SHARD_CYCLIC deals the rows round-robin,
// owner(v) = v % G, local row v / G: every vertex range, hot or cold, is spread
// evenly over the GPUs and the exchange is a balanced all-to-all.
#include <string.h>

#include <algorithm>

#include "common.cuh"
#include "internal.h"

using namespace ag;

namespace {

bool is_cyclic(const ag_features *f) { return f->row_stride > 1; }

int32_t make_view(const ag_features *local, uint32_t world, uint32_t rank, bool cyclic, const uint8_t *const *bases,
                  void *const *opened, PeerBlock *const *blocks, ag_features **out) {
    const uint64_t n = local->num_nodes;
    const uint64_t shard_rows = (n + world - 1) / world;
    ag_features *v = new ag_features();
    v->device = local->device;
    v->num_nodes = n; v->row_begin = 0; v->rows = n; v->dim = local->dim; v->dtype = local->dtype;
    v->payload = local->payload;  // borrowed: the view must not outlive the local shard
    for (uint32_t r = 0; r < world && !v->payload; ++r) v->payload = const_cast<uint8_t *>(bases[r]);
    v->owns_payload = false;
    v->n_shards = world;
    v->shard_rows = cyclic ? (n + world - 1) / world : std::max<uint64_t>(shard_rows, 1);
    v->shard_cyclic = cyclic;
    v->sort = new ag_features::SortState();
    for (uint32_t r = 0; r < world && opened; ++r) { v->ipc_opened[r] = opened[r]; v->legacy_peer |= opened[r] != nullptr; }
    for (uint32_t r = 0; r < world && blocks; ++r) v->peer_opened[r] = blocks[r];
    ag_shard_table t{};
    for (uint32_t r = 0; r < world; ++r) t.base[r] = bases[r];
    t.shard_rows = std::max<uint64_t>(shard_rows, 1);
    t.n_shards = world;
    t.n_sources = world;
    t.self = rank;
    t.hot_slot = nullptr;
    t.cyclic = cyclic ? 1u : 0u;
    if (cudaMalloc(&v->err, 32) != cudaSuccess || cudaMemset(v->err, 0, 32) != cudaSuccess ||
        cudaMalloc(&v->shards, sizeof(ag_shard_table)) != cudaSuccess ||
        cudaMemcpy(v->shards, &t, sizeof(t), cudaMemcpyHostToDevice) != cudaSuccess) {
        const int32_t st = fail(AG_ERR_CUDA, "sharded view allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
        ag_features_free(v);
        return st;
    }
    *out = v;
    return AG_OK;
}

// Does `local` hold exactly the rows shard `rank` of `world` must hold?
int32_t check_local(const ag_features *local, uint32_t world, uint32_t rank, const char *who) {
    if (world == 0 || world > 8 || rank >= world) return fail(AG_ERR_VALUE, "%s: bad rank %u of %u (at most 8 shards)", who, rank, world);
    if (local->shards) return fail(AG_ERR_VALUE, "%s: the local store is already a sharded view", who);
    if (local->dtype == AG_I8) return fail(AG_ERR_VALUE, "%s: the int8 payload cannot be sharded", who);
    const uint64_t n = local->num_nodes;
    if (is_cyclic(local)) {
        const uint64_t rows = n > rank ? (n - rank + world - 1) / world : 0;
        if (local->row_stride != world || local->row_begin != rank || local->rows != rows)
            return fail(AG_ERR_VALUE, "%s: rank %u of %u must hold rows %u, %u + %u, ... (%llu rows); the store holds %llu rows "
                        "from %llu with stride %llu", who, rank, world, rank, rank, world, (unsigned long long)rows,
                        (unsigned long long)local->rows, (unsigned long long)local->row_begin, (unsigned long long)local->row_stride);
        return AG_OK;
    }
    const uint64_t shard_rows = (n + world - 1) / world;
    const uint64_t begin = std::min<uint64_t>((uint64_t)rank * shard_rows, n), end = std::min<uint64_t>(begin + shard_rows, n);
    if (local->row_begin != begin || local->rows != end - begin)
        return fail(AG_ERR_VALUE, "%s: rank %u of %u must hold rows [%llu, %llu) of %llu, the store holds [%llu, %llu)", who,
                    rank, world, (unsigned long long)begin, (unsigned long long)end, (unsigned long long)n,
                    (unsigned long long)local->row_begin, (unsigned long long)(local->row_begin + local->rows));
    return AG_OK;
}

}  // namespace

extern "C" int32_t ag_features_ipc_export(const ag_features *f, void *handle_out) {
    if (!f || !handle_out) return fail(AG_ERR_VALUE, "ag_features_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64 && AG_IPC_HANDLE_BYTES >= 128, "IPC handle size");
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    memset(handle_out, 0, AG_IPC_HANDLE_BYTES);
    if (!f->payload || f->rows == 0) return AG_OK;  // an empty shard has nothing to map
    if (f->block) return peer_block_export(f->block, handle_out);
    cudaIpcMemHandle_t h;
    AG_CUDA(cudaIpcGetMemHandle(&h, f->payload));
    memcpy(handle_out, &h, sizeof(h));
    peer_handle_mark_legacy(handle_out);
    return AG_OK;
}

extern "C" int32_t ag_features_open_sharded(const ag_features *local, uint32_t world, uint32_t rank, const void *handles,
                                            ag_features **out) {
    if (!local || !handles || !out) return fail(AG_ERR_VALUE, "ag_features_open_sharded: null argument");
    AG_TRY(check_local(local, world, rank, "ag_features_open_sharded"));
    DeviceGuard guard(local->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint8_t *bases[8] = {nullptr};
    void *opened[8] = {nullptr};
    PeerBlock *blocks[8] = {nullptr};
    auto close_all = [&] {
        for (void *q : opened) if (q) cudaIpcCloseMemHandle(q);
        for (PeerBlock *b : blocks) if (b) peer_block_free(b);
    };
    const bool cyclic = is_cyclic(local) || (world > 1 && local->row_stride == world);
    const uint64_t n = local->num_nodes, shard_rows = (n + world - 1) / world;
    for (uint32_t r = 0; r < world; ++r) {
        if (r == rank) { bases[r] = local->payload; continue; }
        const bool empty = cyclic ? (uint64_t)r >= n : (uint64_t)r * shard_rows >= n;
        if (empty) continue;
        const uint8_t *handle = (const uint8_t *)handles + (size_t)r * AG_IPC_HANDLE_BYTES;
        const int kind = peer_handle_kind(handle);
        if (kind == 2) {
            const int32_t st = peer_block_import(handle, local->device, &blocks[r]);
            if (st != AG_OK) { close_all(); return st; }
            bases[r] = (const uint8_t *)peer_block_ptr(blocks[r]);
            continue;
        }
        if (kind != 1) { close_all(); return fail(AG_ERR_VALUE, "ag_features_open_sharded: rank %u's handle is empty or malformed", r); }
        cudaIpcMemHandle_t h;
        memcpy(&h, handle, sizeof(h));
        void *p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            close_all();
            return fail(AG_ERR_CUDA, "cannot map the feature shard of rank %u: %s", r, cudaGetErrorString(e));
        }
        opened[r] = p; bases[r] = (const uint8_t *)p;
    }
    const int32_t st = make_view(local, world, rank, cyclic, bases, opened, blocks, out);
    if (st != AG_OK) close_all();
    return st;
}

extern "C" int32_t ag_features_view_sharded(const ag_features *const *shards, uint32_t world, uint32_t rank,
                                            ag_features **out) {
    if (!shards || !out || world == 0 || world > 8 || rank >= world) return fail(AG_ERR_VALUE, "ag_features_view_sharded: bad argument");
    for (uint32_t r = 0; r < world; ++r) {
        if (!shards[r]) return fail(AG_ERR_VALUE, "ag_features_view_sharded: shard %u is null", r);
        if (shards[r]->num_nodes != shards[0]->num_nodes || shards[r]->dim != shards[0]->dim ||
            shards[r]->dtype != shards[0]->dtype || is_cyclic(shards[r]) != is_cyclic(shards[0]))
            return fail(AG_ERR_VALUE, "ag_features_view_sharded: shard %u disagrees on shape, dtype or layout", r);
        AG_TRY(check_local(shards[r], world, r, "ag_features_view_sharded"));
    }
    const ag_features *local = shards[rank];
    DeviceGuard guard(local->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint8_t *bases[8] = {nullptr};
    for (uint32_t r = 0; r < world; ++r) {
        bases[r] = shards[r]->payload;
        if (shards[r]->device == local->device || shards[r]->rows == 0) continue;
        if (shards[r]->block) { AG_TRY(peer_block_grant(shards[r]->block, local->device)); continue; }
        int can = 0;
        AG_CUDA(cudaDeviceCanAccessPeer(&can, local->device, shards[r]->device));
        if (!can) return fail(AG_ERR_CUDA, "GPU %d cannot access GPU %d's memory", local->device, shards[r]->device);
        const cudaError_t e = cudaDeviceEnablePeerAccess(shards[r]->device, 0);
        if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
        else if (e != cudaSuccess) return fail(AG_ERR_CUDA, "enabling peer access to GPU %d failed: %s", shards[r]->device, cudaGetErrorString(e));
    }
    return make_view(local, world, rank, is_cyclic(local), bases, nullptr, nullptr, out);
}

extern "C" int32_t ag_features_set_gather_order(ag_features *view, int32_t order) {
    if (!view) return fail(AG_ERR_VALUE, "ag_features_set_gather_order: null store");
    if (order < AG_GATHER_AUTO || order > AG_GATHER_DIRECT) return fail(AG_ERR_VALUE, "unknown gather order: %d", order);
    view->gather_order = order;
    return AG_OK;
}

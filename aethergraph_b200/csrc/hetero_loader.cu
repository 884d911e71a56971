// Prefetching loader for heterogeneous graphs: the worker / queue / ordering
// contract of the homogeneous loader (loader.cu; reference:
// crates/aethergraph-core/src/loader/prefetch.rs:984-1022 hetero workers,
// :1940-2060 HeteroNeighborLoader) over the heterogeneous sampler.
//
// Each worker thread owns one hetero sampler handle and one CUDA stream; it
// takes up to `group` queued batches and runs them as ONE launch chain
// (sample -> per-type dedup/relabel -> one feature gather per node type).
// Output buffers come from the loader's pool: one device allocation per batch,
// taken by the worker that runs the batch and recycled when the consumer
// releases it.  The feature rows reserved per
// node type follow the counts seen so far (1.5 x the largest + 1024) instead of
// the worst-case bound, which for wide fanouts is orders of magnitude larger;
// a batch that outgrows its reservation reports its true count and the caller
// gathers that type again.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "common.cuh"
#include "internal.h"

using namespace ag;

namespace {

struct HPoolSet {
    void *base = nullptr;
    ag_hetero_buffers bufs{};
    cudaEvent_t last_use = nullptr;
};

struct HWork {
    uint64_t seq = 0;
    int64_t batch_idx = 0;
    std::vector<uint32_t> seeds;
    ag_hetero_buffers bufs{};          // assigned by the worker that runs the batch
    cudaEvent_t after = nullptr;       // last use of recycled buffers
};

struct HDone {
    ag_hetero_batch batch{};
    int32_t status = AG_OK;
    std::string error;
};

using Clock = std::chrono::steady_clock;

uint64_t align256(uint64_t v) { return (v + 255) & ~255ull; }

}  // namespace

struct ag_hetero_loader {
    const ag_hetero_graph *g = nullptr;
    uint32_t nt = 0, ne = 0, seed_type = 0;
    uint64_t type_nodes[AG_MAX_NODE_TYPES] = {};
    const ag_features *feats[AG_MAX_NODE_TYPES] = {};
    bool has_feats = false;
    uint64_t seed = 0;
    bool seeded = true;
    uint32_t depth = 2, threads = 1, group = 1;
    int device = 0;

    std::mutex m;
    std::condition_variable cv_work, cv_space, cv_done, cv_room;
    std::deque<HWork> queue;
    std::map<uint64_t, HDone> ready;
    std::deque<uint64_t> arrival;
    uint64_t next_seq = 0, next_deliver = 0, in_ready = 0;
    bool stop = false;
    std::string fault;
    std::vector<std::thread> workers;
    std::vector<ag_hetero_sampler *> samplers;
    std::vector<cudaStream_t> streams;
    ag_loader_stats stats{};

    std::mutex pool_m;
    std::vector<HPoolSet> pool_free;
    std::unordered_map<void *, HPoolSet> pool_live;   // keyed by bufs.nodes
    uint64_t x_rows[AG_MAX_NODE_TYPES] = {};          // 0: nothing seen yet
    std::atomic<bool> x_seen{false};                  // some batch's counts have been observed
};

namespace {

// Rows of x to reserve for node type t in a batch bounded by cn nodes.
uint64_t want_x_rows(const ag_hetero_loader *l, uint32_t t, uint64_t cn) {
    uint64_t r = std::min<uint64_t>(cn, std::max<uint64_t>(l->type_nodes[t], 1));
    if (l->x_rows[t]) r = std::min<uint64_t>(r, l->x_rows[t]);
    return std::max<uint64_t>(r, 1);
}

void free_set(HPoolSet &p) {
    if (p.last_use) cudaEventDestroy(p.last_use);
    cudaFree(p.base);
}

int32_t pool_take(ag_hetero_loader *l, uint64_t n_seeds, ag_hetero_buffers *out, cudaEvent_t *last_use) {
    uint64_t mn = 0, me = 0;
    AG_TRY(ag_hetero_sampler_bounds(l->samplers[0], n_seeds, &mn, &me));
    const uint64_t cn = std::max<uint64_t>(mn, 1), ce = std::max<uint64_t>(me, 1), cs = std::max<uint64_t>(n_seeds, 1);
    uint64_t want[AG_MAX_NODE_TYPES] = {};
    *last_use = nullptr;
    {
        std::lock_guard<std::mutex> lk(l->pool_m);
        for (uint32_t t = 0; t < l->nt; ++t) want[t] = l->feats[t] ? want_x_rows(l, t, cn) : 0;
        for (size_t i = 0; i < l->pool_free.size();) {
            HPoolSet &p = l->pool_free[i];
            if (p.bufs.cap_nodes != cn || p.bufs.cap_edges != ce || p.bufs.cap_seeds != cs) { ++i; continue; }
            // A set made for an older estimate of the x rows: too small is useless, far
            // too large (the first batches reserve the worst case) wastes memory.
            bool fits = true, bloated = false;
            for (uint32_t t = 0; t < l->nt; ++t) {
                if (!want[t]) continue;
                if (p.bufs.cap_x[t] < want[t]) fits = false;
                if (p.bufs.cap_x[t] > 2 * want[t] + 4096) bloated = true;
            }
            if (fits && !bloated) {
                HPoolSet s = p;
                l->pool_free[i] = l->pool_free.back();
                l->pool_free.pop_back();
                *last_use = s.last_use;
                s.last_use = nullptr;
                *out = s.bufs;
                l->pool_live.emplace(s.bufs.nodes, s);
                return AG_OK;
            }
            free_set(p);
            l->pool_free[i] = l->pool_free.back();
            l->pool_free.pop_back();
        }
    }
    uint64_t off = 0;
    auto carve = [&](uint64_t bytes) { const uint64_t o = off; off += align256(bytes); return o; };
    const uint64_t o_nodes = carve(cn * 4), o_src = carve(ce * 4), o_dst = carve(ce * 4), o_seed = carve(cs * 4),
                   o_nid = carve(cn * 8), o_eil = carve(ce * 16), o_sidx = carve(cs * 8);
    uint64_t o_x[AG_MAX_NODE_TYPES] = {};
    for (uint32_t t = 0; t < l->nt; ++t)
        if (want[t]) o_x[t] = carve(want[t] * l->feats[t]->dim * 4);
    uint8_t *base = nullptr;
    if (cudaMalloc(&base, std::max<uint64_t>(off, 256)) != cudaSuccess)
        return fail(AG_ERR_CUDA, "hetero loader: out of device memory for a %llu-byte batch buffer: %s",
                    (unsigned long long)off, cudaGetErrorString(cudaGetLastError()));
    HPoolSet s;
    s.base = base;
    ag_hetero_buffers &b = s.bufs;
    b.cap_nodes = cn; b.cap_edges = ce; b.cap_seeds = cs;
    b.nodes = (uint32_t *)(base + o_nodes); b.edge_src_local = (uint32_t *)(base + o_src);
    b.edge_dst_local = (uint32_t *)(base + o_dst); b.seed_indices = (uint32_t *)(base + o_seed);
    b.n_id = (int64_t *)(base + o_nid); b.edge_index_local = (int64_t *)(base + o_eil);
    b.seed_index = (int64_t *)(base + o_sidx);
    for (uint32_t t = 0; t < l->nt; ++t)
        if (want[t]) { b.x[t] = (float *)(base + o_x[t]); b.cap_x[t] = want[t]; }
    *out = b;
    std::lock_guard<std::mutex> lk(l->pool_m);
    l->pool_live.emplace(b.nodes, s);
    return AG_OK;
}

void pool_give(ag_hetero_loader *l, const ag_hetero_buffers &bufs, bool record, cudaStream_t stream) {
    std::lock_guard<std::mutex> lk(l->pool_m);
    auto it = l->pool_live.find(bufs.nodes);
    if (it == l->pool_live.end()) return;
    HPoolSet s = it->second;
    l->pool_live.erase(it);
    if (record) {
        if (cudaEventCreateWithFlags(&s.last_use, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(s.last_use, stream) != cudaSuccess) {
            free_set(s);  // cannot order the reuse: do not reuse
            return;
        }
    }
    l->pool_free.push_back(s);
}

void drop_work(ag_hetero_loader *l, HWork &w) {
    if (w.after) { cudaEventDestroy(w.after); w.after = nullptr; }
    pool_give(l, w.bufs, false, nullptr);
}

void worker_main(ag_hetero_loader *l, uint32_t idx) {
    cudaSetDevice(l->device);
    ag_hetero_sampler *s = l->samplers[idx];
    cudaStream_t st = l->streams[idx];
    const uint32_t G = l->group;
    std::vector<HWork> ws;
    std::vector<const uint32_t *> seed_ptrs(G);
    std::vector<uint64_t> n_seeds(G), batch_seeds(G);
    std::vector<ag_hetero_buffers> bufs(G);
    std::vector<ag_hetero_counts> counts(G);
    std::vector<int32_t> statuses(G);
    for (;;) {
        ws.clear();
        {
            std::unique_lock<std::mutex> lk(l->m);
            l->cv_work.wait(lk, [&] { return l->stop || !l->queue.empty(); });
            if (l->stop) return;
            const size_t share = std::max<size_t>(1, (l->queue.size() + l->threads - 1) / l->threads);
            // a full group whenever one is queued: launch floors are paid per chain
            size_t take = l->queue.size() >= G ? G : std::min<size_t>(G, share);
            // Until a batch has been seen, x is reserved at the worst-case bound: one batch per chain.
            if (l->has_feats && !l->x_seen.load()) take = 1;
            while (ws.size() < take && !l->queue.empty()) {
                ws.push_back(std::move(l->queue.front()));
                l->queue.pop_front();
            }
            l->cv_space.notify_all();
        }
        const uint32_t nb = (uint32_t)ws.size();
        const auto t0 = Clock::now();
        int32_t rc = AG_OK;
        bool launched = false;
        for (uint32_t b = 0; b < nb; ++b) {
            HWork &w = ws[b];
            if (rc == AG_OK) rc = pool_take(l, w.seeds.size(), &w.bufs, &w.after);
            if (w.after) {
                if (cudaStreamWaitEvent(st, w.after, 0) != cudaSuccess) rc = fail(AG_ERR_CUDA, "cudaStreamWaitEvent failed");
                cudaEventDestroy(w.after);
                w.after = nullptr;
            }
            seed_ptrs[b] = w.seeds.data();
            n_seeds[b] = w.seeds.size();
            bufs[b] = w.bufs;
            batch_seeds[b] = ag_batch_seed(l->seed, w.seq);  // per-batch reseed (prefetch.rs:1003-1005)
            statuses[b] = AG_OK;
            counts[b] = ag_hetero_counts{};
        }
        std::string err;
        if (rc == AG_OK) {
            // Unseeded loaders have group 1: the worker's own stream continues.
            rc = ag_hetero_sample_group_into(s, nb, l->seed_type, seed_ptrs.data(), n_seeds.data(),
                                             l->seeded ? batch_seeds.data() : nullptr,
                                             l->has_feats ? l->feats : nullptr, bufs.data(), st);
            if (rc == AG_OK) { launched = true; rc = ag_hetero_sample_group_wait(s, counts.data(), statuses.data()); }
        }
        if (rc != AG_OK) err = ag_last_error();
        const uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(Clock::now() - t0).count();
        if (launched && l->has_feats) {
            std::lock_guard<std::mutex> pk(l->pool_m);
            for (uint32_t b = 0; b < nb; ++b)
                for (uint32_t t = 0; t < l->nt; ++t)
                    if (l->feats[t] && statuses[b] == AG_OK) {
                        // Grow in coarse steps (when the margin over the largest count falls
                        // under 25 %): every change of the estimate retires the pooled sets
                        // made for the old one.
                        const uint64_t n = counts[b].nodes[t];
                        if (n + n / 4 + 512 > l->x_rows[t]) l->x_rows[t] = n + n / 2 + 1024;
                    }
            l->x_seen.store(true);
        }
        std::unique_lock<std::mutex> lk(l->m);
        for (uint32_t b = 0; b < nb; ++b) {
            HWork &w = ws[b];
            HDone d;
            d.batch.batch_idx = w.batch_idx; d.batch.seq = w.seq; d.batch.bufs = w.bufs; d.batch.counts = counts[b];
            // A chain that was never launched, or that failed as a whole, fails every batch
            // of the group; a per-batch error fails only that batch.
            const bool chain_failed = rc != AG_OK && statuses[b] == AG_OK &&
                                      (!launched || !(rc == AG_ERR_SAMPLING || rc == AG_ERR_VALUE));
            if (statuses[b] != AG_OK || chain_failed) { d.status = statuses[b] != AG_OK ? statuses[b] : rc; d.error = err; }
            l->cv_room.wait(lk, [&] { return l->stop || l->in_ready < l->depth || w.seq == l->next_deliver; });
            if (l->stop) {
                lk.unlock();
                for (uint32_t r = b; r < nb; ++r) drop_work(l, ws[r]);
                return;
            }
            if (b == 0) { l->stats.sample_time_ns += ns; l->stats.chains += 1; }
            if (d.status != AG_OK && l->fault.empty() && d.status != AG_ERR_SAMPLING && d.status != AG_ERR_VALUE)
                l->fault = d.error;
            l->ready.emplace(w.seq, std::move(d));
            l->arrival.push_back(w.seq);
            l->in_ready++;
            l->cv_done.notify_all();
        }
    }
}

bool has_deliverable(ag_hetero_loader *l) {
    if (l->seeded) return l->ready.count(l->next_deliver) != 0;
    return !l->arrival.empty();
}

// Caller holds l->m and has_deliverable(l) is true.
int32_t deliver(ag_hetero_loader *l, ag_hetero_batch *out, bool waited) {
    auto it = l->seeded ? l->ready.find(l->next_deliver) : l->ready.find(l->arrival.front());
    HDone d = std::move(it->second);
    const uint64_t seq = it->first;
    l->ready.erase(it);
    for (auto a = l->arrival.begin(); a != l->arrival.end(); ++a)
        if (*a == seq) { l->arrival.erase(a); break; }
    if (l->seeded) l->next_deliver++;
    l->in_ready--;
    l->cv_room.notify_all();
    l->stats.total++;
    (waited ? l->stats.misses : l->stats.hits)++;
    if (d.status != AG_OK) {
        pool_give(l, d.batch.bufs, false, nullptr);
        set_error("%s", d.error.c_str());
        return d.status;
    }
    l->stats.edges += d.batch.counts.total_edges;
    l->stats.nodes += d.batch.counts.total_nodes;
    *out = d.batch;
    return AG_OK;
}

int32_t wait_deliverable(ag_hetero_loader *l, std::unique_lock<std::mutex> &lk, int64_t timeout_ms, bool *waited) {
    const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 30000 : timeout_ms);
    while (!has_deliverable(l)) {
        if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
        if (!l->fault.empty()) return fail(AG_ERR_WORKER, "sampler worker failed: %s", l->fault.c_str());
        *waited = true;
        if (l->cv_done.wait_until(lk, deadline) == std::cv_status::timeout && !has_deliverable(l)) {
            if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
            return fail(AG_ERR_TIMEOUT, "timed out waiting for a sampled batch");
        }
    }
    return AG_OK;
}

}  // namespace

extern "C" int32_t ag_hetero_loader_create(const ag_hetero_graph *g, uint32_t seed_type, const uint32_t *fanout,
                                           uint32_t num_hops, int32_t replace, uint64_t seed, int32_t rng_mode,
                                           int32_t seeded, const ag_features *const *feats, uint32_t prefetch_depth,
                                           uint32_t sampler_threads, uint32_t group, ag_hetero_loader **out) {
    if (!g || !fanout || !out) return fail(AG_ERR_VALUE, "ag_hetero_loader_create: null argument");
    if (group == 0) group = 1;
    if (group > 64) return fail(AG_ERR_VALUE, "group must be <= 64");
    if (prefetch_depth == 0) return fail(AG_ERR_VALUE, "prefetch_depth must be >= 1");
    if (sampler_threads == 0 || sampler_threads > 64) return fail(AG_ERR_VALUE, "sampler_threads must be in 1..64");
    ag_hetero_loader *l = new ag_hetero_loader();
    int32_t st = ag_hetero_info(g, &l->nt, &l->ne, l->type_nodes, nullptr, &l->device);
    if (st == AG_OK && seed_type >= l->nt) st = fail(AG_ERR_SAMPLING, "unknown seed node type %u", seed_type);
    if (st != AG_OK) { delete l; return st; }
    l->g = g; l->seed_type = seed_type; l->seed = seed; l->seeded = seeded != 0;
    l->depth = prefetch_depth; l->threads = sampler_threads; l->group = seeded ? group : 1;
    if (feats)
        for (uint32_t t = 0; t < l->nt; ++t)
            if (feats[t]) {
                if (feats[t]->device != l->device) { delete l; return fail(AG_ERR_VALUE, "feature store of node type %u lives on another device", t); }
                l->feats[t] = feats[t];
                l->has_feats = true;
            }
    DeviceGuard guard(l->device);
    if (!guard.ok) { delete l; return AG_ERR_CUDA; }
    for (uint32_t i = 0; i < sampler_threads && st == AG_OK; ++i) {
        ag_hetero_sampler *s = nullptr;
        // Unseeded workers must not replay one another (the reference seeds each from entropy).
        const uint64_t worker_seed = l->seeded ? seed : ag_batch_seed(seed, 0x5eed0000ull + i);
        st = ag_hetero_sampler_create_group(g, fanout, num_hops, replace, worker_seed, rng_mode, l->group, &s);
        if (st != AG_OK) break;
        l->samplers.push_back(s);
        cudaStream_t stream = nullptr;
        if (cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking) != cudaSuccess)
            st = fail(AG_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(cudaGetLastError()));
        else
            l->streams.push_back(stream);
    }
    if (st != AG_OK) {
        for (ag_hetero_sampler *s : l->samplers) ag_hetero_sampler_free(s);
        for (cudaStream_t s : l->streams) cudaStreamDestroy(s);
        delete l;
        return st;
    }
    for (uint32_t i = 0; i < sampler_threads; ++i) l->workers.emplace_back(worker_main, l, i);
    *out = l;
    return AG_OK;
}

extern "C" int32_t ag_hetero_loader_submit(ag_hetero_loader *l, int64_t batch_idx, const uint32_t *seeds, uint64_t n_seeds) {
    if (!l) return fail(AG_ERR_VALUE, "ag_hetero_loader_submit: null loader");
    if (!seeds && n_seeds) return fail(AG_ERR_VALUE, "ag_hetero_loader_submit: null seeds");
    // Range-check where seeds enter (hetero_sampler.rs:174-187).
    for (uint64_t i = 0; i < n_seeds; ++i)
        if ((uint64_t)seeds[i] >= l->type_nodes[l->seed_type])
            return fail(AG_ERR_SAMPLING, "seed node %u (position %llu) is out of range for %llu nodes", seeds[i],
                        (unsigned long long)i, (unsigned long long)l->type_nodes[l->seed_type]);
    DeviceGuard guard(l->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint64_t mn = 0, me = 0;
    AG_TRY(ag_hetero_sampler_bounds(l->samplers[0], n_seeds, &mn, &me));  // refuses a batch past the per-batch limits
    HWork w;
    w.batch_idx = batch_idx;
    w.seeds.assign(seeds, seeds + n_seeds);
    std::unique_lock<std::mutex> lk(l->m);
    const bool room = l->cv_space.wait_for(lk, std::chrono::seconds(30), [&] {
        return l->stop || !l->fault.empty() || l->queue.size() < (size_t)8 * l->depth;
    });
    int32_t rc = AG_OK;
    if (!room) rc = fail(AG_ERR_TIMEOUT, "timed out waiting for room in the work queue (%u batches queued; is anything "
                         "consuming results?)", 8 * l->depth);
    else if (l->stop) rc = fail(AG_ERR_SHUTDOWN, "loader is shut down");
    else if (!l->fault.empty()) rc = fail(AG_ERR_WORKER, "sampler worker failed: %s", l->fault.c_str());
    if (rc != AG_OK) return rc;
    w.seq = l->next_seq++;
    l->stats.submitted++;
    l->queue.push_back(std::move(w));
    lk.unlock();
    l->cv_work.notify_one();
    return AG_OK;
}

extern "C" int32_t ag_hetero_loader_next(ag_hetero_loader *l, int64_t timeout_ms, ag_hetero_batch *out) {
    if (!l || !out) return fail(AG_ERR_VALUE, "ag_hetero_loader_next: null argument");
    std::unique_lock<std::mutex> lk(l->m);
    bool waited = false;
    AG_TRY(wait_deliverable(l, lk, timeout_ms, &waited));
    return deliver(l, out, waited);
}

// Like ag_loader_next_many: waits for the first batch, then also hands over every
// further batch that is already deliverable, up to max_n; a failed batch ends the
// call and is reported by the next one.
extern "C" int32_t ag_hetero_loader_next_many(ag_hetero_loader *l, int64_t timeout_ms, uint32_t max_n,
                                              ag_hetero_batch *out, uint32_t *n_out) {
    if (!l || !out || !n_out || max_n == 0) return fail(AG_ERR_VALUE, "ag_hetero_loader_next_many: bad argument");
    *n_out = 0;
    std::unique_lock<std::mutex> lk(l->m);
    bool waited = false;
    AG_TRY(wait_deliverable(l, lk, timeout_ms, &waited));
    while (*n_out < max_n && has_deliverable(l)) {
        const auto it = l->seeded ? l->ready.find(l->next_deliver) : l->ready.find(l->arrival.front());
        if (it->second.status != AG_OK && *n_out > 0) break;
        const int32_t rc = deliver(l, &out[*n_out], waited && *n_out == 0);
        if (rc != AG_OK) return rc;
        ++*n_out;
    }
    return AG_OK;
}

extern "C" int32_t ag_hetero_loader_release_batch(ag_hetero_loader *l, ag_hetero_batch *batch, void *stream) {
    if (!l || !batch) return fail(AG_ERR_VALUE, "ag_hetero_loader_release_batch: null argument");
    if (batch->bufs.nodes) {
        DeviceGuard guard(l->device);
        pool_give(l, batch->bufs, true, (cudaStream_t)stream);
        batch->bufs = ag_hetero_buffers{};
    }
    return AG_OK;
}

extern "C" int32_t ag_hetero_loader_stats_get(const ag_hetero_loader *l, ag_loader_stats *stats) {
    if (!l || !stats) return fail(AG_ERR_VALUE, "ag_hetero_loader_stats_get: null argument");
    std::unique_lock<std::mutex> lk(const_cast<ag_hetero_loader *>(l)->m);
    *stats = l->stats;
    return AG_OK;
}

extern "C" int32_t ag_hetero_loader_shutdown(ag_hetero_loader *l) {
    if (!l) return fail(AG_ERR_VALUE, "ag_hetero_loader_shutdown: null loader");
    {
        std::unique_lock<std::mutex> lk(l->m);
        l->stop = true;
    }
    l->cv_work.notify_all(); l->cv_space.notify_all(); l->cv_done.notify_all(); l->cv_room.notify_all();
    return AG_OK;
}

extern "C" void ag_hetero_loader_free(ag_hetero_loader *l) {
    if (!l) return;
    ag_hetero_loader_shutdown(l);
    for (std::thread &t : l->workers) if (t.joinable()) t.join();
    DeviceGuard guard(l->device);
    cudaDeviceSynchronize();
    for (HWork &w : l->queue) drop_work(l, w);
    for (auto &kv : l->ready) pool_give(l, kv.second.batch.bufs, false, nullptr);
    for (ag_hetero_sampler *s : l->samplers) ag_hetero_sampler_free(s);
    for (cudaStream_t s : l->streams) cudaStreamDestroy(s);
    // Batches still held by a consumer keep their memory valid until now.
    for (HPoolSet &p : l->pool_free) free_set(p);
    for (auto &kv : l->pool_live) cudaFree(kv.second.base);
    delete l;
}

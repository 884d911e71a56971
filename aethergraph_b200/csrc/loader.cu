// Prefetching loader: host threads that keep several batches in flight on the
// GPU, with the ordering, reseeding, back-pressure, shutdown and error
// contract of the reference pipeline
// (crates/aethergraph-core/src/loader/prefetch.rs:402-560, 911-1073).
//
// Each worker thread owns one sampler handle and one CUDA stream.  A batch is
// one launch chain (sample -> dedup/relabel -> gather) on the worker's stream;
// with T workers, T chains overlap on the device, which is what hides the
// latency-bound sampling kernels behind the bandwidth-bound gather.
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"
#include "internal.h"

using namespace ag;

namespace {

struct Work {
    uint64_t seq = 0;
    int64_t batch_idx = 0;
    std::vector<uint32_t> seeds;       // host copy (AG_MEM_HOST submissions)
    const uint32_t *seeds_dev = nullptr;
    uint64_t n_seeds = 0;
    ag_subgraph_buffers bufs{};
    bool owned = false;
    cudaEvent_t after = nullptr;       // work the buffers' previous user still has queued
};

struct Done {
    ag_batch batch{};
    int32_t status = AG_OK;
    std::string error;
};

using Clock = std::chrono::steady_clock;

}  // namespace

struct ag_loader {
    const ag_graph *g = nullptr;
    const ag_features *f = nullptr;
    ag_sampling_config cfg{};
    bool seeded = true, profiling = false;
    uint32_t depth = 2, threads = 1, group = 1;
    int device = 0;

    std::mutex m;
    std::condition_variable cv_work, cv_space, cv_done, cv_room;
    std::deque<Work> queue;              // bounded: 8 x depth (prefetch.rs:1135-1143)
    std::map<uint64_t, Done> ready;      // finished batches keyed by seq
    std::deque<uint64_t> arrival;        // completion order, for unseeded delivery
    uint64_t next_seq = 0, next_deliver = 0, in_ready = 0;
    bool stop = false;
    std::string fault;                   // first worker failure
    std::vector<std::thread> workers;
    std::vector<ag_sampler *> samplers;
    std::vector<cudaStream_t> streams;
    ag_loader_stats stats{};
};

namespace {

int32_t alloc_owned(ag_loader *l, uint64_t n_seeds, ag_subgraph_buffers *b) {
    uint64_t mn = 0, me = 0;
    AG_TRY(ag_sampler_bounds(l->samplers[0], n_seeds, &mn, &me));
    *b = ag_subgraph_buffers{};
    b->cap_nodes = std::max<uint64_t>(mn, 1); b->cap_edges = std::max<uint64_t>(me, 1);
    b->cap_seeds = std::max<uint64_t>(n_seeds, 1);
    bool ok = cudaMalloc(&b->nodes, b->cap_nodes * 4) == cudaSuccess &&
              cudaMalloc(&b->edge_src, b->cap_edges * 4) == cudaSuccess &&
              cudaMalloc(&b->edge_dst, b->cap_edges * 4) == cudaSuccess &&
              cudaMalloc(&b->src_local, b->cap_edges * 4) == cudaSuccess &&
              cudaMalloc(&b->dst_local, b->cap_edges * 4) == cudaSuccess &&
              cudaMalloc(&b->seed_locals, b->cap_seeds * 4) == cudaSuccess;
    if (ok && l->cfg.track_edge_ids) ok = cudaMalloc(&b->edge_ids, b->cap_edges * 8) == cudaSuccess;
    if (ok && l->f) ok = cudaMalloc(&b->x, b->cap_nodes * l->f->dim * 4) == cudaSuccess;
    if (!ok) return fail(AG_ERR_CUDA, "loader: out of device memory: %s", cudaGetErrorString(cudaGetLastError()));
    return AG_OK;
}

void free_owned(ag_subgraph_buffers *b) {
    void *ptrs[] = {b->nodes, b->edge_src, b->edge_dst, b->edge_ids, b->src_local, b->dst_local,
                    b->seed_locals, b->n_id, b->edge_index_local, b->e_id, b->seed_index, b->x};
    for (void *p : ptrs) cudaFree(p);
    *b = ag_subgraph_buffers{};
}

void worker_main(ag_loader *l, uint32_t idx) {
    cudaSetDevice(l->device);
    ag_sampler *s = l->samplers[idx];
    cudaStream_t st = l->streams[idx];
    const uint32_t G = l->group;
    std::vector<Work> ws;
    std::vector<const uint32_t *> seed_ptrs(G);
    std::vector<uint64_t> n_seeds(G), batch_seeds(G);
    std::vector<ag_subgraph_buffers> bufs(G);
    std::vector<ag_sample_counts> counts(G);
    std::vector<int32_t> statuses(G);
    for (;;) {
        ws.clear();
        {
            std::unique_lock<std::mutex> lk(l->m);
            l->cv_work.wait(lk, [&] { return l->stop || !l->queue.empty(); });
            if (l->stop) return;
            // Take a fair share of what is queued, up to one group: the batches of
            // a group ride one launch chain, so a deep queue costs few launches,
            // while a shallow one is still spread over the workers.  A group is
            // homogeneous in where its seeds live.
            const size_t share = std::max<size_t>(1, (l->queue.size() + l->threads - 1) / l->threads);
            const size_t take = std::min<size_t>(G, share);
            const bool dev_seeds = l->queue.front().seeds_dev != nullptr;
            while (ws.size() < take && !l->queue.empty() && (l->queue.front().seeds_dev != nullptr) == dev_seeds) {
                ws.push_back(std::move(l->queue.front()));
                l->queue.pop_front();
            }
            l->cv_space.notify_all();
        }
        const uint32_t nb = (uint32_t)ws.size();
        const auto t0 = Clock::now();
        int32_t rc = AG_OK;
        for (uint32_t b = 0; b < nb; ++b) {
            Work &w = ws[b];
            if (w.after) {
                if (cudaStreamWaitEvent(st, w.after, 0) != cudaSuccess) rc = fail(AG_ERR_CUDA, "cudaStreamWaitEvent failed");
                cudaEventDestroy(w.after);
                w.after = nullptr;
            }
            seed_ptrs[b] = w.seeds_dev ? w.seeds_dev : w.seeds.data();
            n_seeds[b] = w.n_seeds;
            bufs[b] = w.bufs;
            // Seeded loaders restart the stream per batch from its submission number
            // (prefetch.rs:926-930), so any pool size or grouping yields the same results.
            batch_seeds[b] = ag_batch_seed(l->cfg.seed, w.seq);
            statuses[b] = AG_OK;
        }
        // Unseeded: a worker's own stream continues across its batches, which needs
        // the batches one at a time.
        std::string err;
        if (rc == AG_OK && (l->seeded || nb == 1)) {
            rc = ag_sample_group_into(s, nb, seed_ptrs.data(), n_seeds.data(),
                                      ws[0].seeds_dev ? AG_MEM_DEVICE : AG_MEM_HOST,
                                      l->seeded ? batch_seeds.data() : nullptr, l->f, bufs.data(), st);
            if (rc == AG_OK) rc = ag_sample_group_wait(s, counts.data(), statuses.data());
            if (rc != AG_OK) err = ag_last_error();
        } else if (rc == AG_OK) {
            for (uint32_t b = 0; b < nb; ++b) {
                int32_t r1 = ag_sample_group_into(s, 1, &seed_ptrs[b], &n_seeds[b],
                                                  ws[b].seeds_dev ? AG_MEM_DEVICE : AG_MEM_HOST, nullptr, l->f,
                                                  &bufs[b], st);
                if (r1 == AG_OK) r1 = ag_sample_group_wait(s, &counts[b], &statuses[b]);
                if (r1 != AG_OK) { statuses[b] = r1; rc = r1; err = ag_last_error(); }
            }
        } else {
            err = ag_last_error();
        }
        const uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(Clock::now() - t0).count();
        for (uint32_t b = 0; b < nb; ++b) {
            Work &w = ws[b];
            Done d;
            d.batch.batch_idx = w.batch_idx; d.batch.seq = w.seq; d.batch.bufs = w.bufs; d.batch.owned = w.owned ? 1 : 0;
            d.batch.counts = counts[b];
            // A failure of the whole launch chain fails every batch of the group; a
            // per-batch error (bad seed, small buffer) fails only that batch.
            const bool chain_failed = rc != AG_OK && statuses[b] == AG_OK &&
                                      !(rc == AG_ERR_SAMPLING || rc == AG_ERR_VALUE || rc == AG_ERR_LOAD);
            if (statuses[b] != AG_OK || chain_failed) { d.status = statuses[b] != AG_OK ? statuses[b] : rc; d.error = err; }
            std::unique_lock<std::mutex> lk(l->m);
            // Results channel holds `depth` batches: wait for room (prefetch.rs:1135-1143),
            // except for the batch the consumer is waiting on — holding it back could
            // stall an ordered loader whose later batches filled the channel first.
            l->cv_room.wait(lk, [&] { return l->stop || l->in_ready < l->depth || w.seq == l->next_deliver; });
            if (l->stop) { for (uint32_t r = b; r < nb; ++r) if (ws[r].owned) free_owned(&ws[r].bufs); return; }
            if (b == 0) l->stats.sample_time_ns += ns;
            if (d.status != AG_OK && l->fault.empty() && d.status != AG_ERR_SAMPLING && d.status != AG_ERR_VALUE)
                l->fault = d.error;  // a broken worker poisons the loader; a bad batch does not
            l->ready.emplace(w.seq, std::move(d));
            l->arrival.push_back(w.seq);
            l->in_ready++;
            l->cv_done.notify_all();
        }
    }
}

int32_t deliver(ag_loader *l, std::unique_lock<std::mutex> &lk, ag_batch *out, bool waited) {
    std::map<uint64_t, Done>::iterator it;
    if (l->seeded) {
        it = l->ready.find(l->next_deliver);
    } else {
        it = l->ready.find(l->arrival.front());
    }
    Done d = std::move(it->second);
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
        if (d.batch.owned) free_owned(&d.batch.bufs);
        set_error("%s", d.error.c_str());
        return d.status;
    }
    l->stats.edges += d.batch.counts.num_edges;
    l->stats.nodes += d.batch.counts.num_nodes;
    l->stats.gather_ms += d.batch.counts.gather_ms;
    l->stats.sample_ms += d.batch.counts.sample_ms;
    *out = d.batch;
    return AG_OK;
}

bool has_deliverable(ag_loader *l) {
    if (l->seeded) return l->ready.count(l->next_deliver) != 0;
    return !l->arrival.empty();
}

}  // namespace

extern "C" int32_t ag_loader_create(const ag_graph *g, const ag_features *f, const ag_sampling_config *cfg,
                                    int32_t seeded, uint32_t prefetch_depth, uint32_t sampler_threads,
                                    uint32_t group, int32_t profiling, ag_loader **out) {
    if (!g || !cfg || !out) return fail(AG_ERR_VALUE, "ag_loader_create: null argument");
    if (group == 0) group = 1;
    if (group > 256) return fail(AG_ERR_VALUE, "group must be <= 256");
    if (prefetch_depth == 0) return fail(AG_ERR_VALUE, "prefetch_depth must be >= 1");
    if (sampler_threads == 0) return fail(AG_ERR_VALUE, "sampler_threads must be >= 1");
    if (sampler_threads > 64) return fail(AG_ERR_VALUE, "sampler_threads must be <= 64");
    if (f && f->device != g->device) return fail(AG_ERR_VALUE, "graph and feature store live on different devices");
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_loader *l = new ag_loader();
    l->g = g; l->f = f; l->cfg = *cfg; l->seeded = seeded != 0; l->profiling = profiling != 0;
    l->depth = prefetch_depth; l->threads = sampler_threads; l->device = g->device;
    l->group = seeded ? group : 1;
    int32_t st = AG_OK;
    for (uint32_t i = 0; i < sampler_threads && st == AG_OK; ++i) {
        ag_sampler *s = nullptr;
        ag_sampling_config c = *cfg;
        // Unseeded workers must not replay one another (the reference seeds each from entropy).
        if (!l->seeded) c.seed = ag_batch_seed(cfg->seed, 0x5eed0000ull + i);
        st = ag_sampler_create_group(g, &c, l->group, &s);
        if (st != AG_OK) break;
        l->samplers.push_back(s);
        if (profiling) st = ag_sampler_set_profiling(s, 1);
        cudaStream_t stream = nullptr;
        // Sampling chains run at the highest priority; each handle's gather runs on
        // its own lowest-priority stream, so chains of other workers cut in.
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        if (st == AG_OK && cudaStreamCreateWithPriority(&stream, cudaStreamNonBlocking, hi) != cudaSuccess)
            st = fail(AG_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(cudaGetLastError()));
        if (st == AG_OK) l->streams.push_back(stream);
    }
    if (st != AG_OK) {
        for (ag_sampler *s : l->samplers) ag_sampler_free(s);
        for (cudaStream_t s : l->streams) cudaStreamDestroy(s);
        delete l;
        return st;
    }
    for (uint32_t i = 0; i < sampler_threads; ++i) l->workers.emplace_back(worker_main, l, i);
    *out = l;
    return AG_OK;
}

extern "C" int32_t ag_loader_bounds(const ag_loader *l, uint64_t n_seeds, uint64_t *max_nodes, uint64_t *max_edges) {
    if (!l) return fail(AG_ERR_VALUE, "ag_loader_bounds: null loader");
    return ag_sampler_bounds(l->samplers[0], n_seeds, max_nodes, max_edges);
}

extern "C" int32_t ag_loader_submit(ag_loader *l, int64_t batch_idx, const uint32_t *seeds, uint64_t n_seeds,
                                    int32_t seeds_mem, const ag_subgraph_buffers *bufs, void *after_stream) {
    if (!l || (!seeds && n_seeds)) return fail(AG_ERR_VALUE, "ag_loader_submit: null argument");
    // Range-check where seeds enter (Seeds::new, sampler.rs:230-239; prefetch.rs:389-397 of the bindings).
    if (seeds_mem == AG_MEM_HOST)
        for (uint64_t i = 0; i < n_seeds; ++i)
            if ((uint64_t)seeds[i] >= l->g->num_nodes)
                return fail(AG_ERR_SAMPLING, "seed node %u (position %llu) is out of range for %llu nodes",
                            seeds[i], (unsigned long long)i, (unsigned long long)l->g->num_nodes);
    Work w;
    w.batch_idx = batch_idx; w.n_seeds = n_seeds;
    if (seeds_mem == AG_MEM_HOST) w.seeds.assign(seeds, seeds + n_seeds); else w.seeds_dev = seeds;
    DeviceGuard guard(l->device);
    if (!guard.ok) return AG_ERR_CUDA;
    if (bufs) w.bufs = *bufs;
    else { AG_TRY(alloc_owned(l, n_seeds, &w.bufs)); w.owned = true; }
    if (after_stream || bufs) {
        // Order the batch's kernels after whatever the caller's stream has queued.
        if (cudaEventCreateWithFlags(&w.after, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(w.after, (cudaStream_t)after_stream) != cudaSuccess) {
            if (w.owned) free_owned(&w.bufs);
            return fail(AG_ERR_CUDA, "loader: event record failed: %s", cudaGetErrorString(cudaGetLastError()));
        }
    }
    std::unique_lock<std::mutex> lk(l->m);
    // Blocks while the work queue is full, like the reference's bounded channel; gives
    // up after the same 30 s the consumer side waits, so a caller that submits and
    // consumes on one thread and overfills the queue gets an error, not a hang.
    const bool room = l->cv_space.wait_for(lk, std::chrono::seconds(30), [&] {
        return l->stop || !l->fault.empty() || l->queue.size() < (size_t)8 * l->depth;
    });
    if (!room) {
        lk.unlock();
        if (w.after) cudaEventDestroy(w.after);
        if (w.owned) free_owned(&w.bufs);
        return fail(AG_ERR_TIMEOUT, "timed out waiting for room in the work queue (%u batches queued; is anything "
                    "consuming results?)", 8 * l->depth);
    }
    if (l->stop || !l->fault.empty()) {
        const std::string msg = l->stop ? "loader is shut down" : ("sampler worker failed: " + l->fault);
        const int32_t code = l->stop ? AG_ERR_SHUTDOWN : AG_ERR_WORKER;
        lk.unlock();
        if (w.after) cudaEventDestroy(w.after);
        if (w.owned) free_owned(&w.bufs);
        return fail(code, "%s", msg.c_str());
    }
    w.seq = l->next_seq++;
    l->stats.submitted++;
    l->queue.push_back(std::move(w));
    l->cv_work.notify_one();
    return AG_OK;
}

extern "C" int32_t ag_loader_next(ag_loader *l, int64_t timeout_ms, ag_batch *out) {
    if (!l || !out) return fail(AG_ERR_VALUE, "ag_loader_next: null argument");
    std::unique_lock<std::mutex> lk(l->m);
    bool waited = false;
    const auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms < 0 ? 30000 : timeout_ms);
    while (!has_deliverable(l)) {
        if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
        if (!l->fault.empty()) return fail(AG_ERR_WORKER, "sampler worker failed: %s", l->fault.c_str());
        waited = true;
        if (l->cv_done.wait_until(lk, deadline) == std::cv_status::timeout && !has_deliverable(l)) {
            if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
            return fail(AG_ERR_TIMEOUT, "timed out waiting for a sampled batch");
        }
    }
    return deliver(l, lk, out, waited);
}

extern "C" int32_t ag_loader_try_next(ag_loader *l, ag_batch *out) {
    if (!l || !out) return fail(AG_ERR_VALUE, "ag_loader_try_next: null argument");
    std::unique_lock<std::mutex> lk(l->m);
    if (!has_deliverable(l)) {
        if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
        if (!l->fault.empty()) return fail(AG_ERR_WORKER, "sampler worker failed: %s", l->fault.c_str());
        return fail(AG_ERR_TIMEOUT, "no batch is ready");
    }
    return deliver(l, lk, out, false);
}

extern "C" int32_t ag_loader_release_batch(ag_loader *l, ag_batch *batch) {
    if (!l || !batch) return fail(AG_ERR_VALUE, "ag_loader_release_batch: null argument");
    if (batch->owned) {
        DeviceGuard guard(l->device);
        free_owned(&batch->bufs);
        batch->owned = 0;
    }
    return AG_OK;
}

extern "C" int32_t ag_loader_stats_get(const ag_loader *l, ag_loader_stats *stats) {
    if (!l || !stats) return fail(AG_ERR_VALUE, "ag_loader_stats_get: null argument");
    std::unique_lock<std::mutex> lk(const_cast<ag_loader *>(l)->m);
    *stats = l->stats;
    return AG_OK;
}

extern "C" int32_t ag_loader_shutdown(ag_loader *l) {
    if (!l) return fail(AG_ERR_VALUE, "ag_loader_shutdown: null loader");
    {
        std::unique_lock<std::mutex> lk(l->m);
        l->stop = true;  // wakes submitters, consumers and workers (prefetch.rs:250-313)
    }
    l->cv_work.notify_all(); l->cv_space.notify_all(); l->cv_done.notify_all(); l->cv_room.notify_all();
    return AG_OK;
}

extern "C" void ag_loader_free(ag_loader *l) {
    if (!l) return;
    ag_loader_shutdown(l);
    for (std::thread &t : l->workers) if (t.joinable()) t.join();
    DeviceGuard guard(l->device);
    for (Work &w : l->queue) { if (w.after) cudaEventDestroy(w.after); if (w.owned) free_owned(&w.bufs); }
    for (auto &kv : l->ready) if (kv.second.batch.owned) free_owned(&kv.second.batch.bufs);
    for (ag_sampler *s : l->samplers) ag_sampler_free(s);
    for (cudaStream_t s : l->streams) cudaStreamDestroy(s);
    delete l;
}

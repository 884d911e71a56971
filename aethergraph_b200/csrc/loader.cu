// Prefetching loader: host threads that keep several batches in flight on the
// GPU, with the ordering, reseeding, back-pressure, shutdown and error
// contract of the reference pipeline
// (crates/aethergraph-core/src/loader/prefetch.rs:402-560, 911-1073).
//
// Each worker thread owns one sampler handle and one high-priority CUDA stream.
// A worker takes up to `group` queued batches at a time and runs them as ONE
// launch chain (sample -> dedup/relabel -> gather); with T workers, T chains
// overlap on the device, which is what hides the latency-bound sampling kernels
// behind the bandwidth-bound gather.
//
// Output buffers either come with the submission (caller-owned) or from the
// loader's pool: one device allocation per batch shape, recycled when the
// consumer releases the batch.  A recycled set remembers the event that marks
// the consumer's last use, and the next batch's kernels wait for it.
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
// AG_LOADER_SPIN_WAIT=1 keeps the runtime's spinning waits (A/B measurements).
bool yielding_waits() {
    static const bool on = [] { const char *v = getenv("AG_LOADER_SPIN_WAIT"); return !(v && v[0] == '1'); }();
    return on;
}
}  // namespace

namespace {

struct PoolSet {
    void *base = nullptr;              // one cudaMalloc: every array but x
    void *x_base = nullptr;            // x on its own, so that a batch that outgrew it can get a larger one
    ag_subgraph_buffers bufs{};
    cudaEvent_t last_use = nullptr;    // consumer's last use of the memory, if any
};

struct Work {
    uint64_t seq = 0;
    int64_t batch_idx = 0;
    std::vector<uint32_t> seeds;       // host copy (AG_MEM_HOST submissions)
    const uint32_t *seeds_dev = nullptr;
    uint64_t n_seeds = 0;
    ag_subgraph_buffers bufs{};
    bool owned = false;
    cudaEvent_t after[2] = {nullptr, nullptr};  // work that must finish before the buffers are written
};

struct Done {
    ag_batch batch{};
    int32_t status = AG_OK;
    std::string error;
};

using Clock = std::chrono::steady_clock;

uint64_t align256(uint64_t v) { return (v + 255) & ~255ull; }

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
    // Batch number seq draws from ag_batch_seed(cfg.seed, seed_base + seed_stride * seq):
    // rank r of a W-rank job sets (r, W), so global batch b is sampled from the same
    // stream whatever W is.  Atomic: workers read them without the queue lock.
    std::atomic<uint64_t> seed_base{0}, seed_stride{1};
    bool stop = false;
    std::string fault;                   // first worker failure
    std::vector<std::thread> workers;
    std::vector<ag_sampler *> samplers;
    std::vector<cudaStream_t> streams;
    ag_loader_stats stats{};

    // x of a pooled batch is reserved from the node counts batches really produce (the
    // worst-case bound, every pick a new vertex, is several times larger): 1.5 x the
    // largest batch seen, in steps of 4096 rows, full size until a batch has been seen.
    std::atomic<uint64_t> x_rows_seen{0};
    std::mutex pool_m;
    std::vector<PoolSet> pool_free;
    std::unordered_map<void *, PoolSet> pool_live;  // keyed by bufs.nodes
};

namespace {

// A buffer set for a batch of n_seeds seeds, from the pool or freshly allocated.
// *last_use receives the event the next writer has to wait for (may be null).
int32_t pool_take(ag_loader *l, uint64_t n_seeds, ag_subgraph_buffers *out, cudaEvent_t *last_use) {
    uint64_t mn = 0, me = 0;
    AG_TRY(ag_sampler_bounds(l->samplers[0], n_seeds, &mn, &me));
    const uint64_t cn = std::max<uint64_t>(mn, 1), ce = std::max<uint64_t>(me, 1), cs = std::max<uint64_t>(n_seeds, 1);
    const uint64_t seen = l->x_rows_seen.load();
    const uint64_t cx = seen ? std::min<uint64_t>(cn, ((seen + seen / 2 + 4095) / 4096) * 4096) : cn;
    *last_use = nullptr;
    {
        std::lock_guard<std::mutex> lk(l->pool_m);
        for (size_t i = 0; i < l->pool_free.size(); ++i) {
            PoolSet &p = l->pool_free[i];
            if (p.bufs.cap_nodes == cn && p.bufs.cap_edges == ce && p.bufs.cap_seeds == cs &&
                (!l->f || (p.bufs.cap_x >= cx && p.bufs.cap_x <= 2 * cx))) {
                PoolSet s = p;
                l->pool_free[i] = l->pool_free.back();
                l->pool_free.pop_back();
                *last_use = s.last_use;
                s.last_use = nullptr;
                *out = s.bufs;
                l->pool_live.emplace(s.bufs.nodes, s);
                return AG_OK;
            }
        }
    }
    const bool eids = l->cfg.track_edge_ids != 0;
    const uint64_t dim = l->f ? l->f->dim : 0;
    uint64_t off = 0;
    auto carve = [&](uint64_t bytes) { const uint64_t o = off; off += align256(bytes); return o; };
    const uint64_t o_nodes = carve(cn * 4), o_esrc = carve(ce * 4), o_edst = carve(ce * 4), o_sl = carve(ce * 4),
                   o_dl = carve(ce * 4), o_seedl = carve(cs * 4), o_eid = eids ? carve(ce * 8) : 0,
                   o_nid = carve(cn * 8), o_eil = carve(ce * 16), o_sidx = carve(cs * 8);
    uint8_t *base = nullptr;
    float *xb = nullptr;
    if (cudaMalloc(&base, std::max<uint64_t>(off, 256)) != cudaSuccess ||
        (dim && cudaMalloc(&xb, std::max<uint64_t>(cx * dim * 4, 256)) != cudaSuccess)) {
        cudaFree(base);
        return fail(AG_ERR_CUDA, "loader: out of device memory for a %llu-byte batch buffer: %s",
                    (unsigned long long)(off + cx * dim * 4), cudaGetErrorString(cudaGetLastError()));
    }
    PoolSet s;
    s.base = base; s.x_base = xb;
    ag_subgraph_buffers &b = s.bufs;
    b.cap_nodes = cn; b.cap_edges = ce; b.cap_seeds = cs;
    b.nodes = (uint32_t *)(base + o_nodes); b.edge_src = (uint32_t *)(base + o_esrc);
    b.edge_dst = (uint32_t *)(base + o_edst); b.src_local = (uint32_t *)(base + o_sl);
    b.dst_local = (uint32_t *)(base + o_dl); b.seed_locals = (uint32_t *)(base + o_seedl);
    b.edge_ids = eids ? (uint64_t *)(base + o_eid) : nullptr;
    b.n_id = (int64_t *)(base + o_nid); b.edge_index_local = (int64_t *)(base + o_eil);
    b.e_id = nullptr;  // int64(edge id) shares its bits with the u64 edge_ids
    b.seed_index = (int64_t *)(base + o_sidx);
    b.x = xb; b.cap_x = dim ? cx : 0;
    *out = b;
    std::lock_guard<std::mutex> lk(l->pool_m);
    l->pool_live.emplace(b.nodes, s);
    return AG_OK;
}

// Returns a set to the pool; `stream`'s queued work (when record is true) is the
// consumer's last use of it.
void pool_give(ag_loader *l, const ag_subgraph_buffers &bufs, bool record, cudaStream_t stream) {
    std::lock_guard<std::mutex> lk(l->pool_m);
    auto it = l->pool_live.find(bufs.nodes);
    if (it == l->pool_live.end()) return;
    PoolSet s = it->second;
    l->pool_live.erase(it);
    if (record) {
        if (cudaEventCreateWithFlags(&s.last_use, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(s.last_use, stream) != cudaSuccess) {
            // Cannot order the reuse: do not reuse.
            if (s.last_use) cudaEventDestroy(s.last_use);
            cudaFree(s.base); cudaFree(s.x_base);
            return;
        }
    }
    l->pool_free.push_back(s);
}

void drop_work(ag_loader *l, Work &w) {
    for (cudaEvent_t &e : w.after) if (e) { cudaEventDestroy(e); e = nullptr; }
    if (w.owned) pool_give(l, w.bufs, false, nullptr);
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
            // a full group whenever one is queued: launch floors are paid per chain
            const size_t take = l->queue.size() >= G ? G : std::min<size_t>(G, share);
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
            for (cudaEvent_t &e : w.after) {
                if (!e) continue;
                if (cudaStreamWaitEvent(st, e, 0) != cudaSuccess) rc = fail(AG_ERR_CUDA, "cudaStreamWaitEvent failed");
                cudaEventDestroy(e);
                e = nullptr;
            }
            seed_ptrs[b] = w.seeds_dev ? w.seeds_dev : w.seeds.data();
            n_seeds[b] = w.n_seeds;
            bufs[b] = w.bufs;
            // Seeded loaders restart the stream per batch from its submission number
            // (prefetch.rs:926-930), so any pool size or grouping yields the same results.
            batch_seeds[b] = ag_batch_seed(l->cfg.seed, l->seed_base.load() + l->seed_stride.load() * w.seq);
            statuses[b] = AG_OK;
        }
        // Unseeded: a worker's own stream continues across its batches, which needs
        // the batches one at a time.
        std::string err;
        bool launched = false;  // the chain ran, so statuses[] tells the batches apart
        if (rc == AG_OK && (l->seeded || nb == 1)) {
            rc = ag_sample_group_into(s, nb, seed_ptrs.data(), n_seeds.data(),
                                      ws[0].seeds_dev ? AG_MEM_DEVICE : AG_MEM_HOST,
                                      l->seeded ? batch_seeds.data() : nullptr, l->f, bufs.data(), st);
            if (rc == AG_OK) { launched = true; rc = ag_sample_group_wait(s, counts.data(), statuses.data()); }
            if (rc != AG_OK) err = ag_last_error();
        } else if (rc == AG_OK) {
            launched = true;
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
        if (launched && l->f) {
            for (uint32_t b = 0; b < nb; ++b) {
                if (statuses[b] != AG_OK) continue;
                const uint64_t nn = counts[b].num_nodes;
                uint64_t prev = l->x_rows_seen.load();
                while (nn > prev && !l->x_rows_seen.compare_exchange_weak(prev, nn)) {}
                Work &w = ws[b];
                const uint64_t have = w.bufs.cap_x ? w.bufs.cap_x : w.bufs.cap_nodes;
                if (!w.bufs.x || nn <= have) continue;
                // The batch has more nodes than rows were reserved for: its first `have` rows are
                // in place; gather all of them again into a buffer that fits.  Pooled sets get a
                // new x; a caller's own buffer cannot grow, so that batch is reported as too small.
                if (!w.owned) {
                    statuses[b] = fail(AG_ERR_VALUE, "x holds %llu rows, the batch has %llu nodes", (unsigned long long)have, (unsigned long long)nn);
                    err = ag_last_error();
                    if (rc == AG_OK) rc = statuses[b];
                    continue;
                }
                float *bigger = nullptr;
                const uint64_t rows = ((nn + nn / 4 + 4095) / 4096) * 4096;
                int32_t g = AG_OK;
                if (cudaMalloc(&bigger, rows * l->f->dim * 4) != cudaSuccess) g = fail(AG_ERR_CUDA, "loader: out of device memory for %llu feature rows", (unsigned long long)rows);
                if (g == AG_OK) g = ag_gather(l->f, w.bufs.nodes, 0, nn, nullptr, bigger, st);
                if (g == AG_OK && cudaStreamSynchronize(st) != cudaSuccess) g = fail(AG_ERR_CUDA, "loader: gathering an outgrown batch again failed");
                if (g != AG_OK) { cudaFree(bigger); statuses[b] = g; err = ag_last_error(); if (rc == AG_OK) rc = g; continue; }
                std::lock_guard<std::mutex> pk(l->pool_m);
                auto it = l->pool_live.find(w.bufs.nodes);
                if (it != l->pool_live.end()) {
                    cudaFree(it->second.x_base);
                    it->second.x_base = bigger; it->second.bufs.x = bigger; it->second.bufs.cap_x = rows;
                    w.bufs.x = bigger; w.bufs.cap_x = rows;
                } else {
                    cudaFree(bigger);
                }
            }
        }
        const uint64_t ns = (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(Clock::now() - t0).count();
        std::unique_lock<std::mutex> lk(l->m);
        for (uint32_t b = 0; b < nb; ++b) {
            Work &w = ws[b];
            Done d;
            d.batch.batch_idx = w.batch_idx; d.batch.seq = w.seq; d.batch.bufs = w.bufs; d.batch.owned = w.owned ? 1 : 0;
            d.batch.counts = counts[b];
            // A chain that was refused before launch, or that failed as a whole, fails
            // every batch of the group; a per-batch error (bad seed, small buffer) fails
            // only that batch.
            const bool chain_failed = rc != AG_OK && statuses[b] == AG_OK &&
                                      (!launched || !(rc == AG_ERR_SAMPLING || rc == AG_ERR_VALUE || rc == AG_ERR_LOAD));
            if (statuses[b] != AG_OK || chain_failed) { d.status = statuses[b] != AG_OK ? statuses[b] : rc; d.error = err; }
            // Results channel holds `depth` batches: wait for room (prefetch.rs:1135-1143),
            // except for the batch the consumer is waiting on — holding it back could
            // stall an ordered loader whose later batches filled the channel first.
            auto room = [&] { return l->stop || l->in_ready < l->depth || w.seq == l->next_deliver; };
            if (!room()) {
                l->cv_done.notify_all();  // the consumer drains what is ready while this worker waits for room
                l->cv_room.wait(lk, room);
            }
            if (l->stop) {
                lk.unlock();
                for (uint32_t r = b; r < nb; ++r) drop_work(l, ws[r]);
                return;
            }
            if (b == 0) { l->stats.sample_time_ns += ns; l->stats.chains += (l->seeded || nb == 1) ? 1 : nb; }
            if (d.status != AG_OK && l->fault.empty() && d.status != AG_ERR_SAMPLING && d.status != AG_ERR_VALUE)
                l->fault = d.error;  // a broken worker poisons the loader; a bad batch does not
            l->ready.emplace(w.seq, std::move(d));
            l->arrival.push_back(w.seq);
            l->in_ready++;
        }
        // one wake-up per chain, not per batch: the consumer takes the batches in bulk
        l->cv_done.notify_all();
    }
}

bool has_deliverable(ag_loader *l) {
    if (l->seeded) return l->ready.count(l->next_deliver) != 0;
    return !l->arrival.empty();
}

// Caller holds l->m and has_deliverable(l) is true.
int32_t deliver(ag_loader *l, ag_batch *out, bool waited) {
    std::map<uint64_t, Done>::iterator it = l->seeded ? l->ready.find(l->next_deliver) : l->ready.find(l->arrival.front());
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
        if (d.batch.owned) pool_give(l, d.batch.bufs, false, nullptr);
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

// Builds one work item (no locking); on failure nothing is left allocated.
int32_t make_work(ag_loader *l, int64_t batch_idx, const uint32_t *seeds, uint64_t n_seeds, int32_t seeds_mem,
                  const ag_subgraph_buffers *bufs, void *after_stream, Work *w) {
    if (!seeds && n_seeds) return fail(AG_ERR_VALUE, "ag_loader_submit: null seeds");
    // Range-check where seeds enter (Seeds::new, sampler.rs:230-239).
    if (seeds_mem == AG_MEM_HOST)
        for (uint64_t i = 0; i < n_seeds; ++i)
            if ((uint64_t)seeds[i] >= l->g->num_nodes)
                return fail(AG_ERR_SAMPLING, "seed node %u (position %llu) is out of range for %llu nodes",
                            seeds[i], (unsigned long long)i, (unsigned long long)l->g->num_nodes);
    w->batch_idx = batch_idx; w->n_seeds = n_seeds;
    if (seeds_mem == AG_MEM_HOST) w->seeds.assign(seeds, seeds + n_seeds); else w->seeds_dev = seeds;
    if (bufs) {
        w->bufs = *bufs;
        // Order the batch's kernels after whatever the caller's stream has queued
        // (the previous user of recycled memory).
        if (cudaEventCreateWithFlags(&w->after[0], cudaEventDisableTiming) != cudaSuccess ||
            cudaEventRecord(w->after[0], (cudaStream_t)after_stream) != cudaSuccess) {
            if (w->after[0]) cudaEventDestroy(w->after[0]);
            w->after[0] = nullptr;
            return fail(AG_ERR_CUDA, "loader: event record failed: %s", cudaGetErrorString(cudaGetLastError()));
        }
    } else {
        AG_TRY(pool_take(l, n_seeds, &w->bufs, &w->after[1]));
        w->owned = true;
    }
    return AG_OK;
}

// Caller holds lk.  Waits for queue room like the reference's bounded channel;
// gives up after the same 30 s the consumer side waits.
int32_t enqueue(ag_loader *l, std::unique_lock<std::mutex> &lk, Work &w) {
    const bool room = l->cv_space.wait_for(lk, std::chrono::seconds(30), [&] {
        return l->stop || !l->fault.empty() || l->queue.size() < (size_t)8 * l->depth;
    });
    if (!room)
        return fail(AG_ERR_TIMEOUT, "timed out waiting for room in the work queue (%u batches queued; is anything "
                    "consuming results?)", 8 * l->depth);
    if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
    if (!l->fault.empty()) return fail(AG_ERR_WORKER, "sampler worker failed: %s", l->fault.c_str());
    w.seq = l->next_seq++;
    l->stats.submitted++;
    l->queue.push_back(std::move(w));
    return AG_OK;
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
        if (st == AG_OK && yielding_waits()) st = sampler_set_yielding_wait(s, true);
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

extern "C" int32_t ag_loader_set_seed_sequence(ag_loader *l, uint64_t base, uint64_t stride) {
    if (!l) return fail(AG_ERR_VALUE, "ag_loader_set_seed_sequence: null loader");
    if (stride == 0) return fail(AG_ERR_VALUE, "ag_loader_set_seed_sequence: stride must be >= 1");
    std::unique_lock<std::mutex> lk(l->m);
    if (l->next_seq != 0) return fail(AG_ERR_VALUE, "the seed sequence is set before the first batch is submitted");
    l->seed_base = base; l->seed_stride = stride;
    return AG_OK;
}

extern "C" int32_t ag_loader_bounds(const ag_loader *l, uint64_t n_seeds, uint64_t *max_nodes, uint64_t *max_edges) {
    if (!l) return fail(AG_ERR_VALUE, "ag_loader_bounds: null loader");
    return ag_sampler_bounds(l->samplers[0], n_seeds, max_nodes, max_edges);
}

extern "C" int32_t ag_loader_submit(ag_loader *l, int64_t batch_idx, const uint32_t *seeds, uint64_t n_seeds,
                                    int32_t seeds_mem, const ag_subgraph_buffers *bufs, void *after_stream) {
    if (!l) return fail(AG_ERR_VALUE, "ag_loader_submit: null loader");
    DeviceGuard guard(l->device);
    if (!guard.ok) return AG_ERR_CUDA;
    Work w;
    AG_TRY(make_work(l, batch_idx, seeds, n_seeds, seeds_mem, bufs, after_stream, &w));
    std::unique_lock<std::mutex> lk(l->m);
    const int32_t rc = enqueue(l, lk, w);
    lk.unlock();
    if (rc != AG_OK) { drop_work(l, w); return rc; }
    l->cv_work.notify_one();
    return AG_OK;
}

// Submits n batches in one call (submit_epoch of the reference loader,
// _core.pyi:425).  batch b uses batch_idx[b], seeds[b], n_seeds[b] and bufs[b]
// (bufs == NULL: pooled buffers).  *n_done receives how many were queued before
// an error, if any.
extern "C" int32_t ag_loader_submit_many(ag_loader *l, uint32_t n, const int64_t *batch_idx,
                                         const uint32_t *const *seeds, const uint64_t *n_seeds, int32_t seeds_mem,
                                         const ag_subgraph_buffers *bufs, void *after_stream, uint32_t *n_done) {
    if (n_done) *n_done = 0;
    if (!l || (n && (!batch_idx || !seeds || !n_seeds))) return fail(AG_ERR_VALUE, "ag_loader_submit_many: null argument");
    DeviceGuard guard(l->device);
    if (!guard.ok) return AG_ERR_CUDA;
    for (uint32_t b = 0; b < n; ++b) {
        Work w;
        AG_TRY(make_work(l, batch_idx[b], seeds[b], n_seeds[b], seeds_mem, bufs ? &bufs[b] : nullptr, after_stream, &w));
        std::unique_lock<std::mutex> lk(l->m);
        const int32_t rc = enqueue(l, lk, w);
        lk.unlock();
        if (rc != AG_OK) { drop_work(l, w); return rc; }
        if (n_done) *n_done = b + 1;
        if ((b + 1) % l->group == 0 || b + 1 == n) l->cv_work.notify_all();
    }
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
    return deliver(l, out, waited);
}

// Waits like ag_loader_next for the first batch, then also hands over every
// further batch that is already deliverable, up to max_n.  A batch that failed
// ends the call: the batches before it are returned (*n_out) with AG_OK, and
// the failure is reported by the next call.
extern "C" int32_t ag_loader_next_many(ag_loader *l, int64_t timeout_ms, uint32_t max_n, ag_batch *out,
                                       uint32_t *n_out) {
    if (!l || !out || !n_out || max_n == 0) return fail(AG_ERR_VALUE, "ag_loader_next_many: bad argument");
    *n_out = 0;
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
    while (*n_out < max_n && has_deliverable(l)) {
        // peek: a failed batch is only consumed when it is the first of the call
        const auto it = l->seeded ? l->ready.find(l->next_deliver) : l->ready.find(l->arrival.front());
        if (it->second.status != AG_OK && *n_out > 0) break;
        const int32_t rc = deliver(l, &out[*n_out], waited && *n_out == 0);
        if (rc != AG_OK) return rc;
        ++*n_out;
    }
    return AG_OK;
}

extern "C" int32_t ag_loader_try_next(ag_loader *l, ag_batch *out) {
    if (!l || !out) return fail(AG_ERR_VALUE, "ag_loader_try_next: null argument");
    std::unique_lock<std::mutex> lk(l->m);
    if (!has_deliverable(l)) {
        if (l->stop) return fail(AG_ERR_SHUTDOWN, "loader is shut down");
        if (!l->fault.empty()) return fail(AG_ERR_WORKER, "sampler worker failed: %s", l->fault.c_str());
        return fail(AG_ERR_TIMEOUT, "no batch is ready");
    }
    return deliver(l, out, false);
}

// Hands a pooled batch back.  `stream` is the stream whose already-queued work
// is the consumer's last use of the batch's memory; the next batch that gets the
// buffers waits for it.
extern "C" int32_t ag_loader_release_batch(ag_loader *l, ag_batch *batch, void *stream) {
    if (!l || !batch) return fail(AG_ERR_VALUE, "ag_loader_release_batch: null argument");
    if (batch->owned) {
        DeviceGuard guard(l->device);
        pool_give(l, batch->bufs, true, (cudaStream_t)stream);
        batch->owned = 0;
        batch->bufs = ag_subgraph_buffers{};
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
    cudaDeviceSynchronize();
    for (Work &w : l->queue) drop_work(l, w);
    for (auto &kv : l->ready) if (kv.second.batch.owned) pool_give(l, kv.second.batch.bufs, false, nullptr);
    for (ag_sampler *s : l->samplers) ag_sampler_free(s);
    for (cudaStream_t s : l->streams) cudaStreamDestroy(s);
    // Batches still held by a consumer keep their memory valid until now.
    for (PoolSet &p : l->pool_free) { if (p.last_use) cudaEventDestroy(p.last_use); cudaFree(p.base); cudaFree(p.x_base); }
    for (auto &kv : l->pool_live) { cudaFree(kv.second.base); cudaFree(kv.second.x_base); }
    delete l;
}

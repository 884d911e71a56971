// Seed registration without any allocation.
//
// Some callers cannot allocate device memory while they run: code inside a
// memory-pool or stream callback, a process whose device memory is fully
// budgeted to a framework allocator, or a latency-critical loop that must not
// hit the device-synchronising cudaMalloc / cudaFree pair.  For them this file
// offers the first step of the sampling path — register a batch's seeds:
// collapse duplicates in first-sighting order and give every input seed its
// local index (reference: crates/aethergraph-core/src/loader/sampler.rs:865-872)
// — with all scratch in a fixed array that is part of the library image.
//
// The scratch is a file-scope `static __device__` array of 160 KiB that every
// GPU which loads the library holds until the process exits.  It is shared by
// all calls on a device and keeps the previous call's contents (the kernel
// wipes what it needs first); two calls that overlap on the GPU race on it, so
// callers must order them, e.g. on one stream.
#include <mutex>

#include "common.cuh"
#include "internal.h"
#include "sampler.cuh"

namespace ag {
namespace {

constexpr uint32_t kStaticMaxSeeds = 8192;              // largest batch this entry point takes
constexpr uint32_t kStaticSlots = 2 * kStaticMaxSeeds;  // open addressing at load factor <= 0.5
constexpr int kStaticThreads = 1024;
constexpr uint32_t kStaticPending = 0x80000000u;

struct __align__(256) StaticScratch {
    unsigned long long table[kStaticSlots];  // key << 32 | pending position, later | local id
    uint32_t slot_of_seed[kStaticMaxSeeds];
};
static __device__ __align__(256) StaticScratch g_static_scratch;

// One block does the whole batch: wipe the table, insert every seed with
// atomicMin(position), flag the first sightings, scan the flags in position
// order, then hand out local ids.  Same ordering rule as the sampler's stage 0.
__global__ void __launch_bounds__(kStaticThreads)
k_register_seeds_static(StaticScratch *sc, const uint32_t *__restrict__ seeds, uint32_t n, uint64_t num_nodes,
                        uint32_t *nodes_out, uint32_t *seed_locals_out, uint32_t *count_err_out) {
    __shared__ uint32_t s_warp[kStaticThreads / 32];
    __shared__ uint32_t s_base, s_round, s_err;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (uint32_t i = tid; i < kStaticSlots; i += kStaticThreads) sc->table[i] = kSlotEmpty;
    if (tid == 0) { s_base = 0; s_err = 0; }
    __syncthreads();
    // insert: the smallest position that names a vertex wins its slot
    for (uint32_t i = tid; i < n; i += kStaticThreads) {
        const uint32_t id = seeds[i];
        uint32_t slot = 0xFFFFFFFFu;
        if ((uint64_t)id >= num_nodes) {
            atomicOr(&s_err, kErrBadSeed);
        } else {
            const unsigned long long mine = ((unsigned long long)id << 32) | (kStaticPending | i);
            uint32_t h = (id * 0x9E3779B1u) & (kStaticSlots - 1);
            for (uint32_t probe = 0; probe < kStaticSlots; ++probe) {
                unsigned long long cur = sc->table[h];
                if (cur == kSlotEmpty) {
                    cur = atomicCAS(&sc->table[h], (unsigned long long)kSlotEmpty, mine);
                    if (cur == kSlotEmpty) { slot = h; break; }
                }
                if ((uint32_t)(cur >> 32) == id) { atomicMin(&sc->table[h], mine); slot = h; break; }
                h = (h + 1) & (kStaticSlots - 1);
            }
        }
        sc->slot_of_seed[i] = slot;
    }
    __syncthreads();
    // first sightings, kStaticThreads positions per round, in position order
    for (uint32_t base = 0; base < n; base += kStaticThreads) {
        const uint32_t i = base + tid;
        bool first = false;
        uint32_t slot = 0xFFFFFFFFu;
        if (i < n) {
            slot = sc->slot_of_seed[i];
            if (slot != 0xFFFFFFFFu) first = ((uint32_t)sc->table[slot] == (kStaticPending | i));
        }
        const uint32_t ballot = __ballot_sync(0xffffffffu, first);
        const uint32_t in_warp = __popc(ballot & ((1u << lane) - 1u));
        if (lane == 0) s_warp[warp] = __popc(ballot);
        __syncthreads();
        if (warp == 0) {
            const uint32_t v = s_warp[lane];
            uint32_t incl = v;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t u = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)lane >= o) incl += u;
            }
            s_warp[lane] = incl - v;  // exclusive prefix over the warps
            if (lane == 31) s_round = incl;
        }
        __syncthreads();
        if (first) {
            const uint32_t local = s_base + s_warp[warp] + in_warp;
            nodes_out[local] = seeds[i];
            sc->table[slot] = ((unsigned long long)seeds[i] << 32) | local;
        }
        __syncthreads();
        if (tid == 0) s_base += s_round;
        __syncthreads();
    }
    for (uint32_t i = tid; i < n; i += kStaticThreads) {
        const uint32_t slot = sc->slot_of_seed[i];
        seed_locals_out[i] = (slot == 0xFFFFFFFFu) ? 0xFFFFFFFFu : (uint32_t)sc->table[slot];
    }
    if (tid == 0) { count_err_out[0] = s_base; count_err_out[1] = s_err; }
}

// Device address of the static scratch, resolved once per device.  In host code
// the array's name is only a stand-in for the symbol; the kernel needs the
// address cudaGetSymbolAddress returns with that device current.
constexpr int kMaxDevices = 64;
StaticScratch *g_scratch_ptr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

int32_t static_scratch(int device, StaticScratch **out) {
    if (device < 0 || device >= kMaxDevices) return fail(AG_ERR_VALUE, "device index %d out of range", device);
    std::lock_guard<std::mutex> lk(g_scratch_mutex);
    if (!g_scratch_ptr[device]) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess)
            return fail(AG_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed on device %d: %s", device,
                        cudaGetErrorString(e));
        g_scratch_ptr[device] = (StaticScratch *)ptr;
    }
    *out = g_scratch_ptr[device];
    return AG_OK;
}

}  // namespace
}  // namespace ag

using namespace ag;

extern "C" uint32_t ag_register_seeds_static_max(void) { return kStaticMaxSeeds; }

// Registers up to ag_register_seeds_static_max() seeds on `device` without
// allocating anything: no cudaMalloc, cudaFree or library allocation on any
// path.  seeds_dev, nodes_out_dev (capacity n_seeds), seed_locals_out_dev
// (capacity n_seeds) and count_err_out_dev (two u32: distinct count, error bits)
// are the caller's device buffers.  The first call on a device looks up the
// address of the library's static scratch (cudaGetSymbolAddress); make that
// first call before starting any stream capture.  The work is queued on
// `stream`; the outputs are ready when the stream reaches that point.
extern "C" int32_t ag_register_seeds_static(int32_t device, const uint32_t *seeds_dev, uint32_t n_seeds,
                                            uint64_t num_nodes, uint32_t *nodes_out_dev,
                                            uint32_t *seed_locals_out_dev, uint32_t *count_err_out_dev,
                                            void *stream) {
    if (n_seeds > kStaticMaxSeeds)
        return fail(AG_ERR_VALUE, "ag_register_seeds_static takes at most %u seeds per call (got %u): its scratch is "
                    "a fixed array; use a sampler handle for larger batches", kStaticMaxSeeds, n_seeds);
    if (!count_err_out_dev || (n_seeds && (!seeds_dev || !nodes_out_dev || !seed_locals_out_dev)))
        return fail(AG_ERR_VALUE, "ag_register_seeds_static: null buffer");
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    StaticScratch *sc = nullptr;
    AG_TRY(static_scratch(device, &sc));
    k_register_seeds_static<<<1, kStaticThreads, 0, (cudaStream_t)stream>>>(sc, seeds_dev, n_seeds, num_nodes,
                                                                            nodes_out_dev, seed_locals_out_dev,
                                                                            count_err_out_dev);
    AG_CUDA(cudaGetLastError());
    return AG_OK;
}

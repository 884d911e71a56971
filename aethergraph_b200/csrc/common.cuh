// Shared host/device helpers for libaethergpu: error plumbing, the two RNGs,
// cache-hinted loads/stores and the release/acquire primitives the single-pass
// scans use.  Built for sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string>

#include "../../include/aethergpu.h"

namespace ag {

// ---------------------------------------------------------------- errors --
void set_error(const char *fmt, ...);
int32_t fail(int32_t status, const char *fmt, ...);

#define AG_CUDA(expr)                                                               \
    do {                                                                            \
        cudaError_t _e = (expr);                                                    \
        if (_e != cudaSuccess)                                                      \
            return ::ag::fail(AG_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,          \
                              cudaGetErrorString(_e), __FILE__, __LINE__);          \
    } while (0)

#define AG_TRY(expr)                     \
    do {                                 \
        int32_t _s = (expr);             \
        if (_s != AG_OK) return _s;      \
    } while (0)

// RAII device switch: every entry point runs on its handle's device and
// restores the caller's current device on exit.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; prev = -1; }
        if (ok && prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
        if (!ok) set_error("cannot select CUDA device %d (is a GPU visible?)", dev);
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// Multiprocessors of the CURRENT device (B200: 148 = 2 dies x 74), read once per
// device; grids are sized in multiples of it.  Every entry point selects its
// handle's device before it sizes a grid.
int sm_count();
#define kSMs (::ag::sm_count())

// Device-side error bits (ag_sample_counts.error).
enum : uint32_t {
    kErrSpinTimeout = 1u,   // a bounded wait on another tile ran out
    kErrTableFull = 2u,     // dedup table probe wrapped
    kErrCapacity = 4u,      // an output would not fit the caller's buffers
    kErrBadSeed = 8u,       // device-side seed range check failed
    kErrBadId = 16u,        // gather id outside the feature store
    kErrBadDst = 32u,       // sampled destination outside the graph
};

#ifdef __CUDACC__
// ------------------------------------------------------------------ RNGs --
// WyRand (reference: internal/genstamp.rs:181-202).  The state is an additive
// counter, so draw d (0-based) of a generator seeded `s` is a pure function of
// (s, d): state = s + (d + 1) * C.
__device__ __forceinline__ uint64_t wyrand_at(uint64_t seed, uint64_t d) {
    const uint64_t st = seed + (d + 1ull) * 0xa0761d6478bd642full;
    const uint64_t b = st ^ 0xe7037ed1a0b428dbull;
    return __umul64hi(st, b) ^ (st * b);
}

// Philox4x32-10 (reference: internal/philox.rs:15-40): counter
// (node_lo, node_hi, layer, draw_group), key (seed_lo, seed_hi).
__device__ __forceinline__ uint4 philox4x32_10(uint64_t seed, uint32_t layer, uint64_t node,
                                               uint32_t draw_group) {
    uint32_t c0 = (uint32_t)node, c1 = (uint32_t)(node >> 32), c2 = layer, c3 = draw_group;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        const uint32_t hi0 = __umulhi(c0, 0xD2511F53u), lo0 = c0 * 0xD2511F53u;
        const uint32_t hi1 = __umulhi(c2, 0xCD9E8D57u), lo1 = c2 * 0xCD9E8D57u;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        if (round != 9) { k0 += 0x9E3779B9u; k1 += 0xBB67AE85u; }
    }
    return make_uint4(c0, c1, c2, c3);
}

// reference: internal/philox.rs:43-52
__device__ __forceinline__ uint32_t philox_u32(uint64_t seed, uint32_t layer, uint64_t node,
                                               uint32_t draw_index) {
    const uint4 r = philox4x32_10(seed, layer, node, draw_index >> 2);
    const uint32_t sel = draw_index & 3u;
    return sel == 0 ? r.x : sel == 1 ? r.y : sel == 2 ? r.z : r.w;
}

// ------------------------------------------------- cache-hinted accesses --
// Feature rows and picked destinations are touched once per batch: read them
// through the non-coherent path without allocating in L1, and write results
// with evict-first so a batch does not push the CSR offsets out of L2.
__device__ __forceinline__ uint4 ld_stream_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_v2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ld_stream_u16(const void *p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_stream_v4(void *p, uint4 v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_stream_u32(void *p, uint32_t v) {
    asm volatile("st.global.cs.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}

// ------------------------------------------------------ release/acquire --
__device__ __forceinline__ void st_release_u32(uint32_t *p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t *p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
#endif  // __CUDACC__

}  // namespace ag

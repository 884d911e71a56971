// C ABI: error plumbing, graph handles (AETH v1 files, CSR in HBM) and feature
// store handles (AETHFEAT files, payload in HBM).
#include <errno.h>
#include <fcntl.h>
#include <stdarg.h>
#include <string.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include <cub/device/device_scan.cuh>

#include "common.cuh"
#include "internal.h"

namespace ag {

static thread_local char g_error[1024] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
}

int sm_count() {
    static std::atomic<int> cache[64];  // 0: not read yet
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

int32_t fail(int32_t status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return status;
}

namespace {

// CRC32 (IEEE), the integrity checksum of the AETH body
// (reference: internal/mmap.rs:642-652).
uint32_t crc32_update(uint32_t crc, const void *data, size_t len) {
    static uint32_t table[8][256];
    static std::once_flag built;  // graphs may be loaded and saved from several threads at once
    std::call_once(built, [] {
        for (uint32_t i = 0; i < 256; ++i) {
            uint32_t c = i;
            for (int k = 0; k < 8; ++k) c = (c & 1u) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
            table[0][i] = c;
        }
        for (uint32_t i = 0; i < 256; ++i)
            for (int t = 1; t < 8; ++t) table[t][i] = table[0][table[t - 1][i] & 0xFF] ^ (table[t - 1][i] >> 8);
    });
    const uint8_t *p = (const uint8_t *)data;
    crc = ~crc;
    while (len >= 8) {  // slicing-by-8
        uint32_t a, b;
        memcpy(&a, p, 4); memcpy(&b, p + 4, 4);
        a ^= crc;
        crc = table[7][a & 0xFF] ^ table[6][(a >> 8) & 0xFF] ^ table[5][(a >> 16) & 0xFF] ^ table[4][a >> 24] ^
              table[3][b & 0xFF] ^ table[2][(b >> 8) & 0xFF] ^ table[1][(b >> 16) & 0xFF] ^ table[0][b >> 24];
        p += 8; len -= 8;
    }
    while (len--) crc = table[0][(crc ^ *p++) & 0xFF] ^ (crc >> 8);
    return ~crc;
}

__global__ void k_validate_csr(const uint64_t *offsets, const uint32_t *dst, uint64_t n, uint64_t e,
                               uint64_t dst_bound, uint32_t *flag) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid == 0) {
        if (offsets[0] != 0) atomicOr(flag, 1u);
        if (offsets[n] != e) atomicOr(flag, 2u);
    }
    for (uint64_t i = tid; i < n; i += stride)
        if (offsets[i] > offsets[i + 1]) atomicOr(flag, 4u);
    if (dst)
        for (uint64_t i = tid; i < e; i += stride)
            if ((uint64_t)dst[i] >= dst_bound) atomicOr(flag, 8u);
}

__global__ void k_degrees(const uint64_t *offsets, uint64_t num_nodes, const uint32_t *ids, uint64_t n,
                          uint32_t *out) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x) {
        const uint64_t v = ids ? ids[i] : i;
        uint64_t d = 0;
        if (v < num_nodes) {
            const uint64_t a = offsets[v], b = offsets[v + 1];
            d = b >= a ? b - a : 0;
        }
        out[i] = (uint32_t)std::min<uint64_t>(d, 0xFFFFFFFFull);
    }
}

int grid_for(uint64_t n) {
    const uint64_t b = (n + 255) / 256;
    return (int)std::max<uint64_t>(1, std::min<uint64_t>(b, (uint64_t)kSMs * 8));
}

}  // namespace

cudaError_t launch_validate_csr(const uint64_t *offsets, const uint32_t *dst, uint64_t n, uint64_t e,
                                uint64_t dst_bound, uint32_t *flag_dev, cudaStream_t st) {
    k_validate_csr<<<grid_for(std::max(n, e)), 256, 0, st>>>(offsets, dst, n, e, dst_bound, flag_dev);
    return cudaGetLastError();
}

cudaError_t launch_degrees(const uint64_t *offsets, uint64_t num_nodes, const uint32_t *ids, uint64_t n,
                           uint32_t *out, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    k_degrees<<<grid_for(n), 256, 0, st>>>(offsets, num_nodes, ids, n, out);
    return cudaGetLastError();
}

namespace {

int32_t validate_on_device(const ag_graph *g, bool check_dst) {
    uint32_t *flag = nullptr;
    AG_CUDA(cudaMalloc(&flag, 4));
    cudaMemset(flag, 0, 4);
    cudaError_t e = launch_validate_csr(g->offsets, check_dst ? g->dst : nullptr, g->num_nodes, g->num_edges,
                                        g->num_nodes, flag, 0);
    uint32_t h = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&h, flag, 4, cudaMemcpyDeviceToHost);
    cudaFree(flag);
    if (e != cudaSuccess) return fail(AG_ERR_CUDA, "CSR validation failed to run: %s", cudaGetErrorString(e));
    if (h & 1u) return fail(AG_ERR_LOAD, "invalid CSR: offsets[0] != 0");
    if (h & 2u) return fail(AG_ERR_LOAD, "invalid CSR: offsets[num_nodes] != num_edges");
    if (h & 4u) return fail(AG_ERR_LOAD, "invalid CSR: offsets are not non-decreasing");
    if (h & 8u) return fail(AG_ERR_LOAD, "invalid CSR: an edge destination is >= num_nodes");
    return AG_OK;
}

int32_t upload(void **dev, const void *src, uint64_t bytes, int mem_kind) {
    AG_CUDA(cudaMalloc(dev, std::max<uint64_t>(bytes, 16)));
    if (bytes)
        AG_CUDA(cudaMemcpy(*dev, src, bytes, mem_kind == AG_MEM_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice));
    return AG_OK;
}

// Reads exactly `bytes` at `offset`; false on a short read.
bool read_exact(int fd, void *buf, uint64_t bytes, uint64_t offset) {
    uint8_t *p = (uint8_t *)buf;
    while (bytes) {
        const ssize_t r = pread(fd, p, (size_t)std::min<uint64_t>(bytes, 1ull << 30), (off_t)offset);
        if (r <= 0) return false;
        p += r; offset += (uint64_t)r; bytes -= (uint64_t)r;
    }
    return true;
}

// Streams a file section into device memory through a pinned bounce buffer.
int32_t stream_to_device(int fd, uint64_t offset, uint64_t bytes, void *dev, uint32_t *crc) {
    const uint64_t chunk = 64ull << 20;
    void *pinned = nullptr;
    AG_CUDA(cudaHostAlloc(&pinned, (size_t)std::min(chunk, std::max<uint64_t>(bytes, 16)), cudaHostAllocDefault));
    int32_t st = AG_OK;
    for (uint64_t done = 0; done < bytes; done += chunk) {
        const uint64_t n = std::min(chunk, bytes - done);
        if (!read_exact(fd, pinned, n, offset + done)) { st = fail(AG_ERR_LOAD, "short read at offset %llu", (unsigned long long)(offset + done)); break; }
        if (crc) *crc = crc32_update(*crc, pinned, n);
        if (cudaMemcpy((uint8_t *)dev + done, pinned, n, cudaMemcpyHostToDevice) != cudaSuccess) {
            st = fail(AG_ERR_CUDA, "copy to device failed: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
    }
    cudaFreeHost(pinned);
    return st;
}

int write_all(int fd, const void *buf, uint64_t bytes) {
    const uint8_t *p = (const uint8_t *)buf;
    while (bytes) {
        const ssize_t w = write(fd, p, (size_t)std::min<uint64_t>(bytes, 1ull << 30));
        if (w <= 0) return -1;
        p += w; bytes -= (uint64_t)w;
    }
    return 0;
}

// Writes go to a sibling temporary that is fsynced and renamed over the target
// (reference: internal/mmap.rs:38-87, features/store.rs:923-986).
struct AtomicFile {
    std::string path, tmp, parent;
    int fd = -1;
    bool open_tmp(const char *target) {
        path = target;
        static std::atomic<int> seq{0};
        std::string dir = ".", name = path;
        const size_t slash = path.find_last_of('/');
        if (slash != std::string::npos) { dir = path.substr(0, slash); name = path.substr(slash + 1); if (dir.empty()) dir = "/"; }
        char suffix[64];
        snprintf(suffix, sizeof suffix, ".tmp.%d.%d", (int)getpid(), seq++);
        tmp = dir + "/." + name + suffix;
        parent = dir;
        fd = open(tmp.c_str(), O_WRONLY | O_CREAT | O_EXCL, 0644);
        return fd >= 0;
    }
    bool commit() {
        bool ok = fsync(fd) == 0;
        close(fd); fd = -1;
        if (ok) ok = rename(tmp.c_str(), path.c_str()) == 0;
        if (!ok) { unlink(tmp.c_str()); return false; }
        // the rename itself becomes durable with the directory (internal/mmap.rs:33-87)
        const int dfd = open(parent.c_str(), O_RDONLY | O_DIRECTORY);
        if (dfd >= 0) { fsync(dfd); close(dfd); }
        return true;
    }
    void abort() { if (fd >= 0) { close(fd); fd = -1; unlink(tmp.c_str()); } }
};

constexpr uint32_t kGraphMagic = 0x41455448u;  // "AETH" (internal/mmap.rs:20)
constexpr uint64_t kMaxEdges = 100000000000ull;  // internal/mmap.rs:31
constexpr uint64_t kFullValidationBytes = 512ull << 20;  // internal/mmap.rs:27


// ------------------------------------------------ AETHHETG v1 (hetero graphs) --
// The reference's multi-relational file (internal/mmap_hetero.rs:1-45): 64-byte
// header ("AETHHETG", version, type counts), node type table (64-byte name + u64
// count), edge type table (three 64-byte names, u64 source count, u64 edge count,
// u32 has_weights, u32 pad), then per edge type its CSR over the source type:
// u64 offsets, u32 destinations and optional f32 weights, the u32 sections padded
// to 8 bytes.  Like the reference's loader (mmap_hetero.rs:161-330) every size is
// checked against the file length with overflow-checked arithmetic before anything
// is read, names must be NUL-terminated, and each relation is proven in full
// (offsets start at 0, never decrease, end at the edge count; every destination
// below its destination type's count) — here on the device, after the sections
// were streamed into HBM.
constexpr uint64_t kHetHeader = 64, kHetNodeEntry = 72, kHetEdgeEntry = 216, kHetFormatTypes = 256;
constexpr uint64_t kHetMaxNodes = 0xFFFFFFFFull;

uint64_t pad8(uint64_t len) { return (0 - len) & 7; }

bool checked_add(uint64_t a, uint64_t b, uint64_t *out) { *out = a + b; return *out >= a; }
bool checked_mul(uint64_t a, uint64_t b, uint64_t *out) {
    if (a != 0 && b > 0xFFFFFFFFFFFFFFFFull / a) return false;
    *out = a * b;
    return true;
}

// A 64-byte name field: NUL-terminated, zero-padded (mmap_hetero.rs:73-81).
bool read_name(const uint8_t *field, char *out) {
    const void *nul = memchr(field, 0, 64);
    if (!nul) return false;
    memset(out, 0, 64);
    memcpy(out, field, (const uint8_t *)nul - field);
    return true;
}

__global__ void k_in_adjacency_keys(const uint64_t *in_offsets, const uint32_t *in_sources, uint64_t num_dst, uint64_t e,
                                    uint64_t *keys) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < e; i += (uint64_t)gridDim.x * blockDim.x) {
        // destination of stored position i = the row of the transposed adjacency that holds it
        uint64_t lo = 0, hi = num_dst;  // invariant: in_offsets[lo] <= i < in_offsets[hi]
        while (hi - lo > 1) {
            const uint64_t mid = (lo + hi) / 2;
            if (in_offsets[mid] <= i) lo = mid; else hi = mid;
        }
        keys[i] = ((uint64_t)in_sources[i] << 32) | lo;
    }
}

}  // namespace
}  // namespace ag

using namespace ag;

extern "C" int32_t ag_hetero_load(const char *path, int32_t device, ag_hetero_graph **out, ag_hetero_names *names) {
    if (!path || !out || !names) return fail(AG_ERR_VALUE, "ag_hetero_load: null argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(AG_ERR_LOAD, "failed to open hetero graph file %s: %s", path, strerror(errno));
    struct stat sb;
    if (fstat(fd, &sb) != 0) { close(fd); return fail(AG_ERR_LOAD, "failed to stat %s", path); }
    const uint64_t file_len = (uint64_t)sb.st_size;
    int32_t st = AG_OK;
    std::vector<uint8_t> tables;
    uint8_t header[kHetHeader];
    uint32_t num_nt = 0, num_et = 0;
    uint64_t num_nodes[AG_MAX_NODE_TYPES] = {0}, num_edges[AG_MAX_EDGE_TYPES] = {0};
    uint32_t src_type[AG_MAX_EDGE_TYPES] = {0}, dst_type[AG_MAX_EDGE_TYPES] = {0};
    uint64_t off_at[AG_MAX_EDGE_TYPES] = {0}, dst_at[AG_MAX_EDGE_TYPES] = {0};
    uint64_t *off_dev[AG_MAX_EDGE_TYPES] = {nullptr};
    uint32_t *dst_dev[AG_MAX_EDGE_TYPES] = {nullptr};
    uint32_t *flag = nullptr;
    memset(names, 0, sizeof *names);
    do {
        if (file_len < kHetHeader) { st = fail(AG_ERR_LOAD, "file too small for header: %llu bytes", (unsigned long long)file_len); break; }
        if (!read_exact(fd, header, kHetHeader, 0)) { st = fail(AG_ERR_LOAD, "failed to read the header"); break; }
        if (memcmp(header, "AETHHETG", 8) != 0) { st = fail(AG_ERR_LOAD, "invalid magic (expected AETHHETG)"); break; }
        uint32_t version;
        memcpy(&version, header + 8, 4); memcpy(&num_nt, header + 12, 4); memcpy(&num_et, header + 16, 4);
        if (version != 1) { st = fail(AG_ERR_LOAD, "hetero graph file format version %u is not supported by this build (max 1)", version); break; }
        if (num_nt > kHetFormatTypes || num_et > kHetFormatTypes) {
            st = fail(AG_ERR_LOAD, "type counts (%u node, %u edge) exceed the format limit of 256 - file is corrupt", num_nt, num_et);
            break;
        }
        if (num_nt == 0 || num_nt > AG_MAX_NODE_TYPES || num_et > AG_MAX_EDGE_TYPES) {
            st = fail(AG_ERR_LOAD, "the file holds %u node types and %u edge types; this build samples graphs of 1 to %d node types and "
                      "at most %d edge types", num_nt, num_et, AG_MAX_NODE_TYPES, AG_MAX_EDGE_TYPES);
            break;
        }
        const uint64_t tables_len = kHetHeader + num_nt * kHetNodeEntry + num_et * kHetEdgeEntry;
        if (tables_len > file_len) {
            st = fail(AG_ERR_LOAD, "file truncated: type tables need %llu bytes, file has %llu", (unsigned long long)tables_len, (unsigned long long)file_len);
            break;
        }
        tables.resize(tables_len - kHetHeader);
        if (!tables.empty() && !read_exact(fd, tables.data(), tables.size(), kHetHeader)) { st = fail(AG_ERR_LOAD, "failed to read the type tables"); break; }
        const uint8_t *p = tables.data();
        for (uint32_t t = 0; t < num_nt && st == AG_OK; ++t, p += kHetNodeEntry) {
            if (!read_name(p, names->node_type[t])) { st = fail(AG_ERR_LOAD, "type name field has no NUL terminator - file is corrupt"); break; }
            memcpy(&num_nodes[t], p + 64, 8);
            if (num_nodes[t] > kHetMaxNodes)
                st = fail(AG_ERR_LOAD, "node type '%s' count %llu exceeds maximum %llu - file is corrupt", names->node_type[t],
                          (unsigned long long)num_nodes[t], (unsigned long long)kHetMaxNodes);
        }
        if (st != AG_OK) break;
        uint64_t at = tables_len;
        for (uint32_t e = 0; e < num_et && st == AG_OK; ++e, p += kHetEdgeEntry) {
            if (!read_name(p, names->src[e]) || !read_name(p + 64, names->rel[e]) || !read_name(p + 128, names->dst[e])) {
                st = fail(AG_ERR_LOAD, "type name field has no NUL terminator - file is corrupt");
                break;
            }
            uint64_t ns;
            uint32_t has_w;
            memcpy(&ns, p + 192, 8); memcpy(&num_edges[e], p + 200, 8); memcpy(&has_w, p + 208, 4);
            const char *rel = names->rel[e];
            if (ns > kHetMaxNodes) { st = fail(AG_ERR_LOAD, "edge type '%s' num_src_nodes %llu exceeds maximum %llu - file is corrupt", rel, (unsigned long long)ns, (unsigned long long)kHetMaxNodes); break; }
            if (num_edges[e] > kMaxEdges) { st = fail(AG_ERR_LOAD, "edge type '%s' num_edges %llu exceeds maximum %llu - file is corrupt", rel, (unsigned long long)num_edges[e], (unsigned long long)kMaxEdges); break; }
            int s_id = -1, d_id = -1;
            for (uint32_t t = 0; t < num_nt; ++t) {
                if (s_id < 0 && strcmp(names->node_type[t], names->src[e]) == 0) s_id = (int)t;
                if (d_id < 0 && strcmp(names->node_type[t], names->dst[e]) == 0) d_id = (int)t;
            }
            if (d_id < 0) { st = fail(AG_ERR_LOAD, "edge type '%s' names unknown destination type '%s' - file is corrupt", rel, names->dst[e]); break; }
            if (s_id < 0) { st = fail(AG_ERR_LOAD, "edge type '%s' names unknown source type '%s' - file is corrupt", rel, names->src[e]); break; }
            if (ns != num_nodes[s_id]) {
                st = fail(AG_ERR_LOAD, "edge type '%s' has %llu source rows but node type '%s' holds %llu nodes", rel, (unsigned long long)ns,
                          names->src[e], (unsigned long long)num_nodes[s_id]);
                break;
            }
            src_type[e] = (uint32_t)s_id; dst_type[e] = (uint32_t)d_id;
            uint64_t off_bytes, edge_bytes, end;
            if (!checked_mul(ns + 1, 8, &off_bytes) || !checked_mul(num_edges[e], 4, &edge_bytes)) { st = fail(AG_ERR_LOAD, "section size overflows for edge type '%s'", rel); break; }
            auto take = [&](uint64_t len, const char *what) {
                if (!checked_add(at, len, &end)) { st = fail(AG_ERR_LOAD, "section size overflows for edge type '%s'", rel); return false; }
                if (end > file_len) {
                    st = fail(AG_ERR_LOAD, "file truncated: %s section of edge type '%s' needs bytes %llu..%llu, file has %llu", what, rel,
                              (unsigned long long)at, (unsigned long long)end, (unsigned long long)file_len);
                    return false;
                }
                at = end;
                return true;
            };
            off_at[e] = at;
            if (!take(off_bytes, "offsets")) break;
            dst_at[e] = at;
            if (!take(edge_bytes, "edges")) break;
            at += pad8(edge_bytes);
            if (has_w) {  // weights are validated for size and skipped: hetero sampling is uniform (hetero_sampler.rs:36-39)
                if (!take(edge_bytes, "weights")) break;
                at += pad8(edge_bytes);
            }
            if (at > file_len) { st = fail(AG_ERR_LOAD, "file truncated: section padding of edge type '%s' extends past EOF", rel); break; }
        }
        if (st != AG_OK) break;
        DeviceGuard guard(device);
        if (!guard.ok) { st = AG_ERR_CUDA; break; }
        if (cudaMalloc(&flag, 4) != cudaSuccess) { st = fail(AG_ERR_CUDA, "out of device memory"); break; }
        for (uint32_t e = 0; e < num_et && st == AG_OK; ++e) {
            const uint64_t ns = num_nodes[src_type[e]], E = num_edges[e];
            if (cudaMalloc(&off_dev[e], (ns + 1) * 8) != cudaSuccess || cudaMalloc(&dst_dev[e], std::max<uint64_t>(E, 1) * 4) != cudaSuccess) {
                st = fail(AG_ERR_CUDA, "out of device memory for edge type '%s'", names->rel[e]);
                break;
            }
            if ((st = stream_to_device(fd, off_at[e], (ns + 1) * 8, off_dev[e], nullptr)) != AG_OK) break;
            if (E && (st = stream_to_device(fd, dst_at[e], E * 4, dst_dev[e], nullptr)) != AG_OK) break;
            cudaMemset(flag, 0, 4);
            uint32_t hflag = 0;
            cudaError_t ce = launch_validate_csr(off_dev[e], dst_dev[e], ns, E, num_nodes[dst_type[e]], flag, 0);
            if (ce == cudaSuccess) ce = cudaMemcpy(&hflag, flag, 4, cudaMemcpyDeviceToHost);
            if (ce != cudaSuccess) { st = fail(AG_ERR_CUDA, "validation of edge type '%s' failed to run: %s", names->rel[e], cudaGetErrorString(ce)); break; }
            if (hflag & 1u) st = fail(AG_ERR_LOAD, "edge type '%s': offsets[0] != 0", names->rel[e]);
            else if (hflag & 2u) st = fail(AG_ERR_LOAD, "edge type '%s': offsets[num_src_nodes] != num_edges", names->rel[e]);
            else if (hflag & 4u) st = fail(AG_ERR_LOAD, "edge type '%s': offsets are not non-decreasing", names->rel[e]);
            else if (hflag & 8u) st = fail(AG_ERR_LOAD, "edge type '%s': a destination is >= the count of node type '%s'", names->rel[e], names->dst[e]);
        }
        if (st != AG_OK) break;
        names->num_node_types = num_nt; names->num_edge_types = num_et;
        st = ag_hetero_create(num_nt, num_nodes, num_et, src_type, dst_type, (const uint64_t *const *)off_dev, nullptr,
                              (const uint32_t *const *)dst_dev, num_edges, AG_MEM_DEVICE, device, out);
        if (st == AG_ERR_VALUE) st = AG_ERR_LOAD;  // same message, the reference's class for a bad file
    } while (0);
    close(fd);
    {
        DeviceGuard guard(device);
        for (uint32_t e = 0; e < AG_MAX_EDGE_TYPES; ++e) { cudaFree(off_dev[e]); cudaFree(dst_dev[e]); }
        cudaFree(flag);
    }
    return st;
}

// Writes the graph as AETHHETG v1, atomically (temporary file, fsync, rename:
// mmap_hetero.rs:83-96).  The forward CSR of every edge type is rebuilt from the
// transposed adjacency the handle holds, rows sorted by destination; the
// reference keeps the caller's order within a row, which no sampler observes
// (hetero sampling walks the transposed adjacency, whose order is the same).
extern "C" int32_t ag_hetero_save(const ag_hetero_graph *h, const ag_hetero_names *names, const char *path) {
    if (!h || !names || !path) return fail(AG_ERR_VALUE, "ag_hetero_save: null argument");
    DeviceGuard guard(h->device);
    if (!guard.ok) return AG_ERR_CUDA;
    for (uint32_t t = 0; t < h->nt; ++t)
        if (strnlen(names->node_type[t], 64) >= 64) return fail(AG_ERR_VALUE, "type name too long");
    AtomicFile f;
    if (!f.open_tmp(path)) return fail(AG_ERR_LOAD, "failed to create %s: %s", path, strerror(errno));
    std::vector<uint8_t> head(kHetHeader + h->nt * kHetNodeEntry + h->et * kHetEdgeEntry, 0);
    memcpy(head.data(), "AETHHETG", 8);
    const uint32_t version = 1;
    memcpy(head.data() + 8, &version, 4); memcpy(head.data() + 12, &h->nt, 4); memcpy(head.data() + 16, &h->et, 4);
    uint8_t *p = head.data() + kHetHeader;
    for (uint32_t t = 0; t < h->nt; ++t, p += kHetNodeEntry) {
        memcpy(p, names->node_type[t], strnlen(names->node_type[t], 63));
        memcpy(p + 64, &h->num_nodes[t], 8);
    }
    for (uint32_t e = 0; e < h->et; ++e, p += kHetEdgeEntry) {
        memcpy(p, names->node_type[h->src_type[e]], strnlen(names->node_type[h->src_type[e]], 63));
        memcpy(p + 64, names->rel[e], strnlen(names->rel[e], 63));
        memcpy(p + 128, names->node_type[h->dst_type[e]], strnlen(names->node_type[h->dst_type[e]], 63));
        memcpy(p + 192, &h->num_nodes[h->src_type[e]], 8);
        memcpy(p + 200, &h->num_edges[e], 8);
    }
    int32_t st = AG_OK;
    if (write_all(f.fd, head.data(), head.size()) != 0) st = fail(AG_ERR_LOAD, "failed to write %s: %s", path, strerror(errno));
    std::vector<uint8_t> bounce(64u << 20);
    for (uint32_t e = 0; e < h->et && st == AG_OK; ++e) {
        const uint64_t E = h->num_edges[e], ns = h->num_nodes[h->src_type[e]], nd = h->num_nodes[h->dst_type[e]];
        uint64_t *keys = nullptr, *off = nullptr;
        uint32_t *dst = nullptr;
        if (cudaMalloc(&keys, std::max<uint64_t>(E, 1) * 8) != cudaSuccess) { st = fail(AG_ERR_CUDA, "out of device memory"); break; }
        if (E) k_in_adjacency_keys<<<grid_for(E), 256>>>(h->in_offsets[e], h->in_sources[e], nd, E, keys);
        st = keys_to_sorted_csr(keys, E, ns, &off, &dst);  // consumes keys
        auto dump = [&](const void *dev, uint64_t bytes) {
            for (uint64_t done = 0; done < bytes && st == AG_OK; done += bounce.size()) {
                const uint64_t m = std::min<uint64_t>(bounce.size(), bytes - done);
                if (cudaMemcpy(bounce.data(), (const uint8_t *)dev + done, m, cudaMemcpyDeviceToHost) != cudaSuccess)
                    st = fail(AG_ERR_CUDA, "copy to host failed: %s", cudaGetErrorString(cudaGetLastError()));
                else if (write_all(f.fd, bounce.data(), m) != 0) st = fail(AG_ERR_LOAD, "failed to write %s: %s", path, strerror(errno));
            }
        };
        if (st == AG_OK) dump(off, (ns + 1) * 8);
        if (st == AG_OK) dump(dst, E * 4);
        const uint8_t zeros[8] = {0};
        if (st == AG_OK && pad8(E * 4) && write_all(f.fd, zeros, pad8(E * 4)) != 0) st = fail(AG_ERR_LOAD, "failed to write %s: %s", path, strerror(errno));
        cudaFree(off); cudaFree(dst);
    }
    if (st != AG_OK) { f.abort(); return st; }
    if (!f.commit()) return fail(AG_ERR_LOAD, "failed to replace %s: %s", path, strerror(errno));
    return AG_OK;
}

namespace ag {
namespace {
}  // namespace
}  // namespace ag

using namespace ag;

extern "C" const char *ag_last_error(void) { return g_error; }
extern "C" int32_t ag_abi_version(void) { return 1; }

// reference: loader/sampler.rs:69-75
extern "C" uint64_t ag_batch_seed(uint64_t base, uint64_t batch_idx) {
    uint64_t z = base ^ (batch_idx * 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

// ------------------------------------------------------------------ graph --
extern "C" void ag_graph_free(ag_graph *g) {
    if (!g) return;
    DeviceGuard guard(g->device);
    cudaFree(g->offsets); cudaFree(g->dst); cudaFree(g->weights);
    delete g;
}

extern "C" int32_t ag_graph_from_csr(uint64_t num_nodes, uint64_t num_edges, const uint64_t *offsets,
                                     const uint32_t *dst, const float *weights, int32_t mem_kind,
                                     int32_t device, ag_graph **out) {
    if (!offsets || (!dst && num_edges) || !out) return fail(AG_ERR_VALUE, "ag_graph_from_csr: null argument");
    if (num_nodes > 0xFFFFFFFFull) return fail(AG_ERR_LOAD, "num_nodes %llu exceeds the u32 id space", (unsigned long long)num_nodes);
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_graph *g = new ag_graph();
    g->device = device; g->num_nodes = num_nodes; g->num_edges = num_edges;
    int32_t st = upload((void **)&g->offsets, offsets, (num_nodes + 1) * 8, mem_kind);
    if (st == AG_OK) st = upload((void **)&g->dst, dst, num_edges * 4, mem_kind);
    if (st == AG_OK && weights) st = upload((void **)&g->weights, weights, num_edges * 4, mem_kind);
    if (st == AG_OK) st = validate_on_device(g, true);
    if (st != AG_OK) { ag_graph_free(g); return st; }
    *out = g;
    return AG_OK;
}

extern "C" int32_t ag_graph_adopt_device_csr(uint64_t num_nodes, uint64_t num_edges, uint64_t *offsets_dev,
                                             uint32_t *dst_dev, float *weights_dev, int32_t device, ag_graph **out) {
    if (!offsets_dev || (!dst_dev && num_edges) || !out) return fail(AG_ERR_VALUE, "ag_graph_adopt_device_csr: null argument");
    if (num_nodes > 0xFFFFFFFFull) return fail(AG_ERR_LOAD, "num_nodes %llu exceeds the u32 id space", (unsigned long long)num_nodes);
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_graph tmp;
    tmp.device = device; tmp.num_nodes = num_nodes; tmp.num_edges = num_edges;
    tmp.offsets = offsets_dev; tmp.dst = dst_dev; tmp.weights = weights_dev;
    AG_TRY(validate_on_device(&tmp, true));
    *out = new ag_graph(tmp);
    return AG_OK;
}

// Counting sort by source, input order kept within a row
// (reference: graph/csr.rs:568-571, 631-750).
extern "C" int32_t ag_graph_from_edges(uint64_t num_nodes, const uint32_t *src, const uint32_t *dst,
                                       const float *weights, uint64_t num_edges, int32_t device, ag_graph **out) {
    if ((num_edges && (!src || !dst)) || !out) return fail(AG_ERR_VALUE, "ag_graph_from_edges: null argument");
    for (uint64_t i = 0; i < num_edges; ++i) {
        if ((uint64_t)src[i] >= num_nodes || (uint64_t)dst[i] >= num_nodes)
            return fail(AG_ERR_VALUE, "edge %llu (%u -> %u) is out of range for %llu nodes",
                        (unsigned long long)i, src[i], dst[i], (unsigned long long)num_nodes);
    }
    std::vector<uint64_t> offsets(num_nodes + 1, 0);
    for (uint64_t i = 0; i < num_edges; ++i) offsets[(uint64_t)src[i] + 1]++;
    for (uint64_t v = 0; v < num_nodes; ++v) offsets[v + 1] += offsets[v];
    std::vector<uint64_t> cursor(offsets.begin(), offsets.end() - 1);
    std::vector<uint32_t> edges(num_edges);
    std::vector<float> w(weights ? num_edges : 0);
    for (uint64_t i = 0; i < num_edges; ++i) {
        const uint64_t at = cursor[src[i]]++;
        edges[at] = dst[i];
        if (weights) w[at] = weights[i];
    }
    return ag_graph_from_csr(num_nodes, num_edges, offsets.data(), edges.data(), weights ? w.data() : nullptr,
                             AG_MEM_HOST, device, out);
}

// ------------------------------------------------ AETH version 2 (compressed) --
// The same 32-byte header with version = 2; the checksum covers the payload
// (reference: internal/compressed_graph.rs:1-19,39-88,99-175).  Payload:
//   offsets as Elias-Fano  (internal/succinct.rs:22-92 coding, :198-214 wire format):
//     len u64 | universe u64 | low_bits u32 | low word count u64 | low words |
//     high word count u64 | high words;  element i has a set bit at (v_i >> low_bits) + i
//   edges as StreamVByte wrapping deltas over the WHOLE array (succinct.rs:392-420, :486-500):
//     len u64 | first u32 | control byte count u64 | control | data byte count u64 | data
//   weights, when present, raw f32.
// The reference decodes on the host; here the sections are streamed to the GPU as they
// lie in the file and decoded there: a scan of the high words' popcounts gives every
// word the index of its first element, a scan of the control bytes' lengths gives every
// group of four deltas its place in the data stream, and a wrapping inclusive sum turns
// the deltas into ids.
namespace ag {
namespace {

constexpr uint32_t kCompressedVersion = 2;  // internal/compressed_graph.rs:35

__global__ void k_popcount_words(const uint64_t *__restrict__ w, uint64_t n, uint64_t *__restrict__ counts) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= n; i += (uint64_t)gridDim.x * blockDim.x)
        counts[i] = i < n ? (uint64_t)__popcll(w[i]) : 0ull;  // entry n: receives the total
}

// flag bits: 1 more set bits than elements, 2 an element above the universe
__global__ void k_ef_decode(const uint64_t *__restrict__ high, uint64_t n_words, const uint64_t *__restrict__ first_index,
                            const uint64_t *__restrict__ low, uint32_t low_bits, uint64_t len, uint64_t max_high,
                            uint64_t *__restrict__ out, uint32_t *flag) {
    const uint64_t low_mask = low_bits == 0 ? 0ull : ((1ull << low_bits) - 1ull);
    for (uint64_t wi = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; wi < n_words; wi += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t w = high[wi];
        uint64_t i = first_index[wi];
        while (w) {
            const uint64_t pos = wi * 64 + (uint64_t)(__ffsll((long long)w) - 1);
            w &= w - 1;
            if (i >= len) { atomicOr(flag, 1u); break; }
            const uint64_t high_part = pos - i;
            if (high_part > max_high) { atomicOr(flag, 2u); break; }
            uint64_t low_part = 0;
            if (low_bits) {  // succinct.rs:318-333
                const uint64_t bit = i * low_bits, word = bit >> 6, off = bit & 63;
                low_part = low[word] >> off;
                if (off + low_bits > 64) low_part |= low[word + 1] << (64 - off);
                low_part &= low_mask;
            }
            out[i] = (high_part << low_bits) | low_part;
            ++i;
        }
    }
}

// Data bytes taken by the (up to four) deltas of every control byte.
__global__ void k_svb_group_bytes(const uint8_t *__restrict__ control, uint64_t n_control, uint64_t n_deltas,
                                  uint64_t *__restrict__ bytes) {
    for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c <= n_control; c += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t total = 0;
        if (c < n_control) {
            const uint32_t tags = control[c];
            for (uint32_t j = 0; j < 4 && c * 4 + j < n_deltas; ++j) total += ((tags >> (2 * j)) & 3u) + 1u;
        }
        bytes[c] = total;  // entry n_control: receives the total
    }
}

// out[0] = first, out[i + 1] = delta i (succinct.rs:466-484 before its running sum).
__global__ void k_svb_deltas(const uint8_t *__restrict__ control, const uint8_t *__restrict__ data,
                             const uint64_t *__restrict__ group_at, uint64_t n_control, uint64_t n_deltas, uint32_t first,
                             uint32_t *__restrict__ out) {
    if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = first;
    for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_control; c += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t tags = control[c];
        uint64_t at = group_at[c];
        for (uint32_t j = 0; j < 4 && c * 4 + j < n_deltas; ++j) {
            const uint32_t nbytes = ((tags >> (2 * j)) & 3u) + 1u;
            uint32_t v = 0;
            for (uint32_t b = 0; b < nbytes; ++b) v |= (uint32_t)data[at + b] << (8 * b);
            out[c * 4 + j + 1] = v;
            at += nbytes;
        }
    }
}

template <typename T>
int32_t device_scan(T *d, uint64_t n, bool inclusive) {
    if (n == 0) return AG_OK;
    void *temp = nullptr;
    size_t temp_bytes = 0;
    cudaError_t e = inclusive ? cub::DeviceScan::InclusiveSum(nullptr, temp_bytes, d, d, (size_t)n)
                              : cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, d, d, (size_t)n);
    if (e == cudaSuccess) e = cudaMalloc(&temp, std::max<size_t>(temp_bytes, 16));
    if (e == cudaSuccess)
        e = inclusive ? cub::DeviceScan::InclusiveSum(temp, temp_bytes, d, d, (size_t)n)
                      : cub::DeviceScan::ExclusiveSum(temp, temp_bytes, d, d, (size_t)n);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaFree(temp);
    if (e != cudaSuccess) return fail(AG_ERR_CUDA, "device scan failed: %s", cudaGetErrorString(e));
    return AG_OK;
}

// A cursor over the payload: every byte read goes through the checksum, in file order.
struct PayloadReader {
    int fd;
    uint64_t pos, end;
    uint32_t crc = 0;
    bool take(void *buf, uint64_t n) {
        if (n > end - pos || !read_exact(fd, buf, n, pos)) return false;
        crc = crc32_update(crc, buf, n);
        pos += n;
        return true;
    }
    bool u64(uint64_t *v) { return take(v, 8); }
    bool u32(uint32_t *v) { return take(v, 4); }
    // a section of `bytes` bytes straight into device memory
    int32_t to_device(void *dev, uint64_t bytes) {
        if (bytes > end - pos) return fail(AG_ERR_LOAD, "truncated: need %llu bytes at %llu", (unsigned long long)bytes, (unsigned long long)(pos - 32));
        AG_TRY(stream_to_device(fd, pos, bytes, dev, &crc));
        pos += bytes;
        return AG_OK;
    }
};

struct DevBuf {  // frees what a failed load leaves behind
    void *p = nullptr;
    ~DevBuf() { cudaFree(p); }
    cudaError_t alloc(uint64_t bytes) { return cudaMalloc(&p, std::max<uint64_t>(bytes, 16)); }
    template <typename T> T *as() { return (T *)p; }
    void *release() { void *q = p; p = nullptr; return q; }
};

int32_t load_graph_compressed(int fd, uint64_t file_size, uint64_t n, uint64_t e, bool has_w, uint32_t checksum,
                              int device, ag_graph **out) {
    PayloadReader r{fd, 32, file_size};
    auto truncated = [&](const char *what) {
        return fail(AG_ERR_LOAD, "%s: truncated: the payload ends at byte %llu", what, (unsigned long long)(file_size - 32));
    };
    // ---- offsets section
    uint64_t ef_len, universe, low_words, high_words;
    uint32_t low_bits;
    if (!r.u64(&ef_len) || !r.u64(&universe) || !r.u32(&low_bits) || !r.u64(&low_words)) return truncated("offsets section");
    if (low_bits >= 64) return fail(AG_ERR_LOAD, "offsets section: EF low_bits %u out of range", low_bits);
    if (low_words > (file_size - r.pos) / 8) return truncated("offsets section: EF low words");
    DevBuf low, high, first_index, offsets, control, data, group_at, dst, weights, flag;
    if (low.alloc((low_words + 1) * 8) != cudaSuccess) return fail(AG_ERR_CUDA, "out of device memory for the offsets section");
    AG_CUDA(cudaMemset(low.p, 0, (low_words + 1) * 8));  // one word past the end: the two-word read of the last element
    AG_TRY(r.to_device(low.p, low_words * 8));
    if (!r.u64(&high_words)) return truncated("offsets section");
    if (high_words > (file_size - r.pos) / 8) return truncated("offsets section: EF high words");
    if (ef_len != n + 1) return fail(AG_ERR_LOAD, "offsets section has %llu entries for %llu nodes", (unsigned long long)ef_len, (unsigned long long)n);
    // succinct.rs:236-246: the low array must cover len * low_bits bits
    const unsigned __int128 low_bits_total = (unsigned __int128)ef_len * low_bits;
    if ((unsigned __int128)low_words * 64 < low_bits_total)
        return fail(AG_ERR_LOAD, "offsets section: EF low array truncated: %llu words", (unsigned long long)low_words);
    if (high.alloc(high_words * 8) != cudaSuccess || first_index.alloc((high_words + 1) * 8) != cudaSuccess ||
        offsets.alloc(ef_len * 8) != cudaSuccess || flag.alloc(4) != cudaSuccess)
        return fail(AG_ERR_CUDA, "out of device memory for the offsets section");
    AG_TRY(r.to_device(high.p, high_words * 8));
    AG_CUDA(cudaMemset(flag.p, 0, 4));
    k_popcount_words<<<grid_for(high_words + 1), 256>>>(high.as<uint64_t>(), high_words, first_index.as<uint64_t>());
    AG_TRY(device_scan(first_index.as<uint64_t>(), high_words + 1, false));
    uint64_t ones = 0;
    AG_CUDA(cudaMemcpy(&ones, first_index.as<uint64_t>() + high_words, 8, cudaMemcpyDeviceToHost));
    if (ones != ef_len)
        return fail(AG_ERR_LOAD, "offsets section: EF high array has %llu set bits for %llu elements", (unsigned long long)ones, (unsigned long long)ef_len);
    if (high_words)
        k_ef_decode<<<grid_for(high_words), 256>>>(high.as<uint64_t>(), high_words, first_index.as<uint64_t>(), low.as<uint64_t>(),
                                                   low_bits, ef_len, universe >> low_bits, offsets.as<uint64_t>(), flag.as<uint32_t>());
    uint32_t bad = 0;
    uint64_t last = 0;
    AG_CUDA(cudaMemcpy(&bad, flag.p, 4, cudaMemcpyDeviceToHost));
    if (bad) return fail(AG_ERR_LOAD, "offsets section: an EF element exceeds universe %llu", (unsigned long long)universe);
    AG_CUDA(cudaMemcpy(&last, offsets.as<uint64_t>() + ef_len - 1, 8, cudaMemcpyDeviceToHost));
    if (last != universe)
        return fail(AG_ERR_LOAD, "offsets section: EF last element %llu disagrees with universe %llu", (unsigned long long)last, (unsigned long long)universe);
    cudaFree(low.release()); cudaFree(high.release()); cudaFree(first_index.release());

    // ---- edges section
    uint64_t svb_len, n_control, n_data;
    uint32_t first;
    if (!r.u64(&svb_len) || !r.u32(&first) || !r.u64(&n_control)) return truncated("edges section");
    if (svb_len != e) return fail(AG_ERR_LOAD, "edges section has %llu entries, header says %llu", (unsigned long long)svb_len, (unsigned long long)e);
    const uint64_t n_deltas = svb_len ? svb_len - 1 : 0;
    if (n_control != (n_deltas + 3) / 4)
        return fail(AG_ERR_LOAD, "edges section: SVB control stream is %llu bytes for %llu deltas", (unsigned long long)n_control, (unsigned long long)n_deltas);
    if (n_control > file_size - r.pos) return truncated("edges section: SVB control stream");
    if (control.alloc(n_control) != cudaSuccess || group_at.alloc((n_control + 1) * 8) != cudaSuccess)
        return fail(AG_ERR_CUDA, "out of device memory for the edges section");
    AG_TRY(r.to_device(control.p, n_control));
    if (!r.u64(&n_data)) return truncated("edges section");
    if (n_data > file_size - r.pos) return truncated("edges section: SVB data stream");
    k_svb_group_bytes<<<grid_for(n_control + 1), 256>>>(control.as<uint8_t>(), n_control, n_deltas, group_at.as<uint64_t>());
    AG_TRY(device_scan(group_at.as<uint64_t>(), n_control + 1, false));
    uint64_t need = 0;
    AG_CUDA(cudaMemcpy(&need, group_at.as<uint64_t>() + n_control, 8, cudaMemcpyDeviceToHost));
    if (need != n_data)
        return fail(AG_ERR_LOAD, "edges section: SVB data stream is %llu bytes, control tags call for %llu", (unsigned long long)n_data, (unsigned long long)need);
    if (data.alloc(n_data) != cudaSuccess || dst.alloc(e * 4) != cudaSuccess)
        return fail(AG_ERR_CUDA, "out of device memory for the edges section");
    AG_TRY(r.to_device(data.p, n_data));
    if (e) {
        k_svb_deltas<<<grid_for(std::max<uint64_t>(n_control, 1)), 256>>>(control.as<uint8_t>(), data.as<uint8_t>(), group_at.as<uint64_t>(),
                                                                         n_control, n_deltas, first, dst.as<uint32_t>());
        AG_TRY(device_scan(dst.as<uint32_t>(), e, true));  // wrapping running sum (succinct.rs:472-483)
    }
    cudaFree(control.release()); cudaFree(data.release()); cudaFree(group_at.release());

    // ---- weights
    if (has_w) {
        if (file_size - r.pos != e * 4)
            return fail(AG_ERR_LOAD, "weights section is %llu bytes for %llu edges", (unsigned long long)(file_size - r.pos), (unsigned long long)e);
        if (weights.alloc(e * 4) != cudaSuccess) return fail(AG_ERR_CUDA, "out of device memory for the weights");
        AG_TRY(r.to_device(weights.p, e * 4));
    } else if (r.pos != file_size) {
        return fail(AG_ERR_LOAD, "trailing bytes after edges section");
    }
    // every load with a checksum verifies it (compressed_graph.rs:107-117)
    if (checksum != 0 && r.crc != checksum)
        return fail(AG_ERR_LOAD, "compressed graph checksum mismatch: expected %#x, got %#x", checksum, r.crc);
    AG_CUDA(cudaDeviceSynchronize());
    ag_graph *g = new ag_graph();
    g->device = device; g->num_nodes = n; g->num_edges = e;
    g->offsets = (uint64_t *)offsets.release(); g->dst = (uint32_t *)dst.release();
    g->weights = has_w ? (float *)weights.release() : nullptr;
    const int32_t st = validate_on_device(g, true);  // always Full (compressed_graph.rs:84-89,165-172)
    if (st != AG_OK) { ag_graph_free(g); return st; }
    *out = g;
    return AG_OK;
}

}  // namespace
}  // namespace ag

// Host-side encoder (the write path is not hot): Graph.save(path, compressed=True).
extern "C" int32_t ag_graph_save_compressed(const ag_graph *g, const char *path) {
    if (!g || !path) return fail(AG_ERR_VALUE, "ag_graph_save_compressed: null argument");
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint64_t n = g->num_nodes, e = g->num_edges;
    std::vector<uint64_t> offsets(n + 1);
    std::vector<uint32_t> edges(e);
    std::vector<float> w(g->weights ? e : 0);
    AG_CUDA(cudaMemcpy(offsets.data(), g->offsets, offsets.size() * 8, cudaMemcpyDeviceToHost));
    if (e) AG_CUDA(cudaMemcpy(edges.data(), g->dst, e * 4, cudaMemcpyDeviceToHost));
    if (g->weights && e) AG_CUDA(cudaMemcpy(w.data(), g->weights, e * 4, cudaMemcpyDeviceToHost));
    std::vector<uint8_t> payload;
    auto put = [&](const void *p, size_t bytes) { payload.insert(payload.end(), (const uint8_t *)p, (const uint8_t *)p + bytes); };
    {   // Elias-Fano of the offsets (succinct.rs:52-92)
        const uint64_t len = offsets.size(), universe = offsets.back();
        uint32_t low_bits = 0;
        if (universe >= len) { uint64_t q = universe / len; while (q >>= 1) ++low_bits; }
        const uint64_t high_len = len + (universe >> low_bits) + 1;
        std::vector<uint64_t> high((high_len + 63) / 64, 0), low;
        const uint64_t low_mask = low_bits ? ((1ull << low_bits) - 1ull) : 0ull;
        uint64_t bit_len = 0;
        for (uint64_t i = 0; i < len; ++i) {
            const uint64_t v = offsets[i];
            if (low_bits) {
                const uint64_t value = v & low_mask, word = bit_len / 64, off = bit_len % 64;
                if (word >= low.size()) low.push_back(0);
                low[word] |= value << off;
                if (off + low_bits > 64) low.push_back(value >> (64 - off));
                bit_len += low_bits;
            }
            const uint64_t hp = (v >> low_bits) + i;
            high[hp / 64] |= 1ull << (hp % 64);
        }
        const uint64_t lw = low.size(), hw = high.size();
        put(&len, 8); put(&universe, 8); put(&low_bits, 4); put(&lw, 8); put(low.data(), lw * 8); put(&hw, 8); put(high.data(), hw * 8);
    }
    {   // StreamVByte of the wrapping deltas of the whole edge array (succinct.rs:397-420)
        const uint64_t len = e;
        const uint32_t first = e ? edges[0] : 0;
        const uint64_t n_deltas = e ? e - 1 : 0;
        std::vector<uint8_t> control((n_deltas + 3) / 4, 0), data;
        data.reserve(n_deltas);
        uint32_t prev = first;
        for (uint64_t i = 0; i < n_deltas; ++i) {
            const uint32_t v = edges[i + 1], delta = v - prev;
            const uint32_t nbytes = delta < (1u << 8) ? 1 : delta < (1u << 16) ? 2 : delta < (1u << 24) ? 3 : 4;
            for (uint32_t b = 0; b < nbytes; ++b) data.push_back((uint8_t)(delta >> (8 * b)));
            control[i / 4] |= (uint8_t)((nbytes - 1) << ((i % 4) * 2));
            prev = v;
        }
        const uint64_t nc = control.size(), nd = data.size();
        put(&len, 8); put(&first, 4); put(&nc, 8); put(control.data(), nc); put(&nd, 8); put(data.data(), nd);
    }
    if (g->weights) put(w.data(), w.size() * 4);
    const uint32_t crc = crc32_update(0, payload.data(), payload.size());
    uint8_t h[32] = {0};
    const uint32_t version = kCompressedVersion, has_w = g->weights ? 1 : 0;
    memcpy(h, &kGraphMagic, 4); memcpy(h + 4, &version, 4); memcpy(h + 8, &n, 8);
    memcpy(h + 16, &e, 8); memcpy(h + 24, &has_w, 4); memcpy(h + 28, &crc, 4);
    AtomicFile f;
    if (!f.open_tmp(path)) return fail(AG_ERR_LOAD, "failed to create %s: %s", path, strerror(errno));
    if (write_all(f.fd, h, 32) || write_all(f.fd, payload.data(), payload.size())) {
        f.abort();
        return fail(AG_ERR_LOAD, "failed to write %s: %s", path, strerror(errno));
    }
    if (!f.commit()) return fail(AG_ERR_LOAD, "failed to move output into %s: %s", path, strerror(errno));
    return AG_OK;
}


// AETH v1 (reference: internal/mmap.rs:114-121 header, :502-600 layout,
// :601-632 checksum policy, :633-643 default validation level).
extern "C" int32_t ag_graph_load(const char *path, int32_t validation, int32_t device, ag_graph **out) {
    if (!path || !out) return fail(AG_ERR_VALUE, "ag_graph_load: null argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(AG_ERR_LOAD, "failed to open graph file %s: %s", path, strerror(errno));
    struct stat sb;
    if (fstat(fd, &sb) != 0) { close(fd); return fail(AG_ERR_LOAD, "failed to stat %s", path); }
    const uint64_t file_size = (uint64_t)sb.st_size;
    uint8_t h[32];
    if (file_size < 32 || !read_exact(fd, h, 32, 0)) {
        close(fd);
        return fail(AG_ERR_LOAD, "insufficient bytes for header: got %llu, need 32", (unsigned long long)file_size);
    }
    uint32_t magic, version, has_w, checksum;
    uint64_t n, e;
    memcpy(&magic, h, 4); memcpy(&version, h + 4, 4); memcpy(&n, h + 8, 8); memcpy(&e, h + 16, 8);
    memcpy(&has_w, h + 24, 4); memcpy(&checksum, h + 28, 4);
    auto bail = [&](int32_t st) { close(fd); return st; };
    if (magic != kGraphMagic) return bail(fail(AG_ERR_LOAD, "invalid magic number"));
    if (version != 1 && version != 2) return bail(fail(AG_ERR_LOAD, "unsupported version: expected 1, got %u", version));
    if (n > 0xFFFFFFFFull) return bail(fail(AG_ERR_LOAD, "num_nodes %llu exceeds maximum %llu", (unsigned long long)n, 0xFFFFFFFFull));
    if (e > kMaxEdges) return bail(fail(AG_ERR_LOAD, "num_edges %llu exceeds maximum %llu", (unsigned long long)e, (unsigned long long)kMaxEdges));
    if (version == 2) {  // succinct-coded CSR: decoded on the device, always fully validated
        DeviceGuard guard2(device);
        if (!guard2.ok) return bail(AG_ERR_CUDA);
        const int32_t st2 = load_graph_compressed(fd, file_size, n, e, has_w != 0, checksum, device, out);
        close(fd);
        return st2;
    }
    const uint64_t off_bytes = (n + 1) * 8, edge_bytes = e * 4, w_bytes = has_w ? e * 4 : 0;
    const uint64_t need = 32 + off_bytes + edge_bytes + w_bytes;
    if (file_size < need)
        return bail(fail(AG_ERR_LOAD, "file too small: expected at least %llu bytes, got %llu",
                         (unsigned long long)need, (unsigned long long)file_size));
    if (validation == AG_VALIDATE_AUTO)
        validation = file_size > kFullValidationBytes ? AG_VALIDATE_OFFSETS : AG_VALIDATE_FULL;

    DeviceGuard guard(device);
    if (!guard.ok) return bail(AG_ERR_CUDA);
    ag_graph *g = new ag_graph();
    g->device = device; g->num_nodes = n; g->num_edges = e;
    int32_t st = AG_OK;
    uint32_t crc = 0;
    const bool want_crc = validation == AG_VALIDATE_FULL && checksum != 0;
    do {
        if (cudaMalloc(&g->offsets, std::max<uint64_t>(off_bytes, 16)) != cudaSuccess ||
            cudaMalloc(&g->dst, std::max<uint64_t>(edge_bytes, 16)) != cudaSuccess ||
            (has_w && cudaMalloc(&g->weights, std::max<uint64_t>(w_bytes, 16)) != cudaSuccess)) {
            st = fail(AG_ERR_CUDA, "out of device memory loading %s: %s", path, cudaGetErrorString(cudaGetLastError()));
            break;
        }
        if ((st = stream_to_device(fd, 32, off_bytes, g->offsets, want_crc ? &crc : nullptr)) != AG_OK) break;
        if ((st = stream_to_device(fd, 32 + off_bytes, edge_bytes, g->dst, want_crc ? &crc : nullptr)) != AG_OK) break;
        if (has_w && (st = stream_to_device(fd, 32 + off_bytes + edge_bytes, w_bytes, g->weights, nullptr)) != AG_OK) break;
        if (want_crc && crc != checksum) {
            st = fail(AG_ERR_LOAD, "graph integrity checksum mismatch: expected %#x, got %#x", checksum, crc);
            break;
        }
        // The sampler indexes its tables by destination id, so destinations are
        // always proven in range here, whatever level the caller asked for.
        st = validate_on_device(g, true);
    } while (0);
    close(fd);
    if (st != AG_OK) { ag_graph_free(g); return st; }
    *out = g;
    return AG_OK;
}

extern "C" int32_t ag_graph_save(const ag_graph *g, const char *path) {
    if (!g || !path) return fail(AG_ERR_VALUE, "ag_graph_save: null argument");
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    std::vector<uint64_t> offsets(g->num_nodes + 1);
    std::vector<uint32_t> edges(g->num_edges);
    std::vector<float> w(g->weights ? g->num_edges : 0);
    AG_CUDA(cudaMemcpy(offsets.data(), g->offsets, offsets.size() * 8, cudaMemcpyDeviceToHost));
    if (g->num_edges) AG_CUDA(cudaMemcpy(edges.data(), g->dst, edges.size() * 4, cudaMemcpyDeviceToHost));
    if (g->weights && g->num_edges) AG_CUDA(cudaMemcpy(w.data(), g->weights, w.size() * 4, cudaMemcpyDeviceToHost));
    uint32_t crc = crc32_update(0, offsets.data(), offsets.size() * 8);
    crc = crc32_update(crc, edges.data(), edges.size() * 4);
    uint8_t h[32] = {0};
    const uint32_t version = 1, has_w = g->weights ? 1 : 0;
    memcpy(h, &kGraphMagic, 4); memcpy(h + 4, &version, 4); memcpy(h + 8, &g->num_nodes, 8);
    memcpy(h + 16, &g->num_edges, 8); memcpy(h + 24, &has_w, 4); memcpy(h + 28, &crc, 4);
    AtomicFile f;
    if (!f.open_tmp(path)) return fail(AG_ERR_LOAD, "failed to create %s: %s", path, strerror(errno));
    if (write_all(f.fd, h, 32) || write_all(f.fd, offsets.data(), offsets.size() * 8) ||
        write_all(f.fd, edges.data(), edges.size() * 4) || (has_w && write_all(f.fd, w.data(), w.size() * 4))) {
        f.abort();
        return fail(AG_ERR_LOAD, "failed to write %s: %s", path, strerror(errno));
    }
    if (!f.commit()) return fail(AG_ERR_LOAD, "failed to move output into %s: %s", path, strerror(errno));
    return AG_OK;
}


extern "C" int32_t ag_graph_info(const ag_graph *g, uint64_t *num_nodes, uint64_t *num_edges,
                                 int32_t *has_weights, int32_t *device) {
    if (!g) return fail(AG_ERR_VALUE, "ag_graph_info: null graph");
    if (num_nodes) *num_nodes = g->num_nodes;
    if (num_edges) *num_edges = g->num_edges;
    if (has_weights) *has_weights = g->weights ? 1 : 0;
    if (device) *device = g->device;
    return AG_OK;
}

extern "C" int32_t ag_graph_device_ptrs(const ag_graph *g, const uint64_t **offsets_dev,
                                        const uint32_t **dst_dev, const float **weights_dev) {
    if (!g) return fail(AG_ERR_VALUE, "ag_graph_device_ptrs: null graph");
    if (offsets_dev) *offsets_dev = g->offsets;
    if (dst_dev) *dst_dev = g->dst;
    if (weights_dev) *weights_dev = g->weights;
    return AG_OK;
}

extern "C" int32_t ag_graph_copy_to_host(const ag_graph *g, uint64_t *offsets, uint32_t *dst, float *weights) {
    if (!g) return fail(AG_ERR_VALUE, "ag_graph_copy_to_host: null graph");
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    if (offsets) AG_CUDA(cudaMemcpy(offsets, g->offsets, (g->num_nodes + 1) * 8, cudaMemcpyDeviceToHost));
    if (dst && g->num_edges) AG_CUDA(cudaMemcpy(dst, g->dst, g->num_edges * 4, cudaMemcpyDeviceToHost));
    if (weights && g->weights && g->num_edges)
        AG_CUDA(cudaMemcpy(weights, g->weights, g->num_edges * 4, cudaMemcpyDeviceToHost));
    return AG_OK;
}

extern "C" int32_t ag_features_copy_to_host(const ag_features *f, void *payload) {
    if (!f || !payload) return fail(AG_ERR_VALUE, "ag_features_copy_to_host: null argument");
    if (f->shards) return fail(AG_ERR_VALUE, "ag_features_copy_to_host: a sharded view holds no rows of its own; copy each shard");
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    const uint64_t bytes = f->rows * f->dim * elem_size(f->dtype);
    if (bytes) AG_CUDA(cudaMemcpy(payload, f->payload, bytes, cudaMemcpyDeviceToHost));
    return AG_OK;
}

extern "C" int32_t ag_graph_degrees(const ag_graph *g, const uint32_t *ids, uint64_t n, uint32_t *out) {
    if (!g || (!out && n)) return fail(AG_ERR_VALUE, "ag_graph_degrees: null argument");
    if (n == 0) return AG_OK;
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint32_t *ids_dev = nullptr, *out_dev = nullptr;
    int32_t st = AG_OK;
    do {
        if (ids && (st = upload((void **)&ids_dev, ids, n * 4, AG_MEM_HOST)) != AG_OK) break;
        if (cudaMalloc(&out_dev, n * 4) != cudaSuccess) { st = fail(AG_ERR_CUDA, "out of device memory"); break; }
        cudaError_t e = launch_degrees(g->offsets, g->num_nodes, ids_dev, n, out_dev, 0);
        if (e == cudaSuccess) e = cudaMemcpy(out, out_dev, n * 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) st = fail(AG_ERR_CUDA, "degrees failed: %s", cudaGetErrorString(e));
    } while (0);
    cudaFree(ids_dev); cudaFree(out_dev);
    return st;
}

extern "C" int32_t ag_graph_neighbors(const ag_graph *g, uint32_t node, uint32_t *out, float *weights_out,
                                      uint64_t cap, uint64_t *degree) {
    if (!g) return fail(AG_ERR_VALUE, "ag_graph_neighbors: null graph");
    if (degree) *degree = 0;
    if ((uint64_t)node >= g->num_nodes) return AG_OK;  // empty row, like graph/csr.rs:318-335
    DeviceGuard guard(g->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint64_t ab[2];
    AG_CUDA(cudaMemcpy(ab, g->offsets + node, 16, cudaMemcpyDeviceToHost));
    if (ab[0] > ab[1] || ab[1] > g->num_edges) return AG_OK;
    const uint64_t d = ab[1] - ab[0];
    if (degree) *degree = d;
    const uint64_t m = std::min(d, cap);
    if (m && out) AG_CUDA(cudaMemcpy(out, g->dst + ab[0], m * 4, cudaMemcpyDeviceToHost));
    if (m && weights_out && g->weights) AG_CUDA(cudaMemcpy(weights_out, g->weights + ab[0], m * 4, cudaMemcpyDeviceToHost));
    return AG_OK;
}

// --------------------------------------------------------------- features --
namespace {

constexpr uint64_t kFeatHeader = 32;       // features/header.rs:118
constexpr uint64_t kFeatDataOffset = 512;  // features/store.rs:45
constexpr uint64_t kMaxFeatNodes = 10000000000ull, kMaxFeatDim = 100000ull;  // header.rs:120-121

struct FeatHeader { uint64_t n, dim, offset; int dtype; };

// reference: features/header.rs:165-244
int32_t parse_feature_header(int fd, uint64_t file_size, FeatHeader *out) {
    uint8_t p[33] = {0};
    const uint64_t len = std::min<uint64_t>(33, file_size);
    if (file_size < kFeatHeader || !read_exact(fd, p, len, 0))
        return fail(AG_ERR_LOAD, "feature file too small: %llu bytes", (unsigned long long)file_size);
    if (memcmp(p, "AETHFEAT", 8) != 0) return fail(AG_ERR_LOAD, "invalid feature file format (bad magic)");
    uint64_t n, dim, off;
    memcpy(&n, p + 8, 8); memcpy(&dim, p + 16, 8); memcpy(&off, p + 24, 8);
    if (n > kMaxFeatNodes) return fail(AG_ERR_LOAD, "num_nodes %llu exceeds maximum %llu", (unsigned long long)n, (unsigned long long)kMaxFeatNodes);
    if (dim > kMaxFeatDim) return fail(AG_ERR_LOAD, "feature_dim %llu exceeds maximum %llu", (unsigned long long)dim, (unsigned long long)kMaxFeatDim);
    if (off <= kFeatHeader) return fail(AG_ERR_LOAD, "invalid data_offset %llu (must be > 32)", (unsigned long long)off);
    if (off % 4) return fail(AG_ERR_LOAD, "invalid data_offset %llu (must be 4-byte aligned)", (unsigned long long)off);
    if (off > file_size) return fail(AG_ERR_LOAD, "invalid data_offset %llu for file size %llu", (unsigned long long)off, (unsigned long long)file_size);
    if (len < 33) return fail(AG_ERR_LOAD, "failed to read dtype tag");
    const int tag = p[32];
    if (tag > 2) return fail(AG_ERR_LOAD, "unknown feature dtype tag: %d", tag);
    const uint64_t row = dim * elem_size(tag);
    if (n && row > (0xFFFFFFFFFFFFFFFFull - off) / n) return fail(AG_ERR_LOAD, "feature data size overflow");
    if (file_size < off + n * row)
        return fail(AG_ERR_LOAD, "feature file truncated: expected at least %llu bytes, got %llu",
                    (unsigned long long)(off + n * row), (unsigned long long)file_size);
    out->n = n; out->dim = dim; out->offset = off; out->dtype = tag;
    return AG_OK;
}

ag_features *new_features(int device, uint64_t n, uint64_t begin, uint64_t rows, uint64_t dim, int dtype) {
    ag_features *f = new ag_features();
    f->device = device; f->num_nodes = n; f->row_begin = begin; f->rows = rows; f->dim = dim; f->dtype = dtype;
    return f;
}

int32_t alloc_features(ag_features *f, bool alloc_payload) {
    if (alloc_payload) {
        // a block peers can map with large pages, should the store become a shard of a view
        AG_TRY(alloc_feature_payload(f->device, std::max<uint64_t>(f->rows * f->dim * elem_size(f->dtype), 16), &f->payload,
                                     &f->block));
    }
    if (alloc_payload && f->dtype == AG_I8)
        AG_CUDA(cudaMalloc(&f->scales, std::max<uint64_t>(f->rows * ((f->dim + kQuantBlock - 1) / kQuantBlock) * 4, 16)));
    AG_CUDA(cudaMalloc(&f->err, 32));  // error bits, then the gather counters (internal.h)
    AG_CUDA(cudaMemset(f->err, 0, 32));
    return AG_OK;
}

uint16_t f32_to_bf16_host(float v) {  // features/store.rs:1094-1104
    uint32_t bits;
    memcpy(&bits, &v, 4);
    if (v != v) return (uint16_t)((bits >> 16) | 0x0040u);
    return (uint16_t)((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
}

uint16_t f32_to_f16_host(float v) {  // IEEE RNE, as half::f16::from_f32
    uint32_t x;
    memcpy(&x, &v, 4);
    const uint32_t sign = (x >> 16) & 0x8000u, exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFFu) return (uint16_t)(man ? (sign | 0x7E00u | (man >> 13)) : (sign | 0x7C00u));
    const int e = (int)exp - 112;
    if (e >= 0x1F) return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const uint32_t shift = (uint32_t)(14 - e);
        uint32_t hm = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (hm & 1u))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t hh = ((uint32_t)e << 10) | (man >> 13);
    const uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (hh & 1u))) hh++;
    return (uint16_t)(sign | hh);
}

}  // namespace

// reference: features/store.rs:923-986 (write_feature_file)
extern "C" int32_t ag_features_save(const char *path, const float *features, uint64_t num_nodes, uint64_t dim, int32_t dtype) {
    if (!path || (!features && num_nodes * dim)) return fail(AG_ERR_VALUE, "ag_features_save: null argument");
    if (dtype < 0 || dtype > 2) return fail(AG_ERR_VALUE, "unknown feature dtype tag: %d", dtype);
    AtomicFile f;
    if (!f.open_tmp(path)) return fail(AG_ERR_LOAD, "failed to create feature file %s: %s", path, strerror(errno));
    uint8_t header[kFeatDataOffset] = {0};
    memcpy(header, "AETHFEAT", 8); memcpy(header + 8, &num_nodes, 8); memcpy(header + 16, &dim, 8);
    memcpy(header + 24, &kFeatDataOffset, 8);
    header[32] = (uint8_t)dtype;
    bool ok = write_all(f.fd, header, sizeof header) == 0;
    const uint64_t total = num_nodes * dim;
    if (ok && dtype == AG_F32) ok = write_all(f.fd, features, total * 4) == 0;
    else if (ok) {
        const uint64_t chunk = 1 << 20;
        std::vector<uint16_t> buf(std::min(chunk, std::max<uint64_t>(total, 1)));
        for (uint64_t done = 0; ok && done < total; done += chunk) {
            const uint64_t m = std::min(chunk, total - done);
            for (uint64_t i = 0; i < m; ++i)
                buf[i] = dtype == AG_BF16 ? f32_to_bf16_host(features[done + i]) : f32_to_f16_host(features[done + i]);
            ok = write_all(f.fd, buf.data(), m * 2) == 0;
        }
    }
    if (!ok) { f.abort(); return fail(AG_ERR_LOAD, "failed to write feature file %s: %s", path, strerror(errno)); }
    if (!f.commit()) return fail(AG_ERR_LOAD, "failed to replace %s: %s", path, strerror(errno));
    return AG_OK;
}

extern "C" void ag_features_free(ag_features *f) {
    if (!f) return;
    DeviceGuard guard(f->device);
    if (f->owns_payload) {
        if (f->block) peer_block_free(f->block); else cudaFree(f->payload);
        cudaFree(f->scales);
    }
    for (void *p : f->ipc_opened) if (p) cudaIpcCloseMemHandle(p);
    for (PeerBlock *b : f->peer_opened) if (b) peer_block_free(b);
    if (f->sort) {
        if (f->sort->done) { cudaEventSynchronize(f->sort->done); cudaEventDestroy(f->sort->done); }
        f->sort->scratch.release();
        delete f->sort;
    }
    cudaFree(f->hot_rows); cudaFree(f->hot_slot);
    cudaFree(f->shards);
    cudaFree(f->err);
    delete f;
}

extern "C" int32_t ag_features_load_range(const char *path, int32_t device, uint64_t row_begin, uint64_t row_end, ag_features **out) {
    if (!path || !out) return fail(AG_ERR_VALUE, "ag_features_load: null argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(AG_ERR_LOAD, "failed to open feature file %s: %s", path, strerror(errno));
    struct stat sb;
    if (fstat(fd, &sb) != 0) { close(fd); return fail(AG_ERR_LOAD, "failed to stat feature file"); }
    FeatHeader h{};
    int32_t st = parse_feature_header(fd, (uint64_t)sb.st_size, &h);
    if (st != AG_OK) { close(fd); return st; }
    row_end = std::min(row_end, h.n);
    row_begin = std::min(row_begin, row_end);
    DeviceGuard guard(device);
    if (!guard.ok) { close(fd); return AG_ERR_CUDA; }
    ag_features *f = new_features(device, h.n, row_begin, row_end - row_begin, h.dim, h.dtype);
    st = alloc_features(f, true);
    const uint64_t row = h.dim * elem_size(h.dtype);
    if (st == AG_OK) st = stream_to_device(fd, h.offset + row_begin * row, f->rows * row, f->payload, nullptr);
    close(fd);
    if (st != AG_OK) { ag_features_free(f); return st; }
    *out = f;
    return AG_OK;
}

extern "C" int32_t ag_features_load(const char *path, int32_t device, ag_features **out) {
    return ag_features_load_range(path, device, 0, 0xFFFFFFFFFFFFFFFFull, out);
}

// Shard `rank` of `world` of a feature file.  Range layout: a contiguous block of
// rows.  Cyclic layout: rows rank, rank + world, ...: the file is streamed through
// the pinned bounce buffer in whole multiples of `world` rows and every world-th
// row is picked by a strided copy (cudaMemcpy2D with the host pitch = world rows).
extern "C" int32_t ag_features_load_shard(const char *path, int32_t device, uint32_t rank, uint32_t world, int32_t layout,
                                          ag_features **out) {
    if (!path || !out) return fail(AG_ERR_VALUE, "ag_features_load_shard: null argument");
    if (world == 0 || rank >= world) return fail(AG_ERR_VALUE, "ag_features_load_shard: bad rank %u of %u", rank, world);
    if (layout != AG_SHARD_RANGE && layout != AG_SHARD_CYCLIC) return fail(AG_ERR_VALUE, "unknown shard layout %d", layout);
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(AG_ERR_LOAD, "failed to open feature file %s: %s", path, strerror(errno));
    struct stat sb;
    if (fstat(fd, &sb) != 0) { close(fd); return fail(AG_ERR_LOAD, "failed to stat feature file"); }
    FeatHeader h{};
    int32_t st = parse_feature_header(fd, (uint64_t)sb.st_size, &h);
    if (st != AG_OK) { close(fd); return st; }
    if (layout == AG_SHARD_RANGE || world == 1) {
        close(fd);
        const uint64_t per = (h.n + world - 1) / world;
        return ag_features_load_range(path, device, (uint64_t)rank * per, (uint64_t)rank * per + per, out);
    }
    DeviceGuard guard(device);
    if (!guard.ok) { close(fd); return AG_ERR_CUDA; }
    const uint64_t rows = h.n > rank ? (h.n - rank + world - 1) / world : 0;
    ag_features *f = new_features(device, h.n, rank, rows, h.dim, h.dtype);
    f->row_stride = world;
    st = alloc_features(f, true);
    const uint64_t row = h.dim * elem_size(h.dtype);
    void *pinned = nullptr;
    // rows per chunk: a whole number of `world`-row groups, about 64 MiB
    const uint64_t groups = std::max<uint64_t>(1, (64ull << 20) / std::max<uint64_t>(row * world, 1));
    if (st == AG_OK && rows && row &&
        cudaHostAlloc(&pinned, (size_t)(groups * world * row), cudaHostAllocDefault) != cudaSuccess)
        st = fail(AG_ERR_CUDA, "pinned buffer allocation failed: %s", cudaGetErrorString(cudaGetLastError()));
    for (uint64_t done = 0; st == AG_OK && row && done < rows; done += groups) {
        const uint64_t take = std::min(groups, rows - done);            // shard rows in this chunk
        const uint64_t first = done * world;                            // first file row of the chunk
        const uint64_t file_rows = std::min<uint64_t>(take * world, h.n - first);
        if (!read_exact(fd, pinned, file_rows * row, h.offset + first * row)) { st = fail(AG_ERR_LOAD, "short read in feature payload"); break; }
        if (cudaMemcpy2D(f->payload + done * row, row, (const uint8_t *)pinned + (uint64_t)rank * row, row * world, row, take,
                         cudaMemcpyHostToDevice) != cudaSuccess)
            st = fail(AG_ERR_CUDA, "copy to device failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    if (pinned) cudaFreeHost(pinned);
    close(fd);
    if (st != AG_OK) { ag_features_free(f); return st; }
    *out = f;
    return AG_OK;
}

extern "C" int32_t ag_features_from_memory(const void *payload, uint64_t num_nodes, uint64_t dim, int32_t dtype,
                                           int32_t mem_kind, int32_t device, ag_features **out) {
    if ((!payload && num_nodes * dim) || !out) return fail(AG_ERR_VALUE, "ag_features_from_memory: null argument");
    if (dtype < 0 || dtype > 2) return fail(AG_ERR_VALUE, "unknown feature dtype tag: %d", dtype);
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_features *f = new_features(device, num_nodes, 0, num_nodes, dim, dtype);
    int32_t st = alloc_features(f, true);
    const uint64_t bytes = num_nodes * dim * elem_size(dtype);
    if (st == AG_OK && bytes &&
        cudaMemcpy(f->payload, payload, bytes, mem_kind == AG_MEM_HOST ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice) != cudaSuccess)
        st = fail(AG_ERR_CUDA, "feature upload failed: %s", cudaGetErrorString(cudaGetLastError()));
    if (st != AG_OK) { ag_features_free(f); return st; }
    *out = f;
    return AG_OK;
}

extern "C" int32_t ag_features_from_f32(const float *features, uint64_t num_nodes, uint64_t dim, int32_t dtype,
                                        int32_t mem_kind, int32_t device, ag_features **out) {
    if ((!features && num_nodes * dim) || !out) return fail(AG_ERR_VALUE, "ag_features_from_f32: null argument");
    if (dtype < 0 || dtype > AG_I8) return fail(AG_ERR_VALUE, "unknown feature dtype tag: %d", dtype);
    if (dtype == AG_I8 && dim == 0) return fail(AG_ERR_VALUE, "feature_dim must be non-zero");  // FeatureCodecError::ZeroDim
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_features *f = new_features(device, num_nodes, 0, num_nodes, dim, dtype);
    int32_t st = alloc_features(f, true);
    const uint64_t count = num_nodes * dim;
    float *staged = nullptr;
    uint32_t *bad = nullptr;
    do {
        if (st != AG_OK || count == 0) break;
        const float *src = features;
        if (mem_kind == AG_MEM_HOST) {
            if (cudaMalloc(&staged, count * 4) != cudaSuccess ||
                cudaMemcpy(staged, features, count * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
                st = fail(AG_ERR_CUDA, "feature upload failed: %s", cudaGetErrorString(cudaGetLastError()));
                break;
            }
            src = staged;
        }
        cudaError_t e;
        if (dtype == AG_I8) {
            uint32_t hbad = 0;
            e = cudaMalloc(&bad, 4);
            if (e == cudaSuccess) e = cudaMemset(bad, 0, 4);
            if (e == cudaSuccess) e = launch_encode_i8(src, num_nodes, dim, (int8_t *)f->payload, f->scales, bad, 0);
            if (e == cudaSuccess) e = cudaMemcpy(&hbad, bad, 4, cudaMemcpyDeviceToHost);
            if (e == cudaSuccess && hbad) { st = fail(AG_ERR_VALUE, "feature values must be finite"); break; }  // FeatureCodecError::NotFinite
        } else {
            e = launch_encode(src, f->payload, count, dtype, 0);
        }
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e != cudaSuccess) st = fail(AG_ERR_CUDA, "feature encode failed: %s", cudaGetErrorString(e));
    } while (0);
    cudaFree(staged); cudaFree(bad);
    if (st != AG_OK) { ag_features_free(f); return st; }
    *out = f;
    return AG_OK;
}

extern "C" int32_t ag_features_adopt_device(void *payload_dev, uint64_t num_nodes, uint64_t dim, int32_t dtype,
                                            int32_t device, ag_features **out) {
    if (!payload_dev || !out) return fail(AG_ERR_VALUE, "ag_features_adopt_device: null argument");
    if (dtype < 0 || dtype > AG_I8) return fail(AG_ERR_VALUE, "unknown feature dtype tag: %d", dtype);
    DeviceGuard guard(device);
    if (!guard.ok) return AG_ERR_CUDA;
    ag_features *f = new_features(device, num_nodes, 0, num_nodes, dim, dtype);
    f->payload = (uint8_t *)payload_dev;
    const int32_t st = alloc_features(f, false);
    if (st != AG_OK) { f->owns_payload = false; ag_features_free(f); return st; }
    *out = f;
    return AG_OK;
}

extern "C" int32_t ag_features_info(const ag_features *f, uint64_t *num_nodes, uint64_t *dim, int32_t *dtype,
                                    int32_t *device, uint64_t *row_begin) {
    if (!f) return fail(AG_ERR_VALUE, "ag_features_info: null store");
    if (num_nodes) *num_nodes = f->num_nodes;
    if (dim) *dim = f->dim;
    if (dtype) *dtype = f->dtype;
    if (device) *device = f->device;
    if (row_begin) *row_begin = f->row_begin;
    return AG_OK;
}

extern "C" int32_t ag_features_shard(const ag_features *f, uint64_t *row_begin, uint64_t *rows) {
    if (!f) return fail(AG_ERR_VALUE, "ag_features_shard: null store");
    if (row_begin) *row_begin = f->row_begin;
    if (rows) *rows = f->rows;
    return AG_OK;
}

extern "C" int32_t ag_features_device_ptr(const ag_features *f, const void **payload_dev) {
    if (!f || !payload_dev) return fail(AG_ERR_VALUE, "ag_features_device_ptr: null argument");
    *payload_dev = f->payload;
    return AG_OK;
}

extern "C" int32_t ag_gather(const ag_features *f, const void *ids_dev, int32_t ids_are_i64, uint64_t n,
                             const uint32_t *n_dev, float *out_dev, void *stream) {
    if (!f || (!ids_dev && n) || (!out_dev && n)) return fail(AG_ERR_VALUE, "ag_gather: null argument");
    if (f->row_stride != 1 && !f->shards)
        return fail(AG_ERR_VALUE, "a cyclic shard is read through a sharded view (ag_features_open_sharded / ag_features_view_sharded)");
    if (n == 0) return AG_OK;
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    GatherArgs a{};
    set_gather_source(a, f);
    a.ids = ids_dev; a.ids64 = ids_are_i64; a.n = n; a.n_dev = n_dev; a.out = out_dev;
    const bool aligned = ((uintptr_t)a.payload % 16) == 0 && ((uintptr_t)out_dev % 16) == 0;
    if (f->sort && n >= 2048 && n < (1ull << 23) && sorted_gather_applies(f, a.row_bytes, aligned)) {
        // Remote rows in address order (gather.cu).  The view owns one sort scratch:
        // this call's kernels wait for the previous call's, whatever stream that used.
        cudaStream_t st = (cudaStream_t)stream;
        std::lock_guard<std::mutex> lk(f->sort->m);
        if (!f->sort->done) AG_CUDA(cudaEventCreateWithFlags(&f->sort->done, cudaEventDisableTiming));
        if (f->sort->used) AG_CUDA(cudaStreamWaitEvent(st, f->sort->done, 0));
        if (n > f->sort->scratch.cap && f->sort->used) AG_CUDA(cudaEventSynchronize(f->sort->done));  // about to be freed
        AG_CUDA(launch_gather_sorted(a, nullptr, 1, n, a.row_bytes, a.dim, f->dtype, f, f->sort->scratch, st));
        AG_CUDA(cudaEventRecord(f->sort->done, st));
        f->sort->used = true;
        return AG_OK;
    }
    AG_CUDA(launch_gather(a, f->dtype, (cudaStream_t)stream));
    return AG_OK;
}

extern "C" int32_t ag_features_scales_to_host(const ag_features *f, float *scales) {
    if (!f || !scales) return fail(AG_ERR_VALUE, "ag_features_scales_to_host: null argument");
    if (f->dtype != AG_I8 || !f->scales) return fail(AG_ERR_VALUE, "only the int8 payload carries scales");
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    AG_CUDA(cudaMemcpy(scales, f->scales, f->rows * ((f->dim + kQuantBlock - 1) / kQuantBlock) * 4, cudaMemcpyDeviceToHost));
    return AG_OK;
}

extern "C" int32_t ag_features_gather_stats(const ag_features *f, uint64_t *rows_requested, uint64_t *rows_fetched,
                                            uint64_t *rows_local_copy) {
    if (!f) return fail(AG_ERR_VALUE, "ag_features_gather_stats: null store");
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint64_t h[3] = {0, 0, 0};
    AG_CUDA(cudaMemcpy(h, (const uint8_t *)f->err + 8, 24, cudaMemcpyDeviceToHost));
    if (rows_requested) *rows_requested = h[0];
    if (rows_fetched) *rows_fetched = h[1];
    if (rows_local_copy) *rows_local_copy = h[2];
    return AG_OK;
}

extern "C" int32_t ag_features_check(const ag_features *f) {
    if (!f) return fail(AG_ERR_VALUE, "ag_features_check: null store");
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    uint32_t h = 0;
    AG_CUDA(cudaDeviceSynchronize());
    AG_CUDA(cudaMemcpy(&h, f->err, 4, cudaMemcpyDeviceToHost));
    if (h) {
        cudaMemset(f->err, 0, 4);
        return fail(AG_ERR_VALUE, "a gathered node id is out of bounds (num_nodes=%llu)", (unsigned long long)f->num_nodes);
    }
    return AG_OK;
}

// reference: features/store.rs:691-769 — every id is checked before any row is read.
extern "C" int32_t ag_features_get_batch(const ag_features *f, const int64_t *ids, uint64_t n, float *out) {
    if (!f || (!ids && n) || (!out && n)) return fail(AG_ERR_VALUE, "ag_features_get_batch: null argument");
    if (f->row_stride != 1 && !f->shards)
        return fail(AG_ERR_VALUE, "a cyclic shard is read through a sharded view (ag_features_open_sharded / ag_features_view_sharded)");
    for (uint64_t i = 0; i < n; ++i) {
        if (ids[i] < 0 || (uint64_t)ids[i] > 0xFFFFFFFFull) return fail(AG_ERR_VALUE, "invalid node id: %lld", (long long)ids[i]);
        if ((uint64_t)ids[i] >= f->num_nodes) return fail(AG_ERR_VALUE, "node %lld out of bounds", (long long)ids[i]);
        if ((uint64_t)ids[i] < f->row_begin || (uint64_t)ids[i] >= f->row_begin + f->rows)
            return fail(AG_ERR_VALUE, "node %lld is not held by this shard (rows %llu..%llu)", (long long)ids[i],
                        (unsigned long long)f->row_begin, (unsigned long long)(f->row_begin + f->rows));
    }
    if (n == 0 || f->dim == 0) return AG_OK;
    DeviceGuard guard(f->device);
    if (!guard.ok) return AG_ERR_CUDA;
    int64_t *ids_dev = nullptr;
    float *out_dev = nullptr;
    int32_t st = AG_OK;
    do {
        if (cudaMalloc(&ids_dev, n * 8) != cudaSuccess || cudaMalloc(&out_dev, n * f->dim * 4) != cudaSuccess) {
            st = fail(AG_ERR_CUDA, "out of device memory: %s", cudaGetErrorString(cudaGetLastError()));
            break;
        }
        cudaError_t e = cudaMemcpy(ids_dev, ids, n * 8, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) {
            st = ag_gather(f, ids_dev, 1, n, nullptr, out_dev, nullptr);
            if (st != AG_OK) break;
            e = cudaMemcpy(out, out_dev, n * f->dim * 4, cudaMemcpyDeviceToHost);
        }
        if (e != cudaSuccess) st = fail(AG_ERR_CUDA, "get_batch failed: %s", cudaGetErrorString(e));
    } while (0);
    cudaFree(ids_dev); cudaFree(out_dev);
    return st;
}

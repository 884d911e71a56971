// Device allocations that other GPUs and other processes can map with large pages.
//
// A feature shard that peers read row by row must be mapped into the reader with
// 2 MB pages.  Memory shared through the legacy CUDA IPC handles
// (cudaIpcGetMemHandle / cudaIpcOpenMemHandle) is not: measured on B200 over NVLink,
// random 512-byte rows out of 38 GB of IPC-mapped peer memory arrive at ~31 GB/s and
// even an address-ordered pass costs ~10 ms whatever the number of rows, while the
// same reads out of memory created with cuMemCreate and mapped with cuMemMap run at
// ~765 GB/s, random or ordered.  So every feature payload the library allocates is a
// cuMemCreate allocation that can be exported as a POSIX file descriptor; the
// descriptor travels to the peer process over a unix socket (SCM_RIGHTS), and the
// peer maps it with cuMemImportFromShareableHandle + cuMemMap.
//
// The driver entry points are resolved at run time through the runtime API, so the
// library carries no link-time dependency on the driver and still loads (and lists
// its symbols) on a machine without one.
#include <cuda.h>
#include <errno.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/time.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <random>
#include <thread>

#include "common.cuh"
#include "internal.h"

namespace ag {

namespace {

struct Driver {
    CUresult (*GetGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*Create)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long) = nullptr;
    CUresult (*Release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*Reserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*AddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*Unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t) = nullptr;
    CUresult (*Export)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*Import)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType) = nullptr;
    CUresult (*ErrorString)(CUresult, const char **) = nullptr;
    bool ok = false;
};

template <typename F>
bool resolve(const char *name, F *fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &status) != cudaSuccess || status != cudaDriverEntryPointSuccess || !p) {
        cudaGetLastError();
        return false;
    }
    *fn = reinterpret_cast<F>(p);
    return true;
}

const Driver &driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        d.ok = resolve("cuMemGetAllocationGranularity", &d.GetGranularity) && resolve("cuMemCreate", &d.Create) &&
               resolve("cuMemRelease", &d.Release) && resolve("cuMemAddressReserve", &d.Reserve) &&
               resolve("cuMemAddressFree", &d.AddressFree) && resolve("cuMemMap", &d.Map) && resolve("cuMemUnmap", &d.Unmap) &&
               resolve("cuMemSetAccess", &d.SetAccess) && resolve("cuMemExportToShareableHandle", &d.Export) &&
               resolve("cuMemImportFromShareableHandle", &d.Import) && resolve("cuGetErrorString", &d.ErrorString);
    });
    return d;
}

const char *cu_str(CUresult r) {
    const char *s = nullptr;
    if (driver().ErrorString) driver().ErrorString(r, &s);
    return s ? s : "unknown driver error";
}

#define AG_CU(call, what)                                                                       \
    do {                                                                                        \
        const CUresult r_ = (call);                                                             \
        if (r_ != CUDA_SUCCESS) return fail(AG_ERR_CUDA, "%s failed: %s", what, cu_str(r_));    \
    } while (0)

CUmemAllocationProp props_for(int device) {
    CUmemAllocationProp p{};
    p.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    p.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    p.location.id = device;
    p.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return p;
}

int32_t set_access(CUdeviceptr va, size_t size, int device) {
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    AG_CU(driver().SetAccess(va, size, &acc, 1), "cuMemSetAccess");
    return AG_OK;
}

// What the owner writes behind the 64 bytes of a legacy handle.
struct HandleTail {
    uint32_t kind;    // 0 empty, 1 legacy CUDA IPC handle in the first 64 bytes, 2 file descriptor served on `sock`
    uint32_t pid;
    uint64_t size;    // mapped size of the allocation
    char sock[40];    // abstract unix socket name (without the leading NUL), NUL-terminated
};
static_assert(sizeof(HandleTail) <= AG_IPC_HANDLE_BYTES - 64, "handle tail must fit behind the legacy handle");

socklen_t abstract_addr(const char *name, sockaddr_un *a) {
    memset(a, 0, sizeof(*a));
    a->sun_family = AF_UNIX;
    const size_t n = strlen(name);
    memcpy(a->sun_path + 1, name, n);  // sun_path[0] = 0: abstract namespace, nothing on the file system
    return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool send_fd(int conn, int fd) {
    char byte = 'F';
    iovec iov{&byte, 1};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {0};
    msghdr msg{};
    msg.msg_iov = &iov; msg.msg_iovlen = 1; msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
    cmsghdr *c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET; c->cmsg_type = SCM_RIGHTS; c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
    return sendmsg(conn, &msg, MSG_NOSIGNAL) == 1;
}

int recv_fd(int conn) {
    char byte = 0;
    iovec iov{&byte, 1};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {0};
    msghdr msg{};
    msg.msg_iov = &iov; msg.msg_iovlen = 1; msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
    ssize_t n;
    do { n = recvmsg(conn, &msg, MSG_CMSG_CLOEXEC); } while (n < 0 && errno == EINTR);
    if (n != 1) return -1;
    for (cmsghdr *c = CMSG_FIRSTHDR(&msg); c; c = CMSG_NXTHDR(&msg, c)) {
        if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS && c->cmsg_len >= CMSG_LEN(sizeof(int))) {
            int fd;
            memcpy(&fd, CMSG_DATA(c), sizeof(int));
            return fd;
        }
    }
    return -1;
}

}  // namespace

struct PeerBlock {
    CUdeviceptr va = 0;
    size_t size = 0;
    CUmemGenericAllocationHandle handle = 0;
    int device = 0;
    // owner side, once exported: the descriptor and the thread that hands it out
    std::mutex m;
    int export_fd = -1;
    int listen_fd = -1;
    std::thread server;
    char sock[40] = {0};
};

void *peer_block_ptr(const PeerBlock *b) { return b ? (void *)b->va : nullptr; }

int32_t alloc_feature_payload(int device, size_t bytes, uint8_t **ptr, PeerBlock **block) {
    // AG_FEATURE_ALLOC=cudamalloc: plain device allocations, shared through legacy CUDA
    // IPC handles (kept for A/B measurements and for testing that path)
    static const bool plain = [] {
        const char *v = getenv("AG_FEATURE_ALLOC");
        return v && strcmp(v, "cudamalloc") == 0;
    }();
    *block = nullptr;
    if (plain) {
        AG_CUDA(cudaMalloc(ptr, bytes));
        return AG_OK;
    }
    if (peer_block_alloc(device, bytes, block) == AG_OK) {
        *ptr = (uint8_t *)peer_block_ptr(*block);
        return AG_OK;
    }
    // A driver or a container that does not offer shareable allocations (no virtual memory
    // management, no file-descriptor handles): a plain allocation still works in every
    // respect except that peers have to map it through a legacy IPC handle.  Said once.
    static std::once_flag warned;
    std::call_once(warned, [] {
        fprintf(stderr, "aethergpu: shareable device allocations are unavailable (%s); feature rows fall back to "
                        "cudaMalloc, and shards mapped by other processes to legacy CUDA IPC handles\n", ag_last_error());
    });
    *block = nullptr;
    AG_CUDA(cudaMalloc(ptr, bytes));
    return AG_OK;
}

int32_t peer_block_alloc(int device, size_t bytes, PeerBlock **out) {
    const Driver &d = driver();
    if (!d.ok) return fail(AG_ERR_CUDA, "the CUDA driver does not offer the virtual memory management entry points");
    const CUmemAllocationProp prop = props_for(device);
    size_t gran = 0;
    AG_CU(d.GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    if (gran == 0) gran = 2u << 20;
    const size_t size = (std::max<size_t>(bytes, 1) + gran - 1) / gran * gran;
    PeerBlock *b = new PeerBlock();
    b->device = device; b->size = size;
    CUresult r = d.Create(&b->handle, size, &prop, 0);
    if (r != CUDA_SUCCESS) {
        delete b;
        return fail(AG_ERR_CUDA, "cuMemCreate of %zu bytes on GPU %d failed: %s", size, device, cu_str(r));
    }
    r = d.Reserve(&b->va, size, gran, 0, 0);
    if (r == CUDA_SUCCESS) {
        r = d.Map(b->va, size, 0, b->handle, 0);
        if (r != CUDA_SUCCESS) { d.AddressFree(b->va, size); b->va = 0; }
    }
    if (r != CUDA_SUCCESS) {
        d.Release(b->handle);
        delete b;
        return fail(AG_ERR_CUDA, "mapping %zu bytes on GPU %d failed: %s", size, device, cu_str(r));
    }
    const int32_t st = set_access(b->va, size, device);
    if (st != AG_OK) { peer_block_free(b); return st; }
    *out = b;
    return AG_OK;
}

void peer_block_free(PeerBlock *b) {
    if (!b) return;
    const Driver &d = driver();
    if (b->listen_fd >= 0) {
        shutdown(b->listen_fd, SHUT_RDWR);  // wakes the accept() of the server thread
        if (b->server.joinable()) b->server.join();
        close(b->listen_fd);
    }
    if (b->export_fd >= 0) close(b->export_fd);
    if (b->va) { d.Unmap(b->va, b->size); d.AddressFree(b->va, b->size); }
    if (b->handle) d.Release(b->handle);
    delete b;
}

int32_t peer_block_grant(PeerBlock *b, int reader_device) {
    if (reader_device == b->device) return AG_OK;
    return set_access(b->va, b->size, reader_device);
}

int32_t peer_block_export(PeerBlock *b, void *handle_out) {
    const Driver &d = driver();
    std::lock_guard<std::mutex> lk(b->m);
    if (b->listen_fd < 0) {
        int fd = -1;
        AG_CU(d.Export(&fd, b->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
        std::random_device rd;
        const uint64_t token = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)time(nullptr) << 20);
        snprintf(b->sock, sizeof(b->sock), "aethergpu-%u-%016llx", (unsigned)getpid(), (unsigned long long)token);
        const int ls = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        sockaddr_un addr;
        const socklen_t len = abstract_addr(b->sock, &addr);
        if (ls < 0 || bind(ls, (sockaddr *)&addr, len) != 0 || listen(ls, 16) != 0) {
            const int e = errno;
            if (ls >= 0) close(ls);
            close(fd);
            return fail(AG_ERR_CUDA, "cannot serve the shard's file descriptor on a unix socket: %s", strerror(e));
        }
        b->export_fd = fd; b->listen_fd = ls;
        b->server = std::thread([ls, fd] {
            for (;;) {
                const int c = accept4(ls, nullptr, nullptr, SOCK_CLOEXEC);
                if (c < 0) { if (errno == EINTR || errno == ECONNABORTED) continue; return; }  // shut down
                send_fd(c, fd);
                close(c);
            }
        });
    }
    HandleTail t{};
    t.kind = 2; t.pid = (uint32_t)getpid(); t.size = b->size;
    memcpy(t.sock, b->sock, sizeof(t.sock));
    memset(handle_out, 0, AG_IPC_HANDLE_BYTES);
    memcpy((uint8_t *)handle_out + 64, &t, sizeof(t));
    return AG_OK;
}

int peer_handle_kind(const void *handle) {
    HandleTail t;
    memcpy(&t, (const uint8_t *)handle + 64, sizeof(t));
    return (int)t.kind;
}

void peer_handle_mark_legacy(void *handle) {
    HandleTail t{};
    t.kind = 1; t.pid = (uint32_t)getpid();
    memcpy((uint8_t *)handle + 64, &t, sizeof(t));
}

int32_t peer_block_import(const void *handle, int device, PeerBlock **out) {
    const Driver &d = driver();
    if (!d.ok) return fail(AG_ERR_CUDA, "the CUDA driver does not offer the virtual memory management entry points");
    HandleTail t;
    memcpy(&t, (const uint8_t *)handle + 64, sizeof(t));
    t.sock[sizeof(t.sock) - 1] = 0;
    if (t.kind != 2 || t.size == 0 || t.sock[0] == 0) return fail(AG_ERR_VALUE, "not a shareable shard handle");
    // fetch the descriptor from the owner (bounded: 50 tries 100 ms apart, then a 10 s receive limit)
    int fd = -1, last_errno = 0;
    for (int attempt = 0; attempt < 50 && fd < 0; ++attempt) {
        const int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (s < 0) { last_errno = errno; break; }
        sockaddr_un addr;
        const socklen_t len = abstract_addr(t.sock, &addr);
        timeval tv{10, 0};
        setsockopt(s, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
        if (connect(s, (sockaddr *)&addr, len) == 0) {
            fd = recv_fd(s);
            if (fd < 0) last_errno = errno ? errno : EPROTO;
        } else {
            last_errno = errno;
        }
        close(s);
        if (fd < 0) { timespec ts{0, 100 * 1000 * 1000}; nanosleep(&ts, nullptr); }
    }
    if (fd < 0) return fail(AG_ERR_CUDA, "cannot fetch the shard's file descriptor from process %u: %s", t.pid, strerror(last_errno));
    PeerBlock *b = new PeerBlock();
    b->device = device; b->size = t.size;
    CUresult r = d.Import(&b->handle, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    if (r != CUDA_SUCCESS) { delete b; return fail(AG_ERR_CUDA, "cuMemImportFromShareableHandle failed: %s", cu_str(r)); }
    r = d.Reserve(&b->va, b->size, 2u << 20, 0, 0);
    if (r == CUDA_SUCCESS) {
        r = d.Map(b->va, b->size, 0, b->handle, 0);
        if (r != CUDA_SUCCESS) { d.AddressFree(b->va, b->size); b->va = 0; }
    }
    if (r != CUDA_SUCCESS) {
        d.Release(b->handle);
        delete b;
        return fail(AG_ERR_CUDA, "mapping a peer's shard (%zu bytes) failed: %s", (size_t)t.size, cu_str(r));
    }
    const int32_t st = set_access(b->va, b->size, device);
    if (st != AG_OK) { peer_block_free(b); return st; }
    *out = b;
    return AG_OK;
}

}  // namespace ag

// Symmetric heap: cuMem VMM allocations exchanged between the ranks' processes as POSIX file
// descriptors over abstract unix datagram sockets (SCM_RIGHTS), mapped peer-to-peer.
#include "symm_heap.h"

#include <errno.h>
#include <poll.h>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <mutex>

#include "ptx.cuh"

namespace cb {

static thread_local char g_err[512] = "";
const char *last_error() { return g_err; }
void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

// ----------------------------------------------------------------- driver API ----
static DriverApi g_api;
static std::once_flag g_api_once;
static std::string g_api_why;

template <typename F>
static bool resolve(F &fn, const char *name) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        g_api_why = std::string("cannot resolve ") + name + ": " + cudaGetErrorString(e);
        (void)cudaGetLastError();
        return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
}

const DriverApi *driver_api(std::string *why) {
    std::call_once(g_api_once, [] {
        bool ok = resolve(g_api.MemCreate, "cuMemCreate") && resolve(g_api.MemRelease, "cuMemRelease") &&
                  resolve(g_api.MemAddressReserve, "cuMemAddressReserve") &&
                  resolve(g_api.MemAddressFree, "cuMemAddressFree") && resolve(g_api.MemMap, "cuMemMap") &&
                  resolve(g_api.MemUnmap, "cuMemUnmap") && resolve(g_api.MemSetAccess, "cuMemSetAccess") &&
                  resolve(g_api.MemExportToShareableHandle, "cuMemExportToShareableHandle") &&
                  resolve(g_api.MemImportFromShareableHandle, "cuMemImportFromShareableHandle") &&
                  resolve(g_api.MemGetAllocationGranularity, "cuMemGetAllocationGranularity") &&
                  resolve(g_api.TensorMapEncodeTiled, "cuTensorMapEncodeTiled") &&
                  resolve(g_api.GetErrorString, "cuGetErrorString");
        g_api.loaded = ok;
        if (ok) {      // optional entry points: all or nothing
            const bool mc = resolve(g_api.DeviceGet, "cuDeviceGet") && resolve(g_api.DeviceGetAttribute, "cuDeviceGetAttribute") &&
                            resolve(g_api.MulticastCreate, "cuMulticastCreate") &&
                            resolve(g_api.MulticastAddDevice, "cuMulticastAddDevice") &&
                            resolve(g_api.MulticastBindMem, "cuMulticastBindMem") &&
                            resolve(g_api.MulticastUnbind, "cuMulticastUnbind") &&
                            resolve(g_api.MulticastGetGranularity, "cuMulticastGetGranularity");
            if (!mc) g_api.MulticastCreate = nullptr;
        }
    });
    if (!g_api.loaded) {
        if (why) *why = g_api_why;
        return nullptr;
    }
    return &g_api;
}

static const char *cu_err(const DriverApi *api, CUresult r) {
    const char *s = nullptr;
    api->GetErrorString(r, &s);
    return s ? s : "unknown";
}

#define CU_TRY(call)                                                                    \
    do {                                                                                \
        CUresult _r = (call);                                                           \
        if (_r != CUDA_SUCCESS) {                                                       \
            set_error("%s failed: %s (%s:%d)", #call, cu_err(api, _r), __FILE__, __LINE__); \
            return CATCCOS_ERR_CUDA;                                                    \
        }                                                                               \
    } while (0)
#define RT_TRY(call)                                                                          \
    do {                                                                                      \
        cudaError_t _e = (call);                                                              \
        if (_e != cudaSuccess) {                                                              \
            set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(_e), __FILE__, __LINE__); \
            return CATCCOS_ERR_CUDA;                                                          \
        }                                                                                     \
    } while (0)

static bool multicast_requested() {
    const char *e = getenv("CATCCOS_MULTICAST");
    return e && atoi(e) != 0;
}

// ------------------------------------------------------------------- the team ----
static Team *g_team = nullptr;
Team *team() { return g_team; }

static double now_s() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + ts.tv_nsec * 1e-9;
}

// --------------------------------------------------------------- host messages ----
struct Msg {
    uint32_t magic;
    int32_t type;   // 1 = heap handle, 2 = barrier
    int32_t from;
    uint32_t seq;
};
constexpr uint32_t kMagic = 0xCA7CC05u;
constexpr double kBootstrapTimeoutS = 120.0;

static void make_addr(const std::string &prefix, int pe, sockaddr_un *addr, socklen_t *len) {
    memset(addr, 0, sizeof(*addr));
    addr->sun_family = AF_UNIX;
    std::string name = prefix + "." + std::to_string(pe);
    if (name.size() > sizeof(addr->sun_path) - 2) name.resize(sizeof(addr->sun_path) - 2);
    addr->sun_path[0] = '\0';   // abstract namespace: no file system entry, vanishes with the process
    memcpy(addr->sun_path + 1, name.data(), name.size());
    *len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

static int send_msg(Team *t, int to, const Msg &m, int fd) {
    sockaddr_un addr;
    socklen_t alen;
    make_addr(t->sock_prefix, to, &addr, &alen);
    msghdr mh;
    memset(&mh, 0, sizeof(mh));
    iovec iov{const_cast<Msg *>(&m), sizeof(m)};
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    mh.msg_name = &addr;
    mh.msg_namelen = alen;
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
    if (fd >= 0) {
        memset(ctrl, 0, sizeof(ctrl));
        mh.msg_control = ctrl;
        mh.msg_controllen = sizeof(ctrl);
        cmsghdr *c = CMSG_FIRSTHDR(&mh);
        c->cmsg_level = SOL_SOCKET;
        c->cmsg_type = SCM_RIGHTS;
        c->cmsg_len = CMSG_LEN(sizeof(int));
        memcpy(CMSG_DATA(c), &fd, sizeof(int));
    }
    const double t0 = now_s();
    while (true) {
        ssize_t n = sendmsg(t->sock, &mh, MSG_DONTWAIT);
        if (n == static_cast<ssize_t>(sizeof(m))) return CATCCOS_OK;
        // peer not bound yet (ECONNREFUSED / ENOENT) or its queue is full (EAGAIN): retry, bounded
        if (errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR) {
            set_error("sendmsg to PE %d failed: %s", to, strerror(errno));
            return CATCCOS_ERR_BOOTSTRAP;
        }
        if (now_s() - t0 > kBootstrapTimeoutS) {
            set_error("rendezvous with PE %d timed out after %.0f s (%s)", to, kBootstrapTimeoutS, strerror(errno));
            return CATCCOS_ERR_BOOTSTRAP;
        }
        usleep(2000);
    }
}

// Receives until a message of (type, seq) from every other PE has been seen; other messages are
// parked in t->pending.  fds_out[pe] receives the descriptor carried by type-1 messages.
static int recv_all(Team *t, int type, uint32_t seq, int *fds_out) {
    std::vector<bool> got(t->n_pes, false);
    got[t->my_pe] = true;
    int missing = t->n_pes - 1;
    for (auto it = t->pending.begin(); it != t->pending.end();) {
        if (it->type == type && it->seq == seq && !got[it->from]) {
            got[it->from] = true;
            if (fds_out) fds_out[it->from] = it->fd;
            --missing;
            it = t->pending.erase(it);
        } else {
            ++it;
        }
    }
    const double t0 = now_s();
    while (missing > 0) {
        pollfd pfd{t->sock, POLLIN, 0};
        int pr = poll(&pfd, 1, 200);
        if (pr < 0 && errno != EINTR) {
            set_error("poll failed: %s", strerror(errno));
            return CATCCOS_ERR_BOOTSTRAP;
        }
        if (pr <= 0) {
            if (now_s() - t0 > kBootstrapTimeoutS) {
                set_error("waiting for %d peer message(s) of type %d timed out after %.0f s", missing, type,
                          kBootstrapTimeoutS);
                return CATCCOS_ERR_BOOTSTRAP;
            }
            continue;
        }
        Msg m;
        msghdr mh;
        memset(&mh, 0, sizeof(mh));
        iovec iov{&m, sizeof(m)};
        mh.msg_iov = &iov;
        mh.msg_iovlen = 1;
        alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
        mh.msg_control = ctrl;
        mh.msg_controllen = sizeof(ctrl);
        ssize_t n = recvmsg(t->sock, &mh, MSG_DONTWAIT);
        if (n < 0) {
            if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) continue;
            set_error("recvmsg failed: %s", strerror(errno));
            return CATCCOS_ERR_BOOTSTRAP;
        }
        if (n != static_cast<ssize_t>(sizeof(m)) || m.magic != kMagic || m.from < 0 || m.from >= t->n_pes) continue;
        int fd = -1;
        for (cmsghdr *c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c))
            if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) memcpy(&fd, CMSG_DATA(c), sizeof(int));
        if (m.type == type && m.seq == seq && !got[m.from]) {
            got[m.from] = true;
            if (fds_out) fds_out[m.from] = fd;
            --missing;
        } else {
            t->pending.push_back({m.type, m.from, m.seq, fd});
        }
    }
    return CATCCOS_OK;
}

int team_host_barrier() {
    Team *t = g_team;
    if (!t) {
        set_error("symmetric heap not initialised");
        return CATCCOS_ERR_NOT_INIT;
    }
    if (t->emulated || t->n_pes == 1) return CATCCOS_OK;
    const uint32_t seq = ++t->barrier_seq;
    Msg m{kMagic, 2, t->my_pe, seq};
    for (int pe = 0; pe < t->n_pes; ++pe) {
        if (pe == t->my_pe) continue;
        int rc = send_msg(t, pe, m, -1);
        if (rc) return rc;
    }
    return recv_all(t, 2, seq, nullptr);
}

// ------------------------------------------------------------------- creation ----
static int alloc_local(const DriverApi *api, Team *t, int device, size_t bytes, CUmemGenericAllocationHandle *h,
                       bool shareable) {
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = shareable ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
    CU_TRY(api->MemCreate(h, bytes, &prop, 0));
    (void)t;
    return CATCCOS_OK;
}

static int map_handle(const DriverApi *api, int device, size_t bytes, CUmemGenericAllocationHandle h, uint8_t **va) {
    CUdeviceptr ptr = 0;
    CU_TRY(api->MemAddressReserve(&ptr, bytes, 0, 0, 0));
    CU_TRY(api->MemMap(ptr, bytes, 0, h, 0));
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CU_TRY(api->MemSetAccess(ptr, bytes, &acc, 1));
    *va = reinterpret_cast<uint8_t *>(ptr);
    return CATCCOS_OK;
}

static int common_setup(Team *t, uint64_t local_mem_size, const DriverApi **api_out) {
    std::string why;
    const DriverApi *api = driver_api(&why);
    if (!api) {
        set_error("CUDA driver unavailable: %s", why.c_str());
        return CATCCOS_ERR_CUDA;
    }
    RT_TRY(cudaFree(0));
    RT_TRY(cudaGetDevice(&t->device));
    RT_TRY(cudaDeviceGetAttribute(&t->num_sms, cudaDevAttrMultiProcessorCount, t->device));
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = t->device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    CU_TRY(api->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if (gran == 0) gran = 2u << 20;
    const size_t want = static_cast<size_t>(local_mem_size) + kFlagBytes;
    if (multicast_requested() && api->MulticastCreate && t->n_pes > 1) {
        // the whole heap is bound to the multicast object: its size has to be a multiple of that granularity too
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = static_cast<unsigned>(t->n_pes);
        mp.size = (want + gran - 1) / gran * gran;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg = 0;
        if (api->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    t->heap_bytes = (want + gran - 1) / gran * gran;
    // status words followed by the tile-queue counters of the fused kernels (two per local rank)
    RT_TRY(cudaMalloc(&t->status_dev, (ST_WORDS + 2 * kMaxRanks) * sizeof(int)));
    RT_TRY(cudaMemset(t->status_dev, 0, (ST_WORDS + 2 * kMaxRanks) * sizeof(int)));
    t->sched_dev = t->status_dev + ST_WORDS;
    if (const char *e = getenv("CATCCOS_WAIT_TIMEOUT_MS")) {
        const long ms = atol(e);
        if (ms > 0) t->timeout_ns = static_cast<uint64_t>(ms) * 1000000ull;
    }
    *api_out = api;
    return CATCCOS_OK;
}

// Releases this PE's part of the multicast object: the mapping, then the binding of its heap.  No host barrier:
// also runs from the exit handler of a process that leaves without catccos_shmem_finalize.
static void release_multicast(const DriverApi *api, Team *t) {
    if (!t->mc_handle) return;
    cudaDeviceSynchronize();
    if (t->mc_base) {
        api->MemUnmap(reinterpret_cast<CUdeviceptr>(t->mc_base), t->heap_bytes);
        api->MemAddressFree(reinterpret_cast<CUdeviceptr>(t->mc_base), t->heap_bytes);
        t->mc_base = nullptr;
    }
    CUdevice dev;
    if (api->DeviceGet(&dev, t->device) == CUDA_SUCCESS) api->MulticastUnbind(t->mc_handle, dev, 0, t->heap_bytes);
    api->MemRelease(t->mc_handle);
    t->mc_handle = 0;
}
static void multicast_exit_handler() {
    if (g_team && g_team->mc_handle) {
        const DriverApi *api = driver_api();
        if (api) release_multicast(api, g_team);
    }
}

// One multicast object over all PEs' heaps (PE 0 creates it, the others import it), every PE binds its heap at
// offset 0 and maps the object: t->mc_base.  Collective; needs g_team for the host barrier.
static int setup_multicast(const DriverApi *api, Team *t) {
    if (!api->MulticastCreate) {
        set_error("CATCCOS_MULTICAST=1: the driver has no multicast objects");
        return CATCCOS_ERR_CUDA;
    }
    CUdevice dev;
    CU_TRY(api->DeviceGet(&dev, t->device));
    int supported = 0;
    CU_TRY(api->DeviceGetAttribute(&supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev));
    if (!supported) {
        set_error("CATCCOS_MULTICAST=1: device %d does not support multicast objects", t->device);
        return CATCCOS_ERR_CUDA;
    }
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(t->n_pes);
    mp.size = t->heap_bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    int fd = -1;
    if (t->my_pe == 0) {
        CU_TRY(api->MulticastCreate(&t->mc_handle, &mp));
        CU_TRY(api->MemExportToShareableHandle(&fd, t->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    }
    // every PE sends a type-3 message to every peer; PE 0's carries the object's descriptor
    Msg m{kMagic, 3, t->my_pe, 0};
    for (int pe = 0; pe < t->n_pes; ++pe) {
        if (pe == t->my_pe) continue;
        int rc = send_msg(t, pe, m, fd);
        if (rc) return rc;
    }
    int fds[kMaxRanks];
    for (int i = 0; i < kMaxRanks; ++i) fds[i] = -1;
    int rc = recv_all(t, 3, 0, fds);
    if (rc) return rc;
    if (fd >= 0) close(fd);
    if (t->my_pe != 0) {
        if (fds[0] < 0) {
            set_error("PE 0 sent no multicast handle");
            return CATCCOS_ERR_BOOTSTRAP;
        }
        CU_TRY(api->MemImportFromShareableHandle(&t->mc_handle, reinterpret_cast<void *>(static_cast<intptr_t>(fds[0])),
                                                 CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    }
    for (int pe = 0; pe < t->n_pes; ++pe)
        if (fds[pe] >= 0) close(fds[pe]);
    CU_TRY(api->MulticastAddDevice(t->mc_handle, dev));
    if ((rc = team_host_barrier())) return rc;          // every device is in before anyone binds
    CU_TRY(api->MulticastBindMem(t->mc_handle, 0, t->handles[t->my_pe], 0, t->heap_bytes, 0));
    if ((rc = team_host_barrier())) return rc;
    size_t mg = 0;
    CU_TRY(api->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
    CUdeviceptr ptr = 0;
    CU_TRY(api->MemAddressReserve(&ptr, t->heap_bytes, mg, 0, 0));
    CU_TRY(api->MemMap(ptr, t->heap_bytes, 0, t->mc_handle, 0));
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = t->device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CU_TRY(api->MemSetAccess(ptr, t->heap_bytes, &acc, 1));
    t->mc_base = reinterpret_cast<uint8_t *>(ptr);
    static bool registered = false;
    if (!registered) {
        registered = true;
        atexit(multicast_exit_handler);
    }
    return team_host_barrier();
}

int team_init_emulated(int n_pes, uint64_t local_mem_size) {
    if (g_team) {
        set_error("symmetric heap already initialised");
        return CATCCOS_ERR_INVALID;
    }
    if (n_pes < 1 || n_pes > kMaxRanks) {
        set_error("n_pes must be in [1,%d]", kMaxRanks);
        return CATCCOS_ERR_INVALID;
    }
    Team *t = new Team();
    t->my_pe = 0;
    t->n_pes = n_pes;
    t->emulated = true;
    const DriverApi *api = nullptr;
    int rc = common_setup(t, local_mem_size, &api);
    if (rc) {
        delete t;
        return rc;
    }
    for (int pe = 0; pe < n_pes; ++pe) {
        rc = alloc_local(api, t, t->device, t->heap_bytes, &t->handles[pe], false);
        if (!rc) rc = map_handle(api, t->device, t->heap_bytes, t->handles[pe], &t->base[pe]);
        if (rc) return rc;
        RT_TRY(cudaMemset(t->base[pe], 0, kFlagBytes));
    }
    RT_TRY(cudaDeviceSynchronize());
    g_team = t;
    return CATCCOS_OK;
}

int team_init(int my_pe, int n_pes, uint64_t local_mem_size, const char *ip_port) {
    if (g_team) {
        set_error("symmetric heap already initialised");
        return CATCCOS_ERR_INVALID;
    }
    if (n_pes < 1 || n_pes > kMaxRanks || my_pe < 0 || my_pe >= n_pes) {
        set_error("bad PE numbering: my_pe=%d n_pes=%d (max %d)", my_pe, n_pes, kMaxRanks);
        return CATCCOS_ERR_INVALID;
    }
    // Same rule as the reference's set_attr(): an empty rendezvous string is an invalid value.
    if (ip_port == nullptr || ip_port[0] == '\0') {
        set_error("ip_port must not be empty");
        return CATCCOS_ERR_INVALID;
    }
    Team *t = new Team();
    t->my_pe = my_pe;
    t->n_pes = n_pes;
    const DriverApi *api = nullptr;
    int rc = common_setup(t, local_mem_size, &api);
    if (rc) {
        delete t;
        return rc;
    }
    rc = alloc_local(api, t, t->device, t->heap_bytes, &t->handles[my_pe], n_pes > 1);
    if (!rc) rc = map_handle(api, t->device, t->heap_bytes, t->handles[my_pe], &t->base[my_pe]);
    if (rc) return rc;
    RT_TRY(cudaMemset(t->base[my_pe], 0, kFlagBytes));
    RT_TRY(cudaDeviceSynchronize());

    if (n_pes > 1) {
        t->sock_prefix = std::string("catccos_b200:") + ip_port;
        t->sock = socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
        if (t->sock < 0) {
            set_error("socket() failed: %s", strerror(errno));
            return CATCCOS_ERR_BOOTSTRAP;
        }
        sockaddr_un addr;
        socklen_t alen;
        make_addr(t->sock_prefix, my_pe, &addr, &alen);
        if (bind(t->sock, reinterpret_cast<sockaddr *>(&addr), alen) != 0) {
            set_error("bind of rendezvous socket for PE %d failed: %s", my_pe, strerror(errno));
            return CATCCOS_ERR_BOOTSTRAP;
        }
        int fd = -1;
        CU_TRY(api->MemExportToShareableHandle(&fd, t->handles[my_pe], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        Msg m{kMagic, 1, my_pe, 0};
        for (int pe = 0; pe < n_pes; ++pe) {
            if (pe == my_pe) continue;
            rc = send_msg(t, pe, m, fd);
            if (rc) return rc;
        }
        int fds[kMaxRanks];
        for (int i = 0; i < kMaxRanks; ++i) fds[i] = -1;
        rc = recv_all(t, 1, 0, fds);
        if (rc) return rc;
        close(fd);
        for (int pe = 0; pe < n_pes; ++pe) {
            if (pe == my_pe) continue;
            if (fds[pe] < 0) {
                set_error("PE %d sent no memory handle", pe);
                return CATCCOS_ERR_BOOTSTRAP;
            }
            CU_TRY(api->MemImportFromShareableHandle(&t->handles[pe], reinterpret_cast<void *>(static_cast<intptr_t>(fds[pe])),
                                                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
            close(fds[pe]);
            rc = map_handle(api, t->device, t->heap_bytes, t->handles[pe], &t->base[pe]);
            if (rc) return rc;
        }
    }
    g_team = t;
    // nobody may touch a peer's flags before that peer has zeroed them
    rc = team_host_barrier();
    if (!rc && n_pes > 1 && multicast_requested()) rc = setup_multicast(api, t);
    return rc;
}

int team_finalize() {
    Team *t = g_team;
    if (!t) return CATCCOS_OK;
    const DriverApi *api = driver_api();
    cudaDeviceSynchronize();
    team_host_barrier();   // peers may still be reading this PE's memory
    if (api && t->mc_handle) {
        release_multicast(api, t);
        team_host_barrier();   // every PE has unbound its heap before any heap is released
    }
    if (api) {
        for (int pe = 0; pe < t->n_pes; ++pe) {
            if (t->base[pe]) {
                api->MemUnmap(reinterpret_cast<CUdeviceptr>(t->base[pe]), t->heap_bytes);
                api->MemAddressFree(reinterpret_cast<CUdeviceptr>(t->base[pe]), t->heap_bytes);
            }
            if (t->handles[pe]) api->MemRelease(t->handles[pe]);
        }
    }
    if (t->status_dev) cudaFree(t->status_dev);
    if (t->sock >= 0) close(t->sock);
    for (auto &p : t->pending)
        if (p.fd >= 0) close(p.fd);
    delete t;
    g_team = nullptr;
    return CATCCOS_OK;
}

void *team_malloc(size_t bytes) {
    Team *t = g_team;
    if (!t) {
        set_error("symmetric heap not initialised");
        return nullptr;
    }
    const size_t aligned = (bytes + 1023) / 1024 * 1024;
    if (t->bump + aligned > t->heap_bytes - t->top_reserved) {
        set_error("symmetric heap exhausted: %zu bytes requested, %zu left", bytes,
                  t->heap_bytes - t->top_reserved - t->bump);
        return nullptr;
    }
    void *p = t->base[t->my_pe] + t->bump;
    t->alloc_stack.push_back(t->bump);
    t->bump += aligned;
    return p;
}

// A region at the END of the heap, outside the bump stack that catccos_shmem_malloc/free drive, for
// library-internal buffers (the host-buffer entry point).  Collective like team_malloc: every PE
// asks for the same size in the same order.  Grows in place (same end, lower start); never shrinks.
void *team_top_region(size_t bytes) {
    Team *t = g_team;
    if (!t) {
        set_error("symmetric heap not initialised");
        return nullptr;
    }
    const size_t aligned = (bytes + 1023) / 1024 * 1024;
    if (aligned > t->top_reserved) {
        if (t->bump + aligned > t->heap_bytes) {
            set_error("symmetric heap exhausted: %zu bytes needed at the top, %zu free", bytes, t->heap_bytes - t->bump);
            return nullptr;
        }
        t->top_reserved = aligned;
    }
    return t->base[t->my_pe] + (t->heap_bytes - t->top_reserved);
}

int team_free(void *p) {
    Team *t = g_team;
    if (!t) return CATCCOS_ERR_NOT_INIT;
    const size_t off = static_cast<size_t>(static_cast<uint8_t *>(p) - t->base[t->my_pe]);
    for (size_t i = 0; i < t->alloc_stack.size(); ++i) {
        if (t->alloc_stack[i] == off) {
            t->alloc_stack.resize(i);
            t->bump = off;
            return CATCCOS_OK;
        }
    }
    set_error("pointer %p was not returned by catccos_shmem_malloc", p);
    return CATCCOS_ERR_INVALID;
}

void *team_ptr(const void *local, int pe) {
    Team *t = g_team;
    if (!t || pe < 0 || pe >= t->n_pes) return nullptr;
    const uint8_t *p = static_cast<const uint8_t *>(local);
    const uint8_t *b = t->base[t->my_pe];
    if (p < b || p >= b + t->heap_bytes) return nullptr;
    return t->base[pe] + (p - b);
}

int team_read_status(int *out) {
    Team *t = g_team;
    if (!t) return CATCCOS_ERR_NOT_INIT;
    RT_TRY(cudaMemcpy(out, t->status_dev, ST_WORDS * sizeof(int), cudaMemcpyDeviceToHost));
    return CATCCOS_OK;
}

int team_reset_status() {
    Team *t = g_team;
    if (!t) return CATCCOS_ERR_NOT_INIT;
    // also the tile-queue counters: a launch that gave up may have left them non-zero
    RT_TRY(cudaMemset(t->status_dev, 0, (ST_WORDS + 2 * kMaxRanks) * sizeof(int)));
    return CATCCOS_OK;
}

}  // namespace cb

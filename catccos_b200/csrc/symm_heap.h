// Symmetric heap over cuMem VMM: every PE owns one physical allocation, exports it as a POSIX
// file descriptor, and maps every peer's allocation into its own address space (NVLink P2P).
// Replaces the ACLSHMEM heap the reference initialises with set_attr()/aclshmemx_init_attr()
// (utils/shmem_init.h:16-39) and the shmem_malloc/shmem_ptr/shmem_free calls of its drivers
// (examples/matmul_allreduce/main.cpp:122-135,173-178).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/catccos_b200.h"   // error codes
#include "common.h"

namespace cb {

// Driver entry points, resolved at run time through the CUDA runtime so that the library loads
// on machines without a driver (build and symbol checks) and needs no link against libcuda.
struct DriverApi {
    CUresult (*MemCreate)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*MemExportToShareableHandle)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                           unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
    CUresult (*MemGetAllocationGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
    CUresult (*TensorMapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                     const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                     CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                     CUtensorMapFloatOOBfill);
    CUresult (*GetErrorString)(CUresult, const char **);
    // NVSwitch multicast objects (optional: null when the driver has none)
    CUresult (*DeviceGet)(CUdevice *, int) = nullptr;
    CUresult (*DeviceGetAttribute)(int *, CUdevice_attribute, CUdevice) = nullptr;
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle *, const CUmulticastObjectProp *) = nullptr;
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                                 unsigned long long) = nullptr;
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
    CUresult (*MulticastGetGranularity)(size_t *, const CUmulticastObjectProp *, CUmulticastGranularity_flags) = nullptr;
    bool loaded = false;
};
// Returns nullptr (and sets *why) when no driver is available.
const DriverApi *driver_api(std::string *why = nullptr);


struct Team {
    int my_pe = 0;
    int n_pes = 1;
    bool emulated = false;         // all PEs are regions on the current device of this process
    int device = 0;
    int num_sms = 0;
    size_t heap_bytes = 0;         // per PE, flag region included
    size_t bump = kFlagBytes;      // next free byte of the (symmetric) bump allocator
    std::vector<size_t> alloc_stack;   // offsets of live allocations, in order
    size_t top_reserved = 0;       // bytes at the end of the heap held by team_top_region (not part of the stack)
    uint8_t *base[kMaxRanks] = {};
    CUmemGenericAllocationHandle handles[kMaxRanks] = {};
    // NVSwitch multicast view of all heaps (CATCCOS_MULTICAST=1, one process per PE): a store to mc_base + offset
    // lands at that offset of EVERY PE's heap.  Written with multimem.st only, never read.
    uint8_t *mc_base = nullptr;
    CUmemGenericAllocationHandle mc_handle = 0;
    uint32_t epoch = 0;            // launches so far; identical on all PEs by collective-call order
    int *status_dev = nullptr;     // StatusWord[ST_WORDS]
    int *sched_dev = nullptr;      // tile-queue counters: {next tile, pairs finished} per local rank, zero between launches
    uint64_t timeout_ns = 10ull * 1000 * 1000 * 1000;
    unsigned long long *trace_dev = nullptr;   // optional per-CTA trace buffer (catccos_debug_set_trace)
    uint32_t debug_flags = 0;      // bit 0: compute-only launches (exposed-communication measurement)
    // double-buffered operator regions (see next_slot)
    uint64_t last_sig = 0;
    uint32_t last_sig_epoch = 0;
    int last_half = 0;
    // host rendezvous
    int sock = -1;
    std::string sock_prefix;
    uint32_t barrier_seq = 0;
    struct Pending { int type; int from; uint32_t seq; int fd; };
    std::vector<Pending> pending;
};

// The dense and MXFP8 operators keep two copies ("halves") of their symmetric data region and
// alternate between them when the same operator is launched back to back with the same shape and
// buffer.  A rank may then write into a peer's half as soon as that peer has ENTERED the previous
// launch (which, in stream order, means it has finished the launch before that one, the last
// reader of this half); otherwise it has to wait until the peer has entered this launch.  Ranks
// that run ahead or behind by up to one launch no longer stall one another.
struct LaunchSlot {
    int half;                // which half this launch uses
    uint32_t entered_need;   // peers must have entered this epoch before their half is overwritten
};
inline LaunchSlot peek_slot(const Team *t, uint64_t sig, uint32_t epoch) {
    LaunchSlot s;
    if (sig == t->last_sig && t->last_sig_epoch + 1 == epoch) {
        s.half = t->last_half ^ 1;
        s.entered_need = epoch - 1;
    } else {
        s.half = 0;
        s.entered_need = epoch;
    }
    return s;
}
// called once nothing can stop the launch any more: consumes the epoch and records the slot
inline void commit_slot(Team *t, uint64_t sig, uint32_t epoch, const LaunchSlot &s) {
    t->epoch = epoch;
    t->last_sig = sig;
    t->last_sig_epoch = epoch;
    t->last_half = s.half;
}
inline uint64_t slot_sig(uint64_t h, uint64_t v) { return (h ^ v) * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull; }

Team *team();                       // the process-wide team, nullptr before init
int team_init(int my_pe, int n_pes, uint64_t local_mem_size, const char *ip_port);
int team_init_emulated(int n_pes, uint64_t local_mem_size);
int team_finalize();
void *team_malloc(size_t bytes);    // collective: same offset on every PE; nullptr when exhausted
int team_free(void *p);             // stack discipline: frees p and everything allocated after it
void *team_top_region(size_t bytes);   // collective: library-internal region at the end of the heap, outside the stack
int team_host_barrier();
void *team_ptr(const void *local, int pe);
int team_read_status(int *out_words /* ST_WORDS */);
int team_reset_status();
const char *last_error();
void set_error(const char *fmt, ...);

}  // namespace cb

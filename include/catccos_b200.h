/*
 * C-ABI of the B200 implementation of the fused compute-communication operators.
 *
 * Plain C: pointers and sizes only.  Every function returns 0 on success or one of the
 * CATCCOS_ERR_* codes; catccos_last_error() gives the message of the last failure on the calling
 * thread.  Device pointers are ordinary CUDA device pointers of the calling process; `symmetric`
 * pointers come from catccos_shmem_malloc().  One process per GPU, one rank ("PE") per process;
 * all ranks call the collective entry points with the same shapes in the same order (the
 * reference's rule too: nothing checks it).
 *
 * Each declaration names the reference interface it replaces (paths relative to the reference
 * project root).
 */
#ifndef CATCCOS_B200_H
#define CATCCOS_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define CATCCOS_API __attribute__((visibility("default")))
#else
#define CATCCOS_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

enum {
    CATCCOS_OK = 0,
    CATCCOS_ERR_INVALID = 1,     /* bad argument, unsupported shape or layout */
    CATCCOS_ERR_NOT_INIT = 2,    /* catccos_shmem_init has not been called */
    CATCCOS_ERR_CUDA = 3,        /* a CUDA call failed, or no driver/GPU is present */
    CATCCOS_ERR_BOOTSTRAP = 4,   /* rendezvous with the peer processes failed or timed out */
    CATCCOS_ERR_NOMEM = 5,
    CATCCOS_ERR_DEVICE_WAIT = 6, /* a device-side wait ran out: see catccos_last_status */
    CATCCOS_ERR_RANGE = 7        /* a partial product of Matmul-ReduceScatter / AllReduce left the fp16 range of the
                                    exchange format (see CATCCOS_RS_EXCHANGE): the result is not valid */
};

/* utils/info.h:95-114 — same 17 fields, same order. */
typedef struct CocTilingParams {
    uint32_t m, k, n;
    uint32_t transA, transB;
    uint32_t m0, k0, n0;
    uint32_t commTileM, commInterval, commNpuSplit, commDataSplit, commBlockM;
    uint32_t rankSize, epSize, expertNum, topK;
} CocTilingParams;

/* utils/info.h:123-167 (KernelParams) without the C++ members.  customPtrs order per operator is
 * the reference's: MXFP8 AllGather-Matmul {aScale, bScale}; MoE {b2, expertIdx, probs, bScale, b2Scale}. */
typedef struct CatccosKernelParams {
    uint8_t *ptrA;
    uint8_t *ptrB;
    uint8_t *ptrC;
    uint8_t **customPtrs;
    uint32_t customCount;
} CatccosKernelParams;

/* utils/info.h:46-93: values of CocCommType / CocDataType used by this library. */
enum {
    CATCCOS_MATMUL_ALLREDUCE = 0,
    CATCCOS_ALLGATHER_MATMUL = 1,
    CATCCOS_ASCEND950_ALLGATHER_MATMUL = 2,
    CATCCOS_MATMUL_REDUCE_SCATTER = 3,
    CATCCOS_ASCEND950_MATMUL_REDUCE_SCATTER = 4,
    CATCCOS_ALLGATHER_MATMUL_WITH_GATHER_RESULT = 5,
    CATCCOS_ASCEND950_MXFP8_MATMUL_REDUCE_SCATTER = 18,
    CATCCOS_ASCEND950_MXFP8_MATMUL_ALLTOALL = 19,
    CATCCOS_ALLGATHER_MATMUL_REMOTE_READ = 20,
    CATCCOS_ASCEND950_FP8_MX_ALLGATHER_MATMUL = 22,
    CATCCOS_ASCEND950_FP4_MX_ALLGATHER_MATMUL = 23,
    CATCCOS_MX_QUANT_ALLGATHER = 24,
    CATCCOS_ASCEND950_FP8_MX_GROUPED_MATMUL_ALLTOALLV = 25,
    CATCCOS_ASCEND950_FP4_MX_GROUPED_MATMUL_ALLTOALLV = 26,
    CATCCOS_ASCEND950_FP8_MX_ALLTOALLV_GROUPED_MATMUL = 27,
    CATCCOS_ASCEND950_FP4_MX_ALLTOALLV_GROUPED_MATMUL = 28,
    CATCCOS_ASCEND950_FP4_MX_MATMUL_REDUCE_SCATTER = 30,
    CATCCOS_ASCEND950_DISPATCH_FFN_COMBINE = 32,
    /* not in the reference's enum (its example instantiates the device template directly,
     * examples/ascend950_alltoall_matmul/main.cpp): a value of this library's own */
    CATCCOS_ASCEND950_ALLTOALL_MATMUL = 101,
    CATCCOS_ASCEND950_MATMUL_ALLTOALL = 102      /* likewise (examples/ascend950_matmul_alltoall/main.cpp) */
};
enum { CATCCOS_FP16 = 1, CATCCOS_INT8 = 2, CATCCOS_BF16 = 27, CATCCOS_FP8E4M3FN = 36 };

/* ------------------------------------------------------------------ symmetric heap ---- */

/* Replaces set_attr() + aclshmemx_init_attr() (utils/shmem_init.h:16-39,
 * examples/matmul_allreduce/main.cpp:122-125).  Collective.  Creates this PE's heap of
 * `local_mem_size` bytes on the current CUDA device, exchanges it with the peers found through
 * `ip_port` (any string shared by the job, e.g. "tcp://127.0.0.1:8788"; an empty string is
 * CATCCOS_ERR_INVALID as in set_attr) and maps every peer's heap over NVLink. */
CATCCOS_API int catccos_shmem_init(int32_t my_pe, int32_t n_pes, uint64_t local_mem_size, const char *ip_port);

/* Test/development mode with no counterpart in the reference: all `n_pes` PEs are regions on the
 * current device of this one process; the launch functions then take one parameter block per PE
 * (catccos_launch_emulated) and run all ranks inside one cooperative launch. */
CATCCOS_API int catccos_shmem_init_emulated(int32_t n_pes, uint64_t local_mem_size);

/* shmem_finalize() (examples/matmul_allreduce/main.cpp:178). Collective. */
CATCCOS_API int catccos_shmem_finalize(void);
/* shmem_malloc() / aclshmem_calloc() (main.cpp:135; tests/dynamic_tiling/main.cpp:291): collective,
 * same offset on every PE, 1024-byte aligned; NULL when the heap is exhausted.  Not zero-filled
 * (the kernels need no zeroed data region). */
CATCCOS_API void *catccos_shmem_malloc(size_t bytes);
/* shmem_free(): allocations are released in reverse order of allocation (stack discipline). */
CATCCOS_API void catccos_shmem_free(void *ptr);
/* shmem_ptr(p, pe): address in this process of PE `pe`'s copy of symmetric address `p`. */
CATCCOS_API void *catccos_shmem_ptr(const void *ptr, int32_t pe);
CATCCOS_API int32_t catccos_shmem_my_pe(void);   /* shmem_my_pe() */
CATCCOS_API int32_t catccos_shmem_n_pes(void);   /* shmem_n_pes() */
/* Host-side get (the role of aclshmem_getmem on the host): synchronises the device and copies `bytes`
 * bytes of PE `pe`'s copy of symmetric address `ptr` into host memory. */
CATCCOS_API int catccos_shmem_get_host(void *hostDst, const void *ptr, int32_t pe, size_t bytes);
/* Host-side put (aclshmem_putmem on the host): copies host memory into PE `pe`'s copy of `ptr`. */
CATCCOS_API int catccos_shmem_put_host(void *ptr, int32_t pe, const void *hostSrc, size_t bytes);
/* aclshmem_barrier_all() (examples/ascend950_dispatch_ffn_combine/main.cpp:217-219): host barrier
 * of all PEs after synchronising the device. */
CATCCOS_API int catccos_shmem_barrier_all(void);

/* ----------------------------------------------------------------------- diagnostics ---- */
CATCCOS_API const char *catccos_last_error(void);
/* Synchronises the device and copies the 8 status words {code, wait site, rank, flag index,
 * expected, seen, -, -}.  Returns CATCCOS_ERR_DEVICE_WAIT when code != 0 (CATCCOS_ERR_RANGE for code 5: a
 * partial product left the range of the reduce family's fp16 exchange format).  (The reference has no
 * return codes from kernels and unbounded device waits: utils/utils.h:26-40,
 * include/catccos/arch/cross_rank_sync.hpp:88-97.) */
CATCCOS_API int catccos_last_status(int32_t *words8);
CATCCOS_API int catccos_reset_status(void);
/* Bounded-wait self test: one thread waits `timeout_ms` for a flag nothing sets, then reports
 * through the status words.  Leaves the context usable. */
CATCCOS_API int catccos_debug_wait_unset_flag(void *stream, uint32_t timeout_ms);
/* Measurement switch (no counterpart in the reference): bit 0 makes later launches compute-only —
 * no peer traffic and no flag waits, operating on whatever an earlier fused launch left in the
 * symmetric region — so that exposed communication = fused time - compute-only time. */
CATCCOS_API int catccos_debug_set_flags(uint32_t flags);
/* Device-side tracing, the counterpart of the reference's AscendTimer (tools/AscendTimerDevice.hpp,
 * include/catccos/dgemm/device/device_dgemm.hpp:61-117): `device_buf` (device memory, at least
 * 16 * 8 bytes per CTA of the largest grid, zeroed by the caller) receives per-CTA %globaltimer
 * stamps and accumulated wait times of later launches; NULL switches tracing off. */
CATCCOS_API int catccos_debug_set_trace(void *device_buf);
/* With bit 1 of catccos_debug_set_flags set, a dispatch-FFN-combine launch records CUDA events between its
 * stages; after the stream has drained this returns their count and fills `ms` with the stage times in order:
 * route, quant-dispatch, weight scale atoms, wait for the dispatch, received scale atoms, GEMM1, GEMM2,
 * un-permute.  -1 on error. */
CATCCOS_API int catccos_debug_moe_stage_ms(float *ms, int32_t capacity);

/* The work orders of the CTA-pair kernels, computed on the host by the very functions the kernels use
 * (no device needed; no reference counterpart of their own — the reference's orders are CommSwizzle::GetCoord,
 * include/catccos/catccos.hpp:165-193, and its block schedulers).  Each call fills `out` with up to `capacity`
 * triples and returns how many the order has, or a negative CATCCOS_ERR_* code.
 *   rs_tile_order: pair tiles of Matmul-ReduceScatter / AllReduce for `rank`: (owner, 256-row stripe, column tile);
 *                  `rows_per_rank` rows per owner, `pairs` CTA pairs; *lag (optional) receives the own-stripe lag.
 *   ag_tile_order: pair tiles of AllGather-Matmul in claim order: (source rank, 256-row tile, column tile); m = rows
 *                  of one rank, `group` = 256-row tiles per L2 group (own and gathered rows are grouped separately;
 *                  column-tile major inside a group, odd groups backwards).
 *   ag_push_order: all-gather push units of `rank`: (destination, 128-row chunk, unit inside the chunk). */
CATCCOS_API int catccos_debug_rs_tile_order(int32_t world, int32_t rank, int32_t rows_per_rank, int32_t n, int32_t pairs,
                                            int32_t *out, int32_t capacity, int32_t *lag);
CATCCOS_API int catccos_debug_ag_tile_order(int32_t world, int32_t rank, int32_t m, int32_t n, int32_t group,
                                            int32_t *out, int32_t capacity);
CATCCOS_API int catccos_debug_ag_push_order(int32_t world, int32_t rank, int32_t m, int32_t *out, int32_t capacity);
/* The launcher's choice of `group`: the largest number of 256-row tiles (1..16) for which the group's rows of A
 * plus the column tiles of B in flight with them (`pairs` CTA pairs) stay inside `l2_budget_bytes`;
 * tile_bytes = 256 * k * element size. */
CATCCOS_API int catccos_debug_ag_group_rows(int64_t tile_bytes, int32_t pairs, int64_t l2_budget_bytes);
/* The double-buffering decision of the dense and MXFP8 launchers, replayed on the host for a sequence of `n`
 * launches: sigs[i] identifies operator + shape + buffer of launch i, foreign_before[i] != 0 means a launch of
 * another operator family (which consumes an epoch) happened just before it.  half[i] receives the half of the
 * symmetric region launch i uses, need_back[i] how many epochs back a peer may be and still be written to
 * (1: it has entered the previous launch; 0: it must have entered this one).  No device needed. */
CATCCOS_API int catccos_debug_slot_sequence(const uint64_t *sigs, const uint8_t *foreign_before, int32_t n, int32_t *half,
                                            int32_t *need_back);

/* Bytes of the `symmetric` buffer an operator carves for itself (the reference sizes it as one
 * fixed SHMEM_BUFF_BYTES allocation, utils/info.h:35). */
CATCCOS_API size_t catccos_symmetric_bytes(int32_t commType, int32_t dataType, const CocTilingParams *tiling);
/* GetWorkspaceSize() of the operator classes (utils/catccos_operator.h:39). */
CATCCOS_API size_t catccos_workspace_bytes(int32_t commType, int32_t dataType, const CocTilingParams *tiling);

/* ------------------------------------------------------------------ kernel launchers ---- */
/* tests/dynamic_tiling/include/launch_map.h:15-16 — KernelFuncPtr
 *   void (*)(void *stream, uint32_t blockNum, uint64_t fftsAddr, KernelParams &, uint8_t *workspace,
 *            uint8_t *symmetric, CocTilingParams &, uint32_t transA, uint32_t transB)
 * with the two references turned into pointers and an int status returned.  `stream` is a
 * cudaStream_t.  `blockNum` > 0 caps the number of SMs used (0 = all); `fftsAddr` is ignored.
 * Asynchronous on `stream`.  Shapes come from `tiling` (m, k, n, rankSize). */
#define CATCCOS_DECLARE_LAUNCH(name)                                                                   \
    CATCCOS_API int name(void *stream, uint32_t blockNum, uint64_t fftsAddr, CatccosKernelParams *params,          \
             uint8_t *workspace, uint8_t *symmetric, CocTilingParams *tiling, uint32_t transA, uint32_t transB)

/* tests/dynamic_tiling/impl/kernel_fp16.cpp / kernel_bf16.cpp:72,121,221 */
CATCCOS_DECLARE_LAUNCH(LaunchMatmulAllReduceFP16);
CATCCOS_DECLARE_LAUNCH(LaunchMatmulAllReduceBF16);
CATCCOS_DECLARE_LAUNCH(LaunchAllGatherMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAllGatherMatmulBF16);
CATCCOS_DECLARE_LAUNCH(LaunchMatmulReduceScatterFP16);
CATCCOS_DECLARE_LAUNCH(LaunchMatmulReduceScatterBF16);
/* tests/dynamic_tiling/include/launch_map.h:85-88 (same loops on the newer NPU) */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950AllGatherMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950AllGatherMatmulBF16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MatmulReduceScatterFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MatmulReduceScatterBF16);

/* Data-flow variants of AllGather-Matmul: same operands, tiling meaning and product as LaunchAllGatherMatmul*.
 * WithGatherResult (tests/dynamic_tiling/impl/kernel_bf16.cpp:286, include/catccos/dgemm/kernel/
 * allgather_matmul_with_gather_result.hpp): customPtrs = {gatherA}, a [rankSize*m, k] buffer that receives every
 * rank's A in rank order (examples/allgather_matmul_with_gather_result/..._host.h:51-54,75-79), written by the
 * kernel's copy warps as the rows arrive.
 * RemoteRead (kernel_bf16.cpp:170, include/catccos/dgemm/kernel/allgather_matmul_with_remote_read_local_mm_opt.hpp):
 * every rank stages its A in its own symmetric region and the peers fetch it from there (reads over NVLink,
 * arrival flags stay local) instead of every rank writing into its peers' regions. */
CATCCOS_DECLARE_LAUNCH(LaunchAllGatherMatmulWithGatherResultFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAllGatherMatmulWithGatherResultBF16);
CATCCOS_DECLARE_LAUNCH(LaunchAllGatherMatmulRemoteReadFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAllGatherMatmulRemoteReadBF16);

/* AllToAll-Matmul (examples/ascend950_alltoall_matmul, include/catccos/dgemm/kernel/ascend950_alltoall_matmul.hpp;
 * golden examples/ascend950_alltoall_matmul/scripts/gen_data.py:19-86): every rank holds A [m, k] with m divisible
 * by rankSize; rows [j*m/R, (j+1)*m/R) go to rank j, which multiplies the R blocks it holds afterwards (block i from
 * rank i) by its B [k, n]: ptrC = [m, n].  The AllGather-Matmul kernel with a per-destination source block. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950AllToAllMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950AllToAllMatmulBF16);

/* Matmul-AllToAll (examples/ascend950_matmul_alltoall, include/catccos/dgemm/kernel/ascend950_matmul_alltoall.hpp;
 * golden examples/ascend950_matmul_alltoall/scripts/gen_data.py:19-89): C_i = A_i [m, k] x B_i [k, n] on every rank,
 * then rows [j*m/R, (j+1)*m/R) of C_i go to rank j: ptrC = [m, n] with block i from rank i.  The Matmul-ReduceScatter
 * kernel without the sum; the symmetric region is that operator's. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MatmulAllToAllFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MatmulAllToAllBF16);
/* The same on MXFP8 operands (tests/dynamic_tiling/include/launch_map.h:104, examples/ascend950_mxfp8_matmul_alltoall,
 * row-block form of scripts/gen_data_slice_m.py): e4m3 codes, customPtrs = {aScale, bScale} as
 * LaunchAscend950MxFp8MatmulReduceScatter*, `workspace` = catccos_workspace_bytes() bytes. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MxFp8MatmulAllToAllFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MxFp8MatmulAllToAllBF16);

/* tests/dynamic_tiling/impl/kernel_fp16_ascend950.cpp:274 (MxAllGatherMatmulTla,
 * include/catccos/dgemm/kernel/mx_allgather_matmul.hpp:27-428): ptrA/ptrB = e4m3 operands,
 * customPtrs = {aScale [m, k/64, 2], bScale (transB=0: [k/64, n, 2]; transB=1: [n, k/64, 2])} E8M0 bytes,
 * `workspace` = catccos_workspace_bytes() bytes.  The data type names the 16-bit OUTPUT type (the
 * reference writes fp16, examples/ascend950_fp8_mx_allgather_matmul/..._host.h:33; BF16 is added). */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp8MxAllGatherMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp8MxAllGatherMatmulBF16);

/* tests/dynamic_tiling/include/launch_map.h:95 (Ascend950Fp4MxAllGatherMatmul; operator class
 * examples/ascend950_fp4_mx_allgather_matmul/ascend950_fp4_mx_allgather_matmul_host.h:88): MXFP4 operands --
 * ptrA = e2m1 codes [m, k/2] (two per byte, low nibble first), ptrB = [n, k/2] (transB = 1 only: 4-bit operands
 * are K-major on tcgen05), customPtrs = {aScale [m, k/64, 2], bScale [n, k/64, 2]} E8M0 bytes, one per 32 values
 * along k; k % 64 == 0.  ptrC = 16-bit [rankSize*m, n]; `workspace` = catccos_workspace_bytes() bytes.  One-CTA
 * tcgen05.mma.kind::mxf4nvf4 kernel with the all-gather of codes and scale atoms fused in. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxAllGatherMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxAllGatherMatmulBF16);
/* tests/dynamic_tiling/impl/kernel_fp16_ascend950.cpp:211 (Ascend950Fp4MxMatmulReduceScatter; operator class
 * examples/ascend950_fp4_mx_matmul_reduce_scatter/..._host.h:84): MXFP4 Matmul-ReduceScatter -- operands and scales as
 * LaunchAscend950Fp4MxAllGatherMatmul* (K-major, transB = 1 only; the reference's example runs transB = 0, whose
 * N-packed 4-bit B has no tcgen05 form), m = rows of the full product, ptrC = this rank's [m/rankSize, n] rows;
 * the MXFP8 reduce-scatter pair kernel with tcgen05.mma.kind::mxf4nvf4 on CTA pairs. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxMatmulReduceScatterFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxMatmulReduceScatterBF16);

/* MXFP8 Matmul-ReduceScatter (MatmulReduceScatterMxTla, include/catccos/dgemm/kernel/matmul_reduce_scatter_mx_tla.hpp:39;
 * operator "Ascend950MxFp8MatmulReduceScatter", examples/ascend950_mxfp8_matmul_reduce_scatter/main.cpp:32-141 and
 * ..._host.h:28-142): ptrA/ptrB = float8_e5m2 operands (what that example feeds), customPtrs = {aScale [m, k/64, 2],
 * bScale (transB=0: [k/64, n, 2]; transB=1: [n, k/64, 2])} E8M0 bytes, ptrC = this rank's [m/rankSize, n] rows of the
 * summed product in the 16-bit type the name gives; tiling m = rows of the full product (m/rankSize a multiple of
 * 128), k = this rank's share of the contraction.  `workspace` = catccos_workspace_bytes() bytes, `symmetric` as for
 * Matmul-ReduceScatter.  The E4M3 names take float8_e4m3fn operands (no reference counterpart of their own: the
 * reference kernel is a template over the element type). */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MxFp8MatmulReduceScatterFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MxFp8MatmulReduceScatterBF16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MxFp8E4M3MatmulReduceScatterFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950MxFp8E4M3MatmulReduceScatterBF16);

/* MxQuantAllGather (include/catccos/comm/kernel/mx_quant_allgather.hpp:57-288; registered as
 * REGISTER_KERNEL_FUNC(Ascend950BF16QuantAllGather, MX_QUANT_ALLGATHER, FP8E4M3FN), launch_map.h:91): KernelParams as in
 * examples/ascend950_mx_quant_allgather/mx_quant_allgather_host.h:48 — ptrA = input bf16 [m, n], ptrB = gathered
 * E8M0 scales [rankSize*m, even(n/32)], ptrC = gathered e4m3 codes [rankSize*m, n]; tiling m, n (n % 32 == 0). */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950BF16QuantAllGatherFP8E4M3FN);

/* Standalone MXFP8 AllToAllV-GroupedMatmul (include/catccos/dgemm/kernel/mx_alltoallv_group_matmul.hpp:37-496; operator
 * "Ascend950Fp8MxAllToAllVGroupedMatmul", examples/ascend950_fp8_mx_alltoallv_grouped_matmul/..._host.h:14-156) and
 * GroupedMatmul-AllToAllV (include/catccos/dgemm/kernel/grouped_matmul_alltoallv_mx.hpp:34-409; operator
 * "Ascend950Fp8MxGroupedMatmulAllToAllV").  KernelParams as the operator classes set them: ptrA = float8_e4m3fn rows
 * [m, k], ptrB = weights [expertNum/epSize, k, n], ptrC = 16-bit output with room for [rankSize*m, n],
 * customPtrs = {aScale [m, k/64, 2], bScale [expertNum/epSize, k/64, n, 2], localTokensPerExpert int32 [expertNum],
 * globalTokensPerLocalExpert int32 [rankSize, expertNum/epSize] (not read: the counts are exchanged on the device)}.
 *   AllToAllV-GroupedMatmul: this rank's rows are grouped by global expert with localTokensPerExpert rows each;
 *     every row goes to its expert's owner, which multiplies it with that expert's weight; ptrC receives the
 *     owner's rows in receive order (local expert major, source rank minor), the rest of ptrC is zero.
 *   GroupedMatmul-AllToAllV: ptrA holds the rows of this rank's experts in that receive order; every product row
 *     goes back to the rank it came from, whose ptrC ends up with its rows in global-expert order.
 * tiling: m, n, k (k % 64 == 0, n % 16 == 0), expertNum, epSize = rankSize.  `workspace` =
 * catccos_workspace_bytes() bytes (256-byte aligned), `symmetric` = catccos_symmetric_bytes() bytes. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp8MxAllToAllVGroupedMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp8MxAllToAllVGroupedMatmulBF16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp8MxGroupedMatmulAllToAllVFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp8MxGroupedMatmulAllToAllVBF16);
/* The same two operators on MXFP4 operands (tests/dynamic_tiling/include/launch_map.h:99,101;
 * examples/ascend950_fp4_mx_alltoallv_grouped_matmul, examples/ascend950_fp4_mx_grouped_matmul_alltoallv): ptrA = e2m1
 * codes [rows, k/2], ptrB = K-major weights [expertNum/epSize, n, k/2] (the transB = 1 form; N-packed 4-bit
 * weights have no tcgen05 form), bScale [expertNum/epSize, n, k/64, 2]; k % 256 == 0.  Everything else as above. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxAllToAllVGroupedMatmulFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxAllToAllVGroupedMatmulBF16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxGroupedMatmulAllToAllVFP16);
CATCCOS_DECLARE_LAUNCH(LaunchAscend950Fp4MxGroupedMatmulAllToAllVBF16);

/* The MoE operator: DispatchFFNCombine<...>(fftsAddr, gmA, gmB, gmBScale, gmB2, gmB2Scale, gmD, gmExpertIdx,
 * gmProbs, gmWorkSpace, gmSymmetric, CocTilingParams, ...) (examples/ascend950_dispatch_ffn_combine/
 * ascend950_dispatch_ffn_combine_device.h:617-718), with the operands in the operator class's KernelParams
 * order (ascend950_dispatch_ffn_combine_host.h:121-122, main.cpp:210-214): ptrA = tokens bf16 [m, k],
 * ptrB = up/gate weights e4m3 [E/R, n, k], ptrC = output bf16 [m, k], customPtrs = {b2 e4m3 [E/R, k, n/2],
 * expertIdx int32 [m, topK], probs fp32 [m, topK], bScale E8M0 [E/R, n, k/32], b2Scale E8M0 [E/R, k, n/64]}.
 * tiling: m, k, n, topK, expertNum, epSize (= rankSize).  k % 256 == 0 and n % 512 == 0 as in the reference.
 * `workspace` = catccos_workspace_bytes() bytes, 256-byte aligned. */
CATCCOS_DECLARE_LAUNCH(LaunchAscend950DispatchFFNCombineBF16);

/* KernelDispatcher::GetKernelFunc(commType, dataType) + call (launch_map.h:31-39,
 * tests/dynamic_tiling/main.cpp:351-368): CATCCOS_ERR_INVALID when the pair is not registered. */
CATCCOS_API int catccos_launch(int32_t commType, int32_t dataType, void *stream, uint32_t blockNum, uint64_t fftsAddr,
                   CatccosKernelParams *params, uint8_t *workspace, uint8_t *symmetric, CocTilingParams *tiling,
                   uint32_t transA, uint32_t transB);

/* Emulated-PE form of catccos_launch (see catccos_shmem_init_emulated): `params` and `workspaces`
 * are arrays with one entry per PE. */
CATCCOS_API int catccos_launch_emulated(int32_t commType, int32_t dataType, void *stream, uint32_t blockNum,
                            CatccosKernelParams *params, uint8_t **workspaces, uint8_t *symmetric,
                            CocTilingParams *tiling, uint32_t transA, uint32_t transB);

/* ------------------------------------------------------------------------ FP4 GEMM ---- */
/* Block-scaled FP4 GEMM on one GPU: C[m, n] = alpha * dequant(A)[m, k] x dequant(B)[n, k]^T, fp32 accumulation,
 * C in the 16-bit `dataType` (CATCCOS_FP16 / CATCCOS_BF16).  A and B hold two e2m1 codes per byte (low nibble =
 * even k), both K-major (B as [n, k]).  format 0 = MXFP4: one E8M0 scale per 32 along k, scale rows
 * [rows, even(k/32)] as the reference's FP4 operators store them (examples/ascend950_fp4_mx_allgather_matmul,
 * golden examples/utils/gen_data_fp4_mx_allgather_matmul.py:563-677); format 1 = NVFP4: one E4M3 scale per 16
 * along k, rows [rows, k/16], the two fp32 tensor scales multiplied into `alpha` (no reference counterpart: the
 * reference's FP4 is MXFP4).  k % 64 == 0, n % 8 == 0.  `workspace`: catccos_fp4_gemm_workspace_bytes() bytes of
 * device memory.  Needs no catccos_shmem_init. */
CATCCOS_API size_t catccos_fp4_gemm_workspace_bytes(int32_t format, uint32_t m, uint32_t n, uint32_t k);
CATCCOS_API int catccos_fp4_gemm(void *stream, int32_t format, int32_t dataType, const void *A, const void *B, void *C,
                                 const void *aScale, const void *bScale, float alpha, uint32_t m, uint32_t n, uint32_t k,
                                 void *workspace, uint32_t blockNum);

/* ------------------------------------------------------------------- host-buffer form ---- */
/* The operator classes' AllocateDeviceSpace() (host -> device copy of the inputs), kernel launch
 * and WriteResultFile() (device -> host copy of the result) in one synchronous call, with memory
 * instead of .bin files (examples/matmul_allreduce/matmul_allreduce_host.h:17-85,
 * examples/matmul_allreduce/main.cpp:127-171).  hostA/hostB/hostC (and hostCustom[i]) are host
 * buffers laid out as the operator's device operands; pinned memory copies fastest.  Device
 * staging buffers and the symmetric buffer are created on first use and kept. */
CATCCOS_API int catccos_run_host(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA,
                                 const void *hostB, void *hostC, const void *const *hostCustom, uint32_t customCount,
                                 CocTilingParams *tiling, uint32_t transA, uint32_t transB);
/* The same with operands that stay on the device between calls.  Bit i of `residentMask` (bit 0 = A, bit 1 = B,
 * bit 3 + j = hostCustom[j]) marks an operand as resident: it is copied when its host pointer or size differs
 * from the previous call's and skipped otherwise -- expert weights and weight scales of the MoE operator, the
 * weight matrix of the block-scaled GEMMs.  Serves Ascend950Fp8MxAllGatherMatmul, Ascend950MxFp8MatmulReduceScatter
 * and Ascend950DispatchFFNCombine (hostCustom in the operator's customPtrs order); of the dense operators'
 * operands only B (bit 1) can be resident.  catccos_run_host() is this call with a mask of 0. */
CATCCOS_API int catccos_run_host_resident(int32_t commType, int32_t dataType, uint32_t blockNum, const void *hostA,
                                          const void *hostB, void *hostC, const void *const *hostCustom,
                                          uint32_t customCount, CocTilingParams *tiling, uint32_t transA, uint32_t transB,
                                          uint32_t residentMask);

/* ------------------------------------------------------------------ MX quantisation ---- */
/* CommBlockMxQuant::ComputeMxQuant (include/catccos/comm/block/comm_block_mx_quant.hpp:413-663) on
 * a whole [rows, k] bf16 matrix: e4m3 codes [rows, k] and one E8M0 scale byte per 32 values along k,
 * written as [rows, even(k/32)] bytes (odd counts padded with 127 = 1.0), bit-identical to the
 * reference's host golden (examples/utils/gen_mx_quant_allgather_data.py:168-189,255-313 with the
 * round-to-nearest-even cast).  k must be a multiple of 32.  `sfAtoms` (optional, may be NULL)
 * additionally receives the scales in the tcgen05 scale-factor layout that the MX GEMM kernels read
 * (catccos_sf_atoms_bytes bytes).  Asynchronous on `stream`; needs no symmetric heap. */
CATCCOS_API int catccos_mx_quant(void *stream, const void *inputBf16, uint8_t *codes, uint8_t *scales, uint8_t *sfAtoms,
                                 uint32_t rows, uint32_t k);
CATCCOS_API size_t catccos_sf_atoms_bytes(uint32_t rows, uint32_t k);

/* ------------------------------------------------------------- allocation-free GEMM ---- */
/* No counterpart in the reference.  For callers that cannot allocate device memory where they
 * need a GEMM: plugins inside a runtime that owns and budgets all device memory (an allocation
 * made behind its back breaks its accounting or simply fails), and loops that cannot afford the
 * implicit device synchronisation of an allocation.  Computes C[m,n] = A[m,k] * B (transB=0:
 * B[k,n]; transB=1: B[n,k]) in FP16 or BF16 with fp32 accumulation on the current device,
 * asynchronously on `stream`, with the same tcgen05 kernel as the AllGather-Matmul launchers at a
 * world size of one.  It needs no catccos_shmem_init and calls no cudaMalloc/cudaFree or
 * allocating library routine: the only scratch the kernel needs (8 status words and 16 trace
 * slots per CTA) lives in a fixed array of about 33 KiB inside the library image, which every GPU
 * that loads the library holds until the process exits.
 *   - Limit: at most 256 CTAs (the array has trace slots for 256); on a device with more SMs pass
 *     blockNum <= 256, otherwise CATCCOS_ERR_INVALID.  n and k must be multiples of 8, every
 *     dimension at most 2^30, pointers 16-byte aligned.
 *   - The first call on each device does the set-up for that device (with that device current,
 *     once, under a lock): it looks up the array's device address and sets the shared-memory
 *     attribute of every kernel variant.  That first call should come before any stream capture.
 *   - All calls on a device share the array and each call clears it first (on `stream`): calls
 *     that overlap on the GPU (different streams) race on the status words and trace slots.
 *   - Waits inside the kernel are bounded by CATCCOS_WAIT_TIMEOUT_MS (default 10 s).
 * catccos_gemm_no_alloc_status synchronises the device and copies the 8 status words (and, if
 * `trace` is not NULL, 16 uint64 trace slots for each of `traceCtas` CTAs) of the last call. */
CATCCOS_API int catccos_gemm_no_alloc(void *stream, const void *A, const void *B, void *C, uint32_t m, uint32_t n,
                                      uint32_t k, int32_t dataType, uint32_t transB, uint32_t blockNum);
CATCCOS_API int catccos_gemm_no_alloc_status(int32_t *words8, uint64_t *trace, uint32_t traceCtas);

#ifdef __cplusplus
}
#endif
#endif /* CATCCOS_B200_H */

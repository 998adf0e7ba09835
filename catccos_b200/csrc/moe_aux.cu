// MoE helper kernels: routing (stable counting sort + count exchange + offset tables),
// quantise-and-dispatch, and the weighted un-permute.
//
// Reference semantics:
//   routing      examples/aux_ops/moe_init_routing_v2/moe_init_routing_v2.h:54-241 (stable sort by expert,
//                expandedRowIdx src -> dst, tokens per expert); golden examples/utils/gen_data_moe.py:48-57
//   count gather examples/aux_ops/allgather_kernel_with_flag.h:24-155
//   offsets      include/catccos/comm/block/comm_block_scheduler_alltoallv_gmm.hpp:72-78,131-159 (prevSum, cumsumMM)
//   dispatch     include/catccos/comm/block/comm_block_mx_quant.hpp:318-369 (quantise once, scatter to top-k slots)
//                and include/catccos/dgemm/kernel/ascend950_alltoall_gmm.hpp:419-471 (receive order:
//                local expert major, source rank minor)
//   un-permute   examples/aux_ops/moe_token_unpermute/moe_token_unpermute.h:234-278
#include "moe_ops.h"

#include <stdlib.h>

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace cb {

namespace {

__device__ __forceinline__ uint32_t *mflag(const MoeParams &p, int pe, uint32_t word) {
    return reinterpret_cast<uint32_t *>(p.heap_base[pe]) + word;
}

// ------------------------------------------------------------------------------ routing ----
// One CTA (1024 threads) per rank.  Stable counting sort with warp-private counters: warp w owns
// the w-th contiguous slice of the flattened [m, topK] expert ids, walks it 32 ids at a time and
// ranks equal ids inside a step with __match_any_sync, so equal experts keep their index order.
// lanes of the warp whose key equals this lane's (what __match_any_sync returns), from one ballot per key bit:
// keys are expert ids below 2^bits, or negative for lanes that take no part (they match nobody but themselves)
__device__ __forceinline__ unsigned same_key_lanes(int key, int bits, int lane) {
    const bool valid = key >= 0;
    unsigned mask = __ballot_sync(0xffffffffu, valid);
    for (int b = 0; b < bits; ++b) {
        const unsigned has = __ballot_sync(0xffffffffu, valid && ((key >> b) & 1));
        mask &= ((key >> b) & 1) ? has : ~has;
    }
    return valid ? mask : (1u << lane);
}

__global__ void __launch_bounds__(1024, 1) moe_route_kernel(const MoeParams p) {
    extern __shared__ int smem_i[];
    const int E = p.experts;
    int *cnt = smem_i;                    // [32][E]
    int *scan = smem_i + 32 * E;          // [E] totals, then exclusive prefix
    int *seg_all = scan + E;              // [E] receive segment base of every expert on its owner
    __shared__ int abort_flag;
    __shared__ int seg_end_all[kMaxRanks];

    const int lrank = blockIdx.x;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const int EL = p.experts_per_rank;
    const MoeRankArgs &ra = p.ranks[lrank];
    MoeMeta *meta = ra.meta;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int total = p.m * p.top_k;

    if (tid == 0) abort_flag = 0;
    for (int i = tid; i < 32 * E; i += blockDim.x) cnt[i] = 0;
    if (tid < 4) {
        meta->done_counter[tid] = 0;
        meta->tile_queue[tid >> 1][tid & 1] = 0;
    }
    if (tid == 0) meta->overflow = 0;
    // this rank's symmetric data regions may be overwritten from now on
    if (tid < R && tid != rank) {
        fence_sys();
        st_release_sys(mflag(p, tid, kFlagEntered + rank), p.epoch);
    }
    __syncthreads();

    // equal keys inside a step of 32 ids are found with one ballot per key bit (p.route_ballot; 0: the match instruction)
    int key_bits = 0;
    if (p.route_ballot)
        while ((1 << key_bits) < E) ++key_bits;
    const int chunk = ((total + 31) / 32 + 31) / 32 * 32;
    const int begin = warp * chunk;
    const int end = min(total, begin + chunk);
    // a negative expert id marks a row that takes no part (the all-to-all-v operators pad their row lists with them)
    // the ids are read eight steps at a time, so that their load latencies overlap
    constexpr int kBatch = 8;
    for (int base = begin; base < end; base += 32 * kBatch) {
        int raws[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int i = base + j * 32 + lane;
            raws[j] = i < end ? ra.expert_idx[i] : -1;
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            if (base + j * 32 >= end) break;
            const int raw = raws[j];
            const bool valid = raw >= 0;
            const int key = valid ? raw : -1 - lane;
            const unsigned mask = key_bits ? same_key_lanes(raw, key_bits, lane) : __match_any_sync(0xffffffffu, key);
            if (valid && lane == __ffs(mask) - 1) cnt[warp * E + key] += __popc(mask);
            __syncwarp();
        }
    }
    __syncthreads();
    if (tid < E) {
        int tot = 0;
        for (int w = 0; w < 32; ++w) tot += cnt[w * E + tid];
        scan[tid] = tot;
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = scan[e];
            scan[e] = run;
            run += c;
        }
    }
    __syncthreads();
    int my_count = 0;
    if (tid < E) {
        // counters -> first destination row of (warp, expert)
        int run = scan[tid];
        for (int w = 0; w < 32; ++w) {
            const int c = cnt[w * E + tid];
            cnt[w * E + tid] = run;
            run += c;
        }
        my_count = run - scan[tid];
    }
    __syncthreads();
    for (int base = begin; base < end; base += 32 * kBatch) {
        int raws[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            const int i = base + j * 32 + lane;
            raws[j] = i < end ? ra.expert_idx[i] : -1;
        }
#pragma unroll
        for (int j = 0; j < kBatch; ++j) {
            if (base + j * 32 >= end) break;
            const int i = base + j * 32 + lane;
            const int raw = raws[j];
            const bool valid = raw >= 0;
            const int key = valid ? raw : -1 - lane;
            const unsigned mask = key_bits ? same_key_lanes(raw, key_bits, lane) : __match_any_sync(0xffffffffu, key);
            const int rnk = __popc(mask & ((1u << lane) - 1u));
            int dst = -1;
            if (valid) dst = cnt[warp * E + key] + rnk;
            __syncwarp();
            if (valid && lane == __ffs(mask) - 1) cnt[warp * E + key] += __popc(mask);
            __syncwarp();
            if (i < end) ra.expanded_row_idx[i] = dst;
        }
    }
    __syncthreads();      // the warp counters are dead from here on: their space holds the gathered counts below

    // ---- tokens-per-expert to every rank (the count all-gather), then the offset tables ----
    if (tid < E) {
        for (int pe = 0; pe < R; ++pe) {
            int *dstc = reinterpret_cast<int *>(p.heap_base[pe] + p.lay.counts_off);
            dstc[rank * E + tid] = my_count;
        }
    }
    __syncthreads();
    if (tid < R) {
        fence_sys();
        st_release_sys(mflag(p, tid, kMoeFlagCounts + rank), p.epoch);
    }
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (tid < R) wait_flag_ge(mflag(p, rank, kMoeFlagCounts + tid), p.epoch, ctl, W_MOE_COUNTS, tid);
    __syncthreads();
    if (abort_flag) return;

    // the all-gathered [R][E] table goes into shared memory once; the serial loops below read it from there
    int *counts = cnt;
    {
        const int *counts_g = reinterpret_cast<const int *>(p.heap_base[rank] + p.lay.counts_off);
        for (int i = tid; i < R * E; i += blockDim.x) {
            const int c = counts_g[i];
            counts[i] = c;
            meta->counts_all[i / E][i % E] = c;
        }
    }
    __syncthreads();
    if (tid < R) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            meta->prefix_all[tid][e] = run;
            run += counts[tid * E + e];
        }
    }
    // receive layout of every owner: local-expert segments start on multiples of 128 rows
    if (tid < R) {
        int run = 0;
        for (int le = 0; le < EL; ++le) {
            const int e = tid * EL + le;
            int rows = 0;
            for (int r = 0; r < R; ++r) rows += counts[r * E + e];
            seg_all[e] = run;
            run += (rows + 127) / 128 * 128;
        }
        seg_end_all[tid] = run;
    }
    __syncthreads();
    if (tid < E) {
        int before = 0;
        for (int r = 0; r < rank; ++r) before += counts[r * E + tid];
        meta->dest_base[tid] = seg_all[tid] + before;
    }
    if (tid < EL) {
        const int e = rank * EL + tid;
        int run = 0;
        for (int r = 0; r < R; ++r) {
            meta->cum_src[r][tid] = run;
            run += counts[r * E + e];
        }
        meta->cum_src[R][tid] = run;
        meta->seg_rows[tid] = run;
        meta->seg_base[tid] = seg_all[e];
    }
    if (tid == 0) {
        meta->seg_base[EL] = seg_end_all[rank];
        int tiles = 0, rows = 0;
        for (int le = 0; le < EL; ++le) {
            int r2 = 0;
            for (int r = 0; r < R; ++r) r2 += counts[r * E + rank * EL + le];
            meta->tile_prefix[le] = tiles;
            tiles += (r2 + 127) / 128;
            rows += r2;
        }
        meta->tile_prefix[EL] = tiles;
        meta->total_rows = rows;
        int over = 0;
        for (int o = 0; o < R; ++o)
            if (seg_end_all[o] > p.lay.rows_cap) over = 1;
        if (over) {
            meta->overflow = 1;
            if (atomicCAS(p.status + ST_CODE, 0, 4) == 0) {   // 4: receive capacity exceeded
                p.status[ST_WHERE] = W_MOE_ROWS;
                p.status[ST_RANK] = rank;
                p.status[ST_EXPECTED] = p.lay.rows_cap;
                p.status[ST_SEEN] = seg_end_all[rank];
            }
        }
    }
}

// -------------------------------------------------------------------- quantise + dispatch ----
__device__ __forceinline__ uint32_t abs_max8(const uint4 &v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t m = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        m = max(m, w[i] & 0x7FFFu);
        m = max(m, (w[i] >> 16) & 0x7FFFu);
    }
    return m;
}
__device__ __forceinline__ uint32_t cvt_e4m3(float x) {
    if (x != x) return 0x7Fu | ((__float_as_uint(x) >> 24) & 0x80u);
    return static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

constexpr int kDispWarps = 8;
constexpr int kMaxTopK = 16;

// One warp per token: the row is quantised once and written to each of its top-k destination rows
// (codes as 256-byte warp-wide stores, the row's scale bytes as 8-byte stores from shared memory).
__global__ void __launch_bounds__(kDispWarps * 32) moe_quant_dispatch_kernel(const MoeParams p) {
    __shared__ __align__(16) uint8_t s_scale[kDispWarps][1024];
    __shared__ int abort_flag;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const MoeRankArgs &ra = p.ranks[lrank];
    const MoeMeta *meta = ra.meta;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    // every owner must have entered this epoch before its receive rows are overwritten
    if (threadIdx.x < R && threadIdx.x != rank)
        wait_flag_ge(mflag(p, rank, kFlagEntered + threadIdx.x), p.epoch, ctl, W_ENTERED, threadIdx.x);
    __syncthreads();
    const bool skip = abort_flag || meta->overflow;

    const int K = p.K, EL = p.experts_per_rank, topk = p.top_k;
    const int vec_per_row = K >> 3;
    const int sld = p.lay.scale_ld;
    if (!skip) {
        for (int t = cta * kDispWarps + warp; t < p.m; t += p.ctas_per_rank * kDispWarps) {
            // lane k < topK resolves destination k
            unsigned long long my_codes = 0, my_scales = 0;
            if (lane < topk) {
                const int e = ra.expert_idx[t * topk + lane];
                const int d = ra.expanded_row_idx[t * topk + lane];
                const int row = meta->dest_base[e] + (d - meta->prefix_all[rank][e]);
                const int o = e / EL;
                my_codes = reinterpret_cast<unsigned long long>(p.heap_base[o] + p.lay.recv_codes_off +
                                                                static_cast<size_t>(row) * K);
                my_scales = reinterpret_cast<unsigned long long>(p.heap_base[o] + p.lay.recv_scale_off +
                                                                 static_cast<size_t>(row) * sld);
            }
            const uint4 *src = reinterpret_cast<const uint4 *>(static_cast<const __nv_bfloat16 *>(ra.x) +
                                                               static_cast<size_t>(t) * K);
            for (int v = lane; v < vec_per_row; v += 32) {
                const uint4 x = __ldg(src + v);
                uint32_t am = abs_max8(x);
                am = max(am, __shfl_xor_sync(0xffffffffu, am, 1));
                am = max(am, __shfl_xor_sync(0xffffffffu, am, 2));
                const float amax = __uint_as_float(am << 16);
                uint32_t sb = 127u;
                float inv = 1.0f;
                if (!(amax < 1e-12f)) {
                    const uint32_t e8 = (am >> 7) & 0xFFu;
                    sb = e8 - 8u;
                    inv = __uint_as_float((262u - e8) << 23);
                }
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
                uint32_t c[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    c[2 * i] = cvt_e4m3(__uint_as_float(w[i] << 16) * inv);
                    c[2 * i + 1] = cvt_e4m3(__uint_as_float(w[i] & 0xFFFF0000u) * inv);
                }
                uint2 q;
                q.x = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
                q.y = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
                if ((v & 3) == 0) s_scale[warp][v >> 2] = static_cast<uint8_t>(sb);
                for (int k = 0; k < topk; ++k) {
                    uint8_t *dst = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, my_codes, k));
                    *reinterpret_cast<uint2 *>(dst + static_cast<size_t>(v) * 8) = q;
                }
            }
            // K % 256 == 0: vec_per_row is a multiple of 32, all lanes ran the same number of iterations
            __syncwarp();
            for (int k = 0; k < topk; ++k) {
                uint8_t *dst = reinterpret_cast<uint8_t *>(__shfl_sync(0xffffffffu, my_scales, k));
                for (int j = lane; j < sld / 8; j += 32)
                    *reinterpret_cast<uint2 *>(dst + j * 8) = *reinterpret_cast<const uint2 *>(&s_scale[warp][j * 8]);
            }
            __syncwarp();
        }
    }
    // last CTA of this rank publishes "my rows are in place" to every owner
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(&ra.meta->done_counter[0], 1u);
        if (prev == static_cast<unsigned>(p.ctas_per_rank) - 1u) {
            fence_sys();
            for (int o = 0; o < R; ++o) st_release_sys(mflag(p, o, kMoeFlagDispatch + rank), p.epoch);
        }
    }
}

// -------------------------------------------------------------------------- un-permute ----
// out[t] = bf16_rne( sum_k fp32(combine[idx[t,k]]) * prob[t,k] ), products and sums rounded
// separately (no fused multiply-add) in k order.
__global__ void __launch_bounds__(256) moe_unpermute_kernel(const MoeParams p) {
    __shared__ int abort_flag;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const MoeRankArgs &ra = p.ranks[lrank];
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x < R) wait_flag_ge(mflag(p, rank, kMoeFlagCombine + threadIdx.x), p.epoch, ctl, W_MOE_COMBINE, threadIdx.x);
    __syncthreads();
    if (abort_flag || ra.meta->overflow) return;
    const int K = p.K, topk = p.top_k;
    const int vec_per_row = K >> 3;
    const __nv_bfloat16 *comb = reinterpret_cast<const __nv_bfloat16 *>(p.heap_base[rank] + p.lay.combine_off);
    __shared__ int s_row[kMaxTopK];
    __shared__ float s_w[kMaxTopK];
    // one CTA per token at a time; every thread keeps the token's top-k row pieces in flight together
    for (int t = cta; t < p.m; t += p.ctas_per_rank) {
        __syncthreads();
        if (threadIdx.x < topk) {
            s_row[threadIdx.x] = ra.expanded_row_idx[t * topk + threadIdx.x];
            s_w[threadIdx.x] = ra.probs[t * topk + threadIdx.x];
        }
        __syncthreads();
        for (int v = threadIdx.x; v < vec_per_row; v += blockDim.x) {
            uint4 x[kMaxTopK];
#pragma unroll
            for (int k = 0; k < kMaxTopK; ++k)
                if (k < topk)
                    x[k] = __ldcs(reinterpret_cast<const uint4 *>(comb + static_cast<size_t>(s_row[k]) * K + v * 8));
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
            for (int k = 0; k < kMaxTopK; ++k) {
                if (k < topk) {
                    const float w = s_w[k];
                    const uint32_t xs[4] = {x[k].x, x[k].y, x[k].z, x[k].w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        acc[2 * j] = __fadd_rn(acc[2 * j], __fmul_rn(__uint_as_float(xs[j] << 16), w));
                        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __fmul_rn(__uint_as_float(xs[j] & 0xFFFF0000u), w));
                    }
                }
            }
            uint4 o;
            o.x = Pack2<__nv_bfloat16>::pack(acc[0], acc[1]);
            o.y = Pack2<__nv_bfloat16>::pack(acc[2], acc[3]);
            o.z = Pack2<__nv_bfloat16>::pack(acc[4], acc[5]);
            o.w = Pack2<__nv_bfloat16>::pack(acc[6], acc[7]);
            *reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(ra.out) + static_cast<size_t>(t) * K + v * 8) = o;
        }
    }
}

// ---------------------------------------------- standalone all-to-all-v operators ----
// AllToAllV-GroupedMatmul and GroupedMatmul-AllToAllV take rows that are already MXFP8 and already
// sorted by expert, with the counts given (include/catccos/dgemm/kernel/mx_alltoallv_group_matmul.hpp:37-496,
// grouped_matmul_alltoallv_mx.hpp:34-409).  They reuse the routing kernel (count exchange, offset
// tables) by handing it an expert id per row, synthesised from the counts.

// idx[i] = expert of row i for i < sum(counts), -1 (no row) beyond; one CTA per local rank
__global__ void a2av_expert_idx_kernel(const MoeParams p, A2avPtrs ptrs) {
    __shared__ int prefix[kMoeMaxExperts + 1];
    const int lrank = blockIdx.x;
    const int *counts = ptrs.local_tokens[lrank];
    int *idx = const_cast<int *>(p.ranks[lrank].expert_idx);
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < p.experts; ++e) {
            prefix[e] = run;
            run += max(counts[e], 0);
        }
        prefix[p.experts] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.m; i += blockDim.x) {
        int lo = 0, hi = p.experts;                  // largest e with prefix[e] <= i
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (prefix[mid] <= i) lo = mid; else hi = mid;
        }
        idx[i] = i < prefix[p.experts] ? lo : -1;
    }
}

// One warp per row: copies the row's codes and scale bytes into a receive buffer.
//   mode 0 (dispatch): my row i (global-expert order) -> its expert owner's receive rows;
//   mode 1 (re-layout): my row u (owner order: local expert major, source rank minor, no padding) -> my own
//                       receive rows, whose expert segments start on multiples of 128.
__global__ void __launch_bounds__(256) a2av_move_rows_kernel(const MoeParams p, A2avPtrs ptrs, int mode) {
    __shared__ int abort_flag;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const int R = p.world;
    const MoeRankArgs &ra = p.ranks[lrank];
    const MoeMeta *meta = ra.meta;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    // every rank must have entered this epoch before its symmetric rows are overwritten
    if (threadIdx.x < R && threadIdx.x != rank)
        wait_flag_ge(mflag(p, rank, kFlagEntered + threadIdx.x), p.epoch, ctl, W_ENTERED, threadIdx.x);
    __syncthreads();
    const bool skip = abort_flag || meta->overflow;
    const int K = p.K, EL = p.experts_per_rank, sld = p.lay.scale_ld;
    const int src_sld = ptrs.scale_ld;
    const uint8_t *codes = ptrs.codes[lrank], *scales = ptrs.scales[lrank];
    const int rows = mode == 0 ? p.m : meta->total_rows;
    if (!skip) {
        for (int i = cta * 8 + warp; i < rows; i += p.ctas_per_rank * 8) {
            int o, row;
            if (mode == 0) {
                const int e = ra.expert_idx[i];
                if (e < 0) continue;
                row = meta->dest_base[e] + (ra.expanded_row_idx[i] - meta->prefix_all[rank][e]);
                o = e / EL;
            } else {
                int le = 0, before = 0;
                while (le + 1 < EL && i >= before + meta->seg_rows[le]) before += meta->seg_rows[le++];
                row = meta->seg_base[le] + (i - before);
                o = rank;
            }
            uint8_t *dc = p.heap_base[o] + p.lay.recv_codes_off + static_cast<size_t>(row) * K;
            uint8_t *ds = p.heap_base[o] + p.lay.recv_scale_off + static_cast<size_t>(row) * sld;
            const uint4 *sc = reinterpret_cast<const uint4 *>(codes + static_cast<size_t>(i) * K);
            for (int v = lane; v < K / 16; v += 32) reinterpret_cast<uint4 *>(dc)[v] = __ldg(sc + v);
            for (int v = lane; v < sld; v += 32) ds[v] = v < src_sld ? scales[static_cast<size_t>(i) * src_sld + v] : 127;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned prev = atomicAdd(&ra.meta->done_counter[0], 1u);
        if (prev == static_cast<unsigned>(p.ctas_per_rank) - 1u) {
            fence_sys();
            if (mode == 0) {
                for (int o = 0; o < R; ++o) st_release_sys(mflag(p, o, kMoeFlagDispatch + rank), p.epoch);
            } else {
                st_release_sys(mflag(p, rank, kMoeFlagDispatch + rank), p.epoch);
            }
        }
    }
}

// GroupedMatmul-AllToAllV, last step: my rows have come back into my combine buffer (16-bit, in my
// expert-sorted order); copy them to the caller's output once every owner has flagged completion.
__global__ void __launch_bounds__(256) a2av_copy_out_kernel(const MoeParams p, int n_cols) {
    __shared__ int abort_flag;
    const int lrank = blockIdx.x / p.ctas_per_rank;
    const int cta = blockIdx.x - lrank * p.ctas_per_rank;
    const int rank = p.rank_base + lrank;
    const MoeRankArgs &ra = p.ranks[lrank];
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x < p.world)
        wait_flag_ge(mflag(p, rank, kMoeFlagCombine + threadIdx.x), p.epoch, ctl, W_MOE_COMBINE, threadIdx.x);
    __syncthreads();
    if (abort_flag || ra.meta->overflow) return;
    int mine = 0;
    for (int e = 0; e < p.experts; ++e) mine += ra.meta->counts_all[rank][e];
    const size_t vecs = static_cast<size_t>(mine) * n_cols / 8;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.heap_base[rank] + p.lay.combine_off);
    uint4 *dst = reinterpret_cast<uint4 *>(ra.out);
    for (size_t v = static_cast<size_t>(cta) * blockDim.x + threadIdx.x; v < vecs; v += static_cast<size_t>(p.ctas_per_rank) * blockDim.x)
        dst[v] = src[v];
}

// One CTA per rank: returns once every rank's dispatch rows have landed in my receive buffer.
__global__ void moe_wait_dispatch_kernel(const MoeParams p) {
    __shared__ int abort_flag;
    const int rank = p.rank_base + blockIdx.x;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    WaitCtl ctl;
    ctl.abort_smem = &abort_flag;
    ctl.status = p.status;
    ctl.deadline_ns = globaltimer_ns() + p.timeout_ns;
    ctl.rank = rank;
    if (threadIdx.x < p.world)
        wait_flag_ge(mflag(p, rank, kMoeFlagDispatch + threadIdx.x), p.epoch, ctl, W_MOE_ROWS, threadIdx.x);
}

}  // namespace

int moe_launch_wait_dispatch(const MoeParams &p, cudaStream_t stream) {
    moe_wait_dispatch_kernel<<<p.n_local, 32, 0, stream>>>(p);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("moe_wait_dispatch_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int moe_launch_route(const MoeParams &p_in, cudaStream_t stream) {
    MoeParams p = p_in;
    p.route_ballot = 1;
    if (const char *e = getenv("CATCCOS_ROUTE_BALLOT")) p.route_ballot = atoi(e) != 0;
    const size_t smem = static_cast<size_t>(34) * p.experts * sizeof(int);
    cudaError_t e = cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess) {
        if (p.n_local > 1) {
            void *args[] = {const_cast<MoeParams *>(&p)};
            e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(moe_route_kernel), dim3(p.n_local), dim3(1024), args,
                                            smem, stream);
        } else {
            moe_route_kernel<<<1, 1024, smem, stream>>>(p);
            e = cudaGetLastError();
        }
    }
    if (e != cudaSuccess) {
        set_error("moe_route_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

template <typename K>
static int launch_grid(K kern, const MoeParams &p, int threads, cudaStream_t stream, const char *name) {
    cudaError_t e;
    const int grid = p.ctas_per_rank * p.n_local;
    if (p.n_local > 1) {
        void *args[] = {const_cast<MoeParams *>(&p)};
        e = cudaLaunchCooperativeKernel(reinterpret_cast<void *>(kern), dim3(grid), dim3(threads), args, 0, stream);
    } else {
        kern<<<grid, threads, 0, stream>>>(p);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("%s launch failed: %s", name, cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

// The two HBM-bound kernels wait only for flags of kernels that ran (or run on other GPUs), never
// for their own CTAs, so they need no co-residency: plain launches with several CTAs per SM.
template <typename K>
static int launch_wide(K kern, const MoeParams &p, int threads, int ctas_per_sm, cudaStream_t stream, const char *name) {
    MoeParams q = p;
    q.ctas_per_rank = p.ctas_per_rank * ctas_per_sm;
    kern<<<q.ctas_per_rank * q.n_local, threads, 0, stream>>>(q);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s launch failed: %s", name, cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}
int a2av_launch_expert_idx(const MoeParams &p, const A2avPtrs &ptrs, cudaStream_t stream) {
    a2av_expert_idx_kernel<<<p.n_local, 256, 0, stream>>>(p, ptrs);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("a2av_expert_idx_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}
int a2av_launch_move_rows(const MoeParams &p, const A2avPtrs &ptrs, int mode, cudaStream_t stream) {
    MoeParams q = p;
    q.ctas_per_rank = p.ctas_per_rank * 4;
    a2av_move_rows_kernel<<<q.ctas_per_rank * q.n_local, 256, 0, stream>>>(q, ptrs, mode);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("a2av_move_rows_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}
int a2av_launch_copy_out(const MoeParams &p, int n_cols, cudaStream_t stream) {
    MoeParams q = p;
    q.ctas_per_rank = p.ctas_per_rank * 4;
    a2av_copy_out_kernel<<<q.ctas_per_rank * q.n_local, 256, 0, stream>>>(q, n_cols);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("a2av_copy_out_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}
int moe_launch_dispatch(const MoeParams &p, cudaStream_t stream) {
    return launch_wide(moe_quant_dispatch_kernel, p, kDispWarps * 32, 4, stream, "moe_quant_dispatch_kernel");
}
int moe_launch_unpermute(const MoeParams &p, cudaStream_t stream) {
    // a thread count that divides the 16-byte pieces of a row leaves no thread idle in the last pass over a token
    const int vecs = p.K / 8;
    const int threads = vecs % 256 == 0 ? 256 : vecs % 224 == 0 ? 224 : vecs % 192 == 0 ? 192 : 256;
    return launch_wide(moe_unpermute_kernel, p, threads, 6, stream, "moe_unpermute_kernel");
}

}  // namespace cb

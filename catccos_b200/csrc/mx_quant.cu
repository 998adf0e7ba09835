// MX block quantisation (bf16 -> e4m3 codes + E8M0 scale per 32 along K): HBM-bound kernels.
//
// Follows the reference's host golden bit for bit (examples/utils/gen_mx_quant_allgather_data.py:
// 168-189, 255-313 with the round-to-nearest-even cast of gen_data_moe.py:482-493), which is also
// what the reference's device code does (include/catccos/comm/block/comm_block_mx_quant.hpp:413-663)
// except for blocks whose largest magnitude is below 1e-12, where the golden's rule (scale 1.0) wins.
#include "mx_quant.h"

#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "ptx.cuh"

namespace cb {

namespace {

__device__ __forceinline__ uint32_t bf16_abs_max(const uint4 &v) {
    // largest |bits| of the 8 bf16 values (integer order == magnitude order; NaN sorts above Inf)
    // two 16-bit magnitudes per word, SIMD-in-word unsigned max
    const uint32_t m01 = __vmaxu2(v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu);
    const uint32_t m23 = __vmaxu2(v.z & 0x7FFF7FFFu, v.w & 0x7FFF7FFFu);
    const uint32_t m = __vmaxu2(m01, m23);
    return max(m & 0xFFFFu, m >> 16);
}

// scale byte and the exact reciprocal 2^-exp for a block whose largest |bf16 bits| is amax_bits
__device__ __forceinline__ void block_scale(uint32_t amax_bits, uint32_t *scale_byte, float *inv_scale) {
    const float amax = __uint_as_float(amax_bits << 16);
    // `amax < 1e-12` is false for NaN, as in the golden
    if (amax < 1e-12f) {
        *scale_byte = 127u;
        *inv_scale = 1.0f;
        return;
    }
    const uint32_t e = (amax_bits >> 7) & 0xFFu;     // biased exponent; floor(log2(amax)) = e - 127
    *scale_byte = e - 8u;                            // (e - 127 - emax) + 127 with emax = 8; e >= 87 here
    *inv_scale = __uint_as_float((262u - e) << 23);  // 2^-(e - 135)
}

__device__ __forceinline__ uint32_t to_e4m3(float x) {
    // round-to-nearest-even, saturating at +-448; NaN keeps its sign (0x7F / 0xFF) as torch's cast does
    if (x != x) return 0x7Fu | ((__float_as_uint(x) >> 24) & 0x80u);
    return static_cast<uint32_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}

// `has_nan`: the block holds a NaN (its largest |bits| is above Inf); only then is the per-value NaN
// handling needed — otherwise two values go through one cvt.rn.satfinite.e4m3x2.f32.
__device__ __forceinline__ uint2 quantise8(const uint4 &v, float inv_scale, bool has_nan) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t h[4];
    if (!has_nan) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = make_float2(__uint_as_float(w[i] << 16) * inv_scale,
                                         __uint_as_float(w[i] & 0xFFFF0000u) * inv_scale);
            h[i] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(f, __NV_SATFINITE, __NV_E4M3));   // .x in the low byte
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
            h[i] = to_e4m3(__uint_as_float(w[i] << 16) * inv_scale) |
                   (to_e4m3(__uint_as_float(w[i] & 0xFFFF0000u) * inv_scale) << 8);
    }
    uint2 r;
    r.x = h[0] | (h[1] << 16);
    r.y = h[2] | (h[3] << 16);
    return r;
}

// offset of (row, kb) inside the tcgen05 scale-factor atoms: atoms of 128 rows x 4 k-blocks
__device__ __host__ __forceinline__ size_t sf_atom_offset(uint32_t row, uint32_t kb, uint32_t kb4_count) {
    return (static_cast<size_t>(row >> 7) * kb4_count + (kb >> 2)) * 512 + (row & 31u) * 16 + ((row >> 5) & 3u) * 4 +
           (kb & 3u);
}

// 256-bit global accesses (one 32-byte sector per thread and instruction); addresses 32-byte aligned
struct alignas(32) Vec8 {
    uint4 lo, hi;
};
__device__ __forceinline__ Vec8 ld_stream_256(const void *p) {
    Vec8 v;
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(v.lo.x), "=r"(v.lo.y), "=r"(v.lo.z), "=r"(v.lo.w), "=r"(v.hi.x), "=r"(v.hi.y), "=r"(v.hi.z), "=r"(v.hi.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ void st_256(void *p, const uint2 &a, const uint2 &b, const uint2 &c, const uint2 &d) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(b.x), "r"(b.y),
                 "r"(c.x), "r"(c.y), "r"(d.x), "r"(d.y)
                 : "memory");
}

// One thread owns one whole 32-value block: 64 contiguous input bytes (two 256-bit loads, or four
// 128-bit ones when the buffers are only 16-byte aligned), the block's largest magnitude and scale
// without any exchange between threads, 32 contiguous code bytes (one 256-bit store) and one scale
// byte.  A warp covers 32 consecutive blocks, so every load and store instruction touches whole
// 32-byte sectors and a warp's scale bytes are one contiguous 32-byte run.  Blocks are walked flat
// over the matrix (grid-stride) with the (row, k-block) pair advanced incrementally.
// codes: [rows, k] bytes (row stride code_ld).  scales_rm: optional [rows, scale_ld] bytes.
// sf_atoms: optional tcgen05 atom layout.
template <bool WIDE>
__global__ void __launch_bounds__(256) mx_quant_kernel(const uint8_t *__restrict__ in, int rows, int k, uint8_t *codes,
                                                       size_t code_ld, uint8_t *scales_rm, int scale_ld,
                                                       uint8_t *sf_atoms, int kb4_count) {
    const int nblocks = k >> 5;
    const long long total = static_cast<long long>(rows) * nblocks;
    const long long stride = static_cast<long long>(gridDim.x) * 256;
    long long b = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x;
    if (b >= total) return;
    int row = static_cast<int>(b / nblocks);
    int kb = static_cast<int>(b - static_cast<long long>(row) * nblocks);
    const int step_row = static_cast<int>(stride / nblocks);
    const int step_kb = static_cast<int>(stride - static_cast<long long>(step_row) * nblocks);
    const size_t row_bytes = static_cast<size_t>(k) * 2;
    for (; b < total; b += stride) {
        const uint8_t *src = in + static_cast<size_t>(row) * row_bytes + static_cast<size_t>(kb) * 64;
        uint4 x[4];
        if (WIDE) {
            const Vec8 v0 = ld_stream_256(src), v1 = ld_stream_256(src + 32);
            x[0] = v0.lo;
            x[1] = v0.hi;
            x[2] = v1.lo;
            x[3] = v1.hi;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) x[i] = __ldg(reinterpret_cast<const uint4 *>(src) + i);
        }
        const uint32_t am = max(max(bf16_abs_max(x[0]), bf16_abs_max(x[1])), max(bf16_abs_max(x[2]), bf16_abs_max(x[3])));
        uint32_t sb;
        float inv;
        block_scale(am, &sb, &inv);
        const bool has_nan = am > 0x7F80u;
        uint2 q[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = quantise8(x[i], inv, has_nan);
        uint8_t *dst = codes + static_cast<size_t>(row) * code_ld + static_cast<size_t>(kb) * 32;
        if (WIDE) {
            st_256(dst, q[0], q[1], q[2], q[3]);
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<uint2 *>(dst + i * 8) = q[i];
        }
        if (scales_rm) {
            uint8_t *srow = scales_rm + static_cast<size_t>(row) * scale_ld;
            srow[kb] = static_cast<uint8_t>(sb);
            if (kb == nblocks - 1 && (nblocks & 1)) srow[kb + 1] = 127;      // rows are padded to an even count
        }
        if (sf_atoms) sf_atoms[sf_atom_offset(row, kb, kb4_count)] = static_cast<uint8_t>(sb);
        row += step_row;
        kb += step_kb;
        if (kb >= nblocks) {
            kb -= nblocks;
            ++row;
        }
    }
}

// scale bytes in one of the operator layouts -> tcgen05 atoms (pad positions keep the 127 = 1.0 fill)
//   kind 0: [rows, ld] row-major (activations, transposed weights)
//   kind 1: [kblocks/2, rows, 2]  (weights of a [K, N] operand: reference layout [K/64, N, 2])
__global__ void sf_to_atoms_kernel(const uint8_t *__restrict__ src, int kind, int rows, int kblocks, int ld,
                                   uint8_t *atoms, int kb4_count) {
    const size_t total = static_cast<size_t>(rows) * kblocks;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const uint32_t row = static_cast<uint32_t>(i / kblocks);
        const uint32_t kb = static_cast<uint32_t>(i - static_cast<size_t>(row) * kblocks);
        uint8_t v;
        if (kind == 0)
            v = src[static_cast<size_t>(row) * ld + kb];
        else
            v = src[(static_cast<size_t>(kb >> 1) * rows + row) * 2 + (kb & 1u)];
        atoms[sf_atom_offset(row, kb, kb4_count)] = v;
    }
}

// Row-major [rows, ld] scale bytes -> atoms through a shared-memory transpose: a CTA takes one
// 128-row tile and 16 k-block groups (64 scale bytes per row), reads 16-byte pieces of rows and writes
// whole 16-byte atom lines.  Needs 16-byte aligned rows (ld % 16 == 0).
__global__ void __launch_bounds__(256) sf_rows_to_atoms_kernel(const uint8_t *__restrict__ src, int rows, int kblocks,
                                                               int ld, uint8_t *atoms, int kb4_count) {
    __shared__ __align__(16) uint8_t tile[128][80];
    const int groups = (kb4_count + 15) / 16;
    const int row_tiles = (rows + 127) / 128;
    for (int w = blockIdx.x; w < row_tiles * groups; w += gridDim.x) {
        const int rt = w / groups, g = w - rt * groups;
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int idx = threadIdx.x + i * 256;
            const int r = idx >> 2, c16 = idx & 3;
            const int row = rt * 128 + r;
            const int byte0 = g * 64 + c16 * 16;
            uint4 v = make_uint4(0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu, 0x7F7F7F7Fu);
            if (row < rows && byte0 < ld) {
                v = *reinterpret_cast<const uint4 *>(src + static_cast<size_t>(row) * ld + byte0);
                // bytes past the last real k-block of the row are padding: neutral scale
                if (byte0 + 16 > kblocks) {
                    uint8_t *b = reinterpret_cast<uint8_t *>(&v);
                    for (int j = 0; j < 16; ++j)
                        if (byte0 + j >= kblocks) b[j] = 127;
                }
            }
            *reinterpret_cast<uint4 *>(&tile[r][c16 * 16]) = v;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int o = threadIdx.x + i * 256;
            const int a = o >> 5, l = o & 31;
            const int kb4 = g * 16 + a;
            if (kb4 >= kb4_count) continue;
            uint4 v;
            v.x = *reinterpret_cast<const uint32_t *>(&tile[l][a * 4]);
            v.y = *reinterpret_cast<const uint32_t *>(&tile[l + 32][a * 4]);
            v.z = *reinterpret_cast<const uint32_t *>(&tile[l + 64][a * 4]);
            v.w = *reinterpret_cast<const uint32_t *>(&tile[l + 96][a * 4]);
            *reinterpret_cast<uint4 *>(atoms + (static_cast<size_t>(rt) * kb4_count + kb4) * 512 + l * 16) = v;
        }
    }
}

}  // namespace

size_t sf_atoms_bytes(int rows, int k) {
    const size_t row_tiles = (static_cast<size_t>(rows) + 127) / 128;
    const size_t kb4 = (static_cast<size_t>(k) + 127) / 128;
    return row_tiles * kb4 * 512;
}

static int grid_for(size_t work_items, int threads) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    size_t blocks = (work_items + threads - 1) / threads;
    const size_t cap = static_cast<size_t>(sms) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

int mx_quant_launch(cudaStream_t stream, const void *in_bf16, int rows, int k, uint8_t *codes, size_t code_ld,
                    uint8_t *scales_rm, int scale_ld, uint8_t *sf_atoms) {
    if (rows <= 0 || k <= 0 || (k % 32) != 0) {
        set_error("MX quantisation needs rows > 0 and k a positive multiple of 32 (rows=%d k=%d)", rows, k);
        return CATCCOS_ERR_INVALID;
    }
    if (!in_bf16 || !codes || (reinterpret_cast<uintptr_t>(in_bf16) & 15) || (reinterpret_cast<uintptr_t>(codes) & 7) ||
        (code_ld & 7)) {
        set_error("MX quantisation: input must be 16-byte aligned, codes 8-byte aligned with a row stride multiple of 8");
        return CATCCOS_ERR_INVALID;
    }
    const int kb4 = (k + 127) / 128;
    if (sf_atoms) {
        cudaError_t e = cudaMemsetAsync(sf_atoms, 127, sf_atoms_bytes(rows, k), stream);
        if (e != cudaSuccess) {
            set_error("cudaMemsetAsync failed: %s", cudaGetErrorString(e));
            return CATCCOS_ERR_CUDA;
        }
    }
    // one thread per 32-value block; a grid of whole waves (all resident CTAs of every SM) walks the matrix
    const size_t blocks32 = static_cast<size_t>(rows) * (k / 32);
    const int grid = grid_for(blocks32, 256);
    const bool wide = (reinterpret_cast<uintptr_t>(in_bf16) & 31) == 0 && (reinterpret_cast<uintptr_t>(codes) & 31) == 0 &&
                      (code_ld & 31) == 0;
    if (wide)
        mx_quant_kernel<true><<<grid, 256, 0, stream>>>(static_cast<const uint8_t *>(in_bf16), rows, k, codes, code_ld,
                                                        scales_rm, scale_ld, sf_atoms, kb4);
    else
        mx_quant_kernel<false><<<grid, 256, 0, stream>>>(static_cast<const uint8_t *>(in_bf16), rows, k, codes, code_ld,
                                                         scales_rm, scale_ld, sf_atoms, kb4);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("mx_quant_kernel launch failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

int sf_to_atoms_launch(cudaStream_t stream, const uint8_t *src, int kind, int rows, int kblocks, int ld, uint8_t *atoms) {
    const int k = kblocks * 32;
    if (kind == 0 && (ld & 15) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(atoms) & 15) == 0) {
        // fast path: writes every byte of the atom buffer itself (padding included)
        const int kb4c = (k + 127) / 128;
        const size_t work = static_cast<size_t>((rows + 127) / 128) * ((kb4c + 15) / 16);
        sf_rows_to_atoms_kernel<<<grid_for(work * 256, 256), 256, 0, stream>>>(src, rows, kblocks, ld, atoms, kb4c);
        cudaError_t e2 = cudaGetLastError();
        if (e2 != cudaSuccess) {
            set_error("scale re-layout failed: %s", cudaGetErrorString(e2));
            return CATCCOS_ERR_CUDA;
        }
        return CATCCOS_OK;
    }
    cudaError_t e = cudaMemsetAsync(atoms, 127, sf_atoms_bytes(rows, k), stream);
    if (e == cudaSuccess) {
        const size_t total = static_cast<size_t>(rows) * kblocks;
        sf_to_atoms_kernel<<<grid_for(total, 256), 256, 0, stream>>>(src, kind, rows, kblocks, ld, atoms, (k + 127) / 128);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_error("scale re-layout failed: %s", cudaGetErrorString(e));
        return CATCCOS_ERR_CUDA;
    }
    return CATCCOS_OK;
}

}  // namespace cb

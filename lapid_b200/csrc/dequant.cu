// Dequantization to f32, bit-identical to lapid-quant, and the GGUF -> lapid layout conversion.
//
//   dequantize_q4k   crates/lapid-quant/src/kquant.rs:337-352   y = (d*sc)*q - (dmin*m)
//   dequantize_q5k   crates/lapid-quant/src/kquant.rs:355-373   y = (d*sc)*(q + 16*h) - (dmin*m)
//   dequantize_q6k   crates/lapid-quant/src/kquant.rs:376-396   y = (d*sc)*(q-32)
//   Int8 rows        crates/lapid-quant/src/imp.rs:143-148      y = f32(q) * f32(d)
//   Int4 rows        crates/lapid-quant/src/imp.rs:148-156      y = f32(nibble - 8) * f32(d)
//   from_ggml_blocks crates/lapid-quant/src/imp.rs:171-200
//
// One CTA of 256 threads expands one 256-element super-block (or eight Int8 groups); thread t
// owns element t, so stores are fully coalesced and the block's bytes are read through L1.
// The kernels are bound by the 4 bytes written per element (HBM store bandwidth).
#include "common.cuh"
#include "iquant.cuh"
#include "kernels.h"

namespace lb {

// element e (0..255) of the Q4_K super-block at b
__device__ __forceinline__ float q4k_element(const uint8_t *b, int e) {
    int j = e >> 6, h = (e >> 5) & 1, l = e & 31;
    float d = half_bits_to_float(b[0] | (b[1] << 8));
    float dmin = half_bits_to_float(b[2] | (b[3] << 8));
    int sc, mn;
    scale_min_k4(2 * j + h, b + 4, sc, mn);
    float d1 = xmul(d, (float)sc);
    float m1 = xmul(dmin, (float)mn);
    int q = (b[16 + 32 * j + l] >> (4 * h)) & 15;
    return xsub(xmul(d1, (float)q), m1);
}
// element e (0..255) of the Q5_K super-block at b: Q4_K's arithmetic with a fifth bit from qh
__device__ __forceinline__ float q5k_element(const uint8_t *b, int e) {
    int j = e >> 6, h = (e >> 5) & 1, l = e & 31;
    float d = half_bits_to_float(b[0] | (b[1] << 8));
    float dmin = half_bits_to_float(b[2] | (b[3] << 8));
    int sc, mn;
    scale_min_k4(2 * j + h, b + 4, sc, mn);
    float d1 = xmul(d, (float)sc);
    float m1 = xmul(dmin, (float)mn);
    int q = ((b[48 + 32 * j + l] >> (4 * h)) & 15) + (((b[16 + l] >> (2 * j + h)) & 1) << 4);
    return xsub(xmul(d1, (float)q), m1);
}
// element e (0..255) of the Q6_K super-block at b
__device__ __forceinline__ float q6k_element(const uint8_t *b, int e) {
    int n = e >> 7, w = (e >> 5) & 3, l = e & 31;
    float d = half_bits_to_float(b[208] | (b[209] << 8));
    int lo = (b[64 * n + 32 * (w & 1) + l] >> (4 * (w >> 1))) & 15;
    int hi = (b[128 + 32 * n + l] >> (2 * w)) & 3;
    int q = (lo | (hi << 4)) - 32;
    int sc = (int8_t)b[192 + 8 * n + 2 * w + (l >> 4)];
    return xmul(xmul(d, (float)sc), (float)q);
}

__global__ void __launch_bounds__(256) dequant_q4k_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst,
                                                          uint64_t n_blocks) {
    for (uint64_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x)
        dst[blk * QK + threadIdx.x] = q4k_element(src + blk * Q4K_BYTES, threadIdx.x);
}

__global__ void __launch_bounds__(256) dequant_q5k_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst,
                                                          uint64_t n_blocks) {
    for (uint64_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x)
        dst[blk * QK + threadIdx.x] = q5k_element(src + blk * Q5K_BYTES, threadIdx.x);
}

__global__ void __launch_bounds__(256) dequant_q6k_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst,
                                                          uint64_t n_blocks) {
    for (uint64_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x)
        dst[blk * QK + threadIdx.x] = q6k_element(src + blk * Q6K_BYTES, threadIdx.x);
}

// Gather: out[i, :] = dequant(table[ids[i], :]) (lapid's Kernel::Gather, crates/lapid-compiler/src/ir.rs:284-300;
// CPU: crates/lapid-cpu/src/rows.rs:164-215 -- the embedding lookup from a quantized table). One CTA
// per (output row, 256 columns); an index outside [0, rows) is not read: the row is skipped and bit
// 128 of the host-visible status word reports it ("index_out_of_range" after the launch sequence).
template <int FMT>
__global__ void __launch_bounds__(256) gather_kernel(const uint8_t *__restrict__ table, uint64_t scales_offset,
                                                     const int32_t *__restrict__ ids, uint64_t rows, uint64_t cols, uint64_t count,
                                                     float *__restrict__ out, int *status, const uint8_t *__restrict__ iq_grid = nullptr) {
    const uint64_t per_row = (cols + 255) / 256;
    for (uint64_t u = blockIdx.x; u < count * per_row; u += gridDim.x) {
        const uint64_t i = u / per_row, c = (u % per_row) * 256 + threadIdx.x;
        const int64_t r = ids[i];
        if (r < 0 || (uint64_t)r >= rows) {
            if (threadIdx.x == 0 && status) atomicOr(status, 128);
            continue;
        }
        if (c >= cols) continue;
        float v;
        if (FMT == FMT_Q4K) v = q4k_element(table + ((uint64_t)r * (cols / QK) + c / QK) * Q4K_BYTES, (int)(c % QK));
        else if (FMT == FMT_Q5K) v = q5k_element(table + ((uint64_t)r * (cols / QK) + c / QK) * Q5K_BYTES, (int)(c % QK));
        else if (FMT == FMT_Q6K) v = q6k_element(table + ((uint64_t)r * (cols / QK) + c / QK) * Q6K_BYTES, (int)(c % QK));
        else if (FMT == FMT_MXFP4) v = mxfp4_element(table + (((uint64_t)r * cols + c) >> 5) * MXFP4_BYTES, (uint32_t)(c & 31));
        else if (is_iq(FMT)) v = iq_element<FMT>(table + ((uint64_t)r * (cols / QK) + c / QK) * iq_block_bytes(FMT), (int)(c % QK), iq_grid);
        else if (FMT == FMT_INT4) {
            const uint64_t pos = (uint64_t)r * cols + c, g = pos >> 5;
            const uint32_t e = (uint32_t)(pos & 31);
            const uint8_t b = table[g * 16 + (e & 15)];
            v = xmul((float)((int)((e < 16 ? b : (b >> 4)) & 15) - 8), half_bits_to_float(((const uint16_t *)(table + scales_offset))[g]));
        } else if (FMT == FMT_INT8)
            v = xmul((float)((const int8_t *)table)[(uint64_t)r * cols + c],
                     half_bits_to_float(((const uint16_t *)(table + scales_offset))[((uint64_t)r * cols + c) >> 5]));
        else v = ((const float *)table)[(uint64_t)r * cols + c];
        out[i * cols + c] = v;
    }
}

// element c of row-major position `pos` = r * cols + c in an Int4 plane (crates/lapid-quant/src/imp.rs:148-156)
__device__ __forceinline__ float int4_element(const uint8_t *qs, const uint16_t *scales, uint64_t pos) {
    const uint64_t g = pos >> 5;
    const uint32_t e = (uint32_t)(pos & 31);
    const uint8_t b = qs[g * 16 + (e & 15)];
    const int q = (int)((e < 16 ? b : (b >> 4)) & 15) - 8;
    return xmul((float)q, half_bits_to_float(scales[g]));
}

__global__ void __launch_bounds__(256) dequant_int4_kernel(const uint8_t *__restrict__ qs, const uint16_t *__restrict__ scales,
                                                           float *__restrict__ dst, uint64_t n_elems) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += stride) dst[i] = int4_element(qs, scales, i);
}

// one CTA per i-quant block, one thread per element (crates/lapid-quant/src/iq2.rs:38-90, iq3.rs:18-39)
template <int FMT>
__global__ void __launch_bounds__(256) dequant_iq_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst, uint64_t n_blocks,
                                                         const uint8_t *__restrict__ grid) {
    for (uint64_t blk = blockIdx.x; blk < n_blocks; blk += gridDim.x)
        dst[blk * QK + threadIdx.x] = iq_element<FMT>(src + blk * iq_block_bytes(FMT), threadIdx.x, grid);
}

__global__ void __launch_bounds__(256) dequant_mxfp4_kernel(const uint8_t *__restrict__ src, float *__restrict__ dst, uint64_t n_elems) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += stride)
        dst[i] = mxfp4_element(src + (i >> 5) * MXFP4_BYTES, (uint32_t)(i & 31));
}

// GGUF block_q4_0 (f16 d + 16 nibble bytes, 18 bytes) -> nibble plane + scales plane: the same nibble order.
__global__ void __launch_bounds__(256) q4_0_to_planes_kernel(const uint8_t *__restrict__ blocks, uint8_t *__restrict__ qs,
                                                             uint8_t *__restrict__ scales, uint64_t n_groups) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups * 16; i += stride) {
        uint64_t g = i >> 4;
        int t = (int)(i & 15);
        const uint8_t *b = blocks + g * 18;
        qs[i] = b[2 + t];
        if (t < 2) scales[g * 2 + t] = b[t];
    }
}

__global__ void __launch_bounds__(256) dequant_int8_kernel(const int8_t *__restrict__ qs,
                                                           const uint16_t *__restrict__ scales,
                                                           float *__restrict__ dst, uint64_t n_elems) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += stride) {
        float d = half_bits_to_float(scales[i >> 5]);
        dst[i] = xmul((float)qs[i], d);
    }
}

// GGUF block_q8_0 (f16 d + 32 x i8, 34 bytes) -> quants plane + scales plane. One thread per byte
// of payload; thread 0 of each group also moves the scale.
__global__ void __launch_bounds__(256) q8_0_to_planes_kernel(const uint8_t *__restrict__ blocks,
                                                             uint8_t *__restrict__ qs, uint8_t *__restrict__ scales,
                                                             uint64_t n_groups) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_groups * 32; i += stride) {
        uint64_t g = i >> 5;
        int t = (int)(i & 31);
        const uint8_t *b = blocks + g * 34;
        qs[i] = b[2 + t];
        if (t < 2) scales[g * 2 + t] = b[t];
    }
}

static int grid_for(uint64_t work_items, int sm_count) {
    uint64_t want = work_items;
    uint64_t cap = (uint64_t)sm_count * 8;  // 8 resident CTAs of 256 threads per SM
    return (int)(want < cap ? (want ? want : 1) : cap);
}

cudaError_t launch_dequantize(int fmt, const void *src, uint64_t rows, uint64_t cols, uint64_t scales_offset,
                              float *dst, int sm_count, cudaStream_t stream) {
    uint64_t n = rows * cols;
    if (n == 0) return cudaSuccess;
    if (fmt == FMT_Q4K) {
        dequant_q4k_kernel<<<grid_for(n / QK, sm_count), 256, 0, stream>>>((const uint8_t *)src, dst, n / QK);
    } else if (fmt == FMT_Q5K) {
        dequant_q5k_kernel<<<grid_for(n / QK, sm_count), 256, 0, stream>>>((const uint8_t *)src, dst, n / QK);
    } else if (fmt == FMT_Q6K) {
        dequant_q6k_kernel<<<grid_for(n / QK, sm_count), 256, 0, stream>>>((const uint8_t *)src, dst, n / QK);
    } else if (fmt == FMT_MXFP4) {
        dequant_mxfp4_kernel<<<grid_for((n + 255) / 256, sm_count), 256, 0, stream>>>((const uint8_t *)src, dst, n);
    } else if (is_iq(fmt)) {
        const uint8_t *grids = iq_grids();
        if (!grids) return cudaErrorNotReady;
        const uint8_t *g = grids + iq_grid_offset(fmt), *b = (const uint8_t *)src;
        const int ctas = grid_for(n / QK, sm_count);
        if (fmt == FMT_IQ2XXS) dequant_iq_kernel<FMT_IQ2XXS><<<ctas, 256, 0, stream>>>(b, dst, n / QK, g);
        else if (fmt == FMT_IQ2XS) dequant_iq_kernel<FMT_IQ2XS><<<ctas, 256, 0, stream>>>(b, dst, n / QK, g);
        else if (fmt == FMT_IQ2S) dequant_iq_kernel<FMT_IQ2S><<<ctas, 256, 0, stream>>>(b, dst, n / QK, g);
        else dequant_iq_kernel<FMT_IQ3XXS><<<ctas, 256, 0, stream>>>(b, dst, n / QK, g);
    } else if (fmt == FMT_INT4) {
        const uint8_t *p = (const uint8_t *)src;
        dequant_int4_kernel<<<grid_for((n + 255) / 256, sm_count), 256, 0, stream>>>(p, (const uint16_t *)(p + scales_offset), dst, n);
    } else {
        const uint8_t *p = (const uint8_t *)src;
        dequant_int8_kernel<<<grid_for((n + 255) / 256, sm_count), 256, 0, stream>>>(
            (const int8_t *)p, (const uint16_t *)(p + scales_offset), dst, n);
    }
    return cudaGetLastError();
}

// fmt < 0: plain f32 table
cudaError_t launch_gather(int fmt, const void *table, uint64_t scales_offset, const int32_t *ids, uint64_t rows, uint64_t cols,
                          uint64_t count, float *out, int *status, int sm_count, cudaStream_t stream) {
    if (count == 0 || cols == 0) return cudaSuccess;
    const int grid = grid_for(count * ((cols + 255) / 256), sm_count);
    const uint8_t *t = (const uint8_t *)table;
    if (fmt == FMT_Q4K) gather_kernel<FMT_Q4K><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status);
    else if (fmt == FMT_Q5K) gather_kernel<FMT_Q5K><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status);
    else if (fmt == FMT_Q6K) gather_kernel<FMT_Q6K><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status);
    else if (fmt == FMT_INT8) gather_kernel<FMT_INT8><<<grid, 256, 0, stream>>>(t, scales_offset, ids, rows, cols, count, out, status);
    else if (fmt == FMT_INT4) gather_kernel<FMT_INT4><<<grid, 256, 0, stream>>>(t, scales_offset, ids, rows, cols, count, out, status);
    else if (fmt == FMT_MXFP4) gather_kernel<FMT_MXFP4><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status);
    else if (is_iq(fmt)) {
        const uint8_t *grids = iq_grids();
        if (!grids) return cudaErrorNotReady;
        const uint8_t *g = grids + iq_grid_offset(fmt);
        if (fmt == FMT_IQ2XXS) gather_kernel<FMT_IQ2XXS><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status, g);
        else if (fmt == FMT_IQ2XS) gather_kernel<FMT_IQ2XS><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status, g);
        else if (fmt == FMT_IQ2S) gather_kernel<FMT_IQ2S><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status, g);
        else gather_kernel<FMT_IQ3XXS><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status, g);
    }
    else gather_kernel<-1><<<grid, 256, 0, stream>>>(t, 0, ids, rows, cols, count, out, status);
    return cudaGetLastError();
}

cudaError_t launch_q4_0_to_planes(const void *blocks, void *dst, uint64_t scales_offset, uint64_t n_groups,
                                  int sm_count, cudaStream_t stream) {
    if (n_groups == 0) return cudaSuccess;
    uint8_t *d = (uint8_t *)dst;
    q4_0_to_planes_kernel<<<grid_for((n_groups * 16 + 255) / 256, sm_count), 256, 0, stream>>>(
        (const uint8_t *)blocks, d, d + scales_offset, n_groups);
    return cudaGetLastError();
}

cudaError_t launch_q8_0_to_planes(const void *blocks, void *dst, uint64_t scales_offset, uint64_t n_groups,
                                  int sm_count, cudaStream_t stream) {
    if (n_groups == 0) return cudaSuccess;
    uint8_t *d = (uint8_t *)dst;
    q8_0_to_planes_kernel<<<grid_for((n_groups * 32 + 255) / 256, sm_count), 256, 0, stream>>>(
        (const uint8_t *)blocks, d, d + scales_offset, n_groups);
    return cudaGetLastError();
}

}  // namespace lb

// Exact-f32 quantized GEMM: f32 activations x weights dequantized to f32 with lapid-quant's
// arithmetic, every output accumulated over k = 0..K-1 in order with one fused multiply-add per
// term from a zero accumulator. That is the arithmetic of lapid-cpu's `qdeq` path on x86-64 with
// AVX2+FMA (crates/lapid-cpu/src/matmul/qdeq.rs:57-123, kernels.rs:95-119), so results are
// bit-identical to it. This is the reference-exact path for more than 8 activation rows; the
// tensor-core kernel is the fast one.
//
// Expert-indexed launches (Kernel::MatMulId above decode sizes) run through the same kernel: the
// activation tiles are runs of (token, slot) pairs grouped by expert (moe.cu), a tile looks up its
// expert's matrix, rows are gathered and scattered through the pair table. Every output is still
// the in-order FMA sum over k, i.e. what lapid-cpu's per-expert matmul gives
// (crates/lapid-cpu/src/moe.rs:80-118 with float_act, :109).
//
// CUDA-core kernel: 64x64 output tile per CTA, 4x4 register tile per thread, k in steps of one
// 32-element group; the W tile is expanded into shared memory once per step (so each weight is
// dequantized once per 64 activation rows) and A is staged beside it.
#include "common.cuh"
#include "iquant.cuh"
#include "kernels.h"

namespace lb {

constexpr int BM = 64, BN = 64, BK = 32, PADF = 4;

// Eight consecutive elements k0..k0+7 (k0 % 8 == 0) of weight row `row`, bit-exact dequant.
template <int FMT>
__device__ __forceinline__ void dequant8(const GemmF32Args &p, uint32_t row, uint32_t k0, float (&y)[8]) {
    if constexpr (FMT == FMT_Q4K) {
        const uint8_t *b = p.w + ((uint64_t)row * (p.k / QK) + k0 / QK) * Q4K_BYTES;
        uint32_t e = k0 % QK, j = e >> 6, h = (e >> 5) & 1, l0 = e & 31;
        float d = half_bits_to_float(b[0] | (b[1] << 8)), dmin = half_bits_to_float(b[2] | (b[3] << 8));
        int sc, mn;
        scale_min_k4(2 * j + h, b + 4, sc, mn);
        float d1 = xmul(d, (float)sc), m1 = xmul(dmin, (float)mn);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int q = (b[16 + 32 * j + l0 + i] >> (4 * h)) & 15;
            y[i] = xsub(xmul(d1, (float)q), m1);
        }
    } else if constexpr (FMT == FMT_Q5K) {
        const uint8_t *b = p.w + ((uint64_t)row * (p.k / QK) + k0 / QK) * Q5K_BYTES;
        uint32_t e = k0 % QK, j = e >> 6, h = (e >> 5) & 1, l0 = e & 31;
        float d = half_bits_to_float(b[0] | (b[1] << 8)), dmin = half_bits_to_float(b[2] | (b[3] << 8));
        int sc, mn;
        scale_min_k4(2 * j + h, b + 4, sc, mn);
        float d1 = xmul(d, (float)sc), m1 = xmul(dmin, (float)mn);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int q = ((b[48 + 32 * j + l0 + i] >> (4 * h)) & 15) + (((b[16 + l0 + i] >> (2 * j + h)) & 1) << 4);
            y[i] = xsub(xmul(d1, (float)q), m1);
        }
    } else if constexpr (FMT == FMT_Q6K) {
        const uint8_t *b = p.w + ((uint64_t)row * (p.k / QK) + k0 / QK) * Q6K_BYTES;
        uint32_t e = k0 % QK, nh = e >> 7, w = (e >> 5) & 3, l0 = e & 31;
        float d = half_bits_to_float(b[208] | (b[209] << 8));
        float t = xmul(d, (float)(int8_t)b[192 + 8 * nh + 2 * w + (l0 >> 4)]);
#pragma unroll
        for (int i = 0; i < 8; i++) {
            int lo = (b[64 * nh + 32 * (w & 1) + l0 + i] >> (4 * (w >> 1))) & 15;
            int hi = (b[128 + 32 * nh + l0 + i] >> (2 * w)) & 3;
            y[i] = xmul(t, (float)((lo | (hi << 4)) - 32));
        }
    } else if constexpr (FMT == FMT_MXFP4) {
        const uint8_t *b = p.w + (((uint64_t)row * p.k + k0) / GROUP) * MXFP4_BYTES;
        const uint32_t e = k0 % GROUP;  // 0, 8, 16 or 24
#pragma unroll
        for (int i = 0; i < 8; i++) y[i] = mxfp4_element(b, e + i);
    } else if constexpr (is_iq(FMT)) {  // one 8-group: y = db * grid byte * sign (crates/lapid-quant/src/iq2.rs:38-90, iq3.rs:18-39)
        const uint8_t *b = p.w + ((uint64_t)row * (p.k / QK) + k0 / QK) * iq_block_bytes(FMT);
        const uint32_t e = k0 % QK;
        uint32_t lo, hi, signs;
        iq_group8<FMT>(b, (int)(e >> 3), p.iq_grid, lo, hi, signs);
        const float db = iq_half_scale<FMT>(b, (int)(e >> 4));
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float v = xmul(db, (float)(((i < 4 ? lo : hi) >> (8 * (i & 3))) & 255u));
            y[i] = (signs >> i) & 1u ? -v : v;
        }
    } else if constexpr (FMT == FMT_INT4) {
        const uint64_t g = ((uint64_t)row * p.k + k0) / GROUP;
        const uint32_t e = k0 % GROUP;  // 0, 8, 16 or 24: elements 16.. are the high nibbles of the same bytes
        const uint8_t *b = p.w + g * 16 + (e & 15);
        const float d = half_bits_to_float(((const uint16_t *)(p.w + p.scales_offset))[g]);
#pragma unroll
        for (int i = 0; i < 8; i++) y[i] = xmul((float)((int)((e < 16 ? b[i] : (b[i] >> 4)) & 15) - 8), d);
    } else {
        const int8_t *q = (const int8_t *)p.w + (uint64_t)row * p.k + k0;
        const uint16_t *s = (const uint16_t *)(p.w + p.scales_offset);
        float d = half_bits_to_float(s[(uint64_t)row * (p.k / GROUP) + k0 / GROUP]);
#pragma unroll
        for (int i = 0; i < 8; i++) y[i] = xmul((float)q[i], d);
    }
}

template <int FMT> __global__ void __launch_bounds__(256) qgemm_f32_kernel(GemmF32Args p) {
    __shared__ float As[BK][BM + PADF];
    __shared__ float Bs[BK][BN + PADF];
    const int tid = threadIdx.x;
    const uint32_t row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    if (p.tile_expert) {  // expert-indexed launch (moe.cu): this activation tile multiplies one expert's matrix
        const int32_t e = p.tile_expert[blockIdx.y];
        if (e < 0) return;
        p.w += (uint64_t)e * p.id_stride;
    }
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;

    const int lr = tid >> 2, part = tid & 3;  // loader role: tile row / weight row, 8-element part
    const uint32_t arow = row0 + lr;
    const void *aptr = nullptr;
    if (p.tile_expert) {
        const int32_t pair = p.row_pair[arow];
        if (pair >= 0) aptr = (const char *)p.a + (p.a_off + (uint64_t)((uint32_t)pair / p.id_r) * p.a_rs) * act_elem_bytes(p.a_type);
    } else if (arow < p.rows) {
        aptr = act_row(p.a, p.a_type, p.a_off, p.a_bs, p.a_rs, arow, p.m);
    }
    const uint32_t wrow = col0 + lr;

    for (uint32_t k0 = 0; k0 < p.k; k0 += BK) {
        float av[8], wv[8];
#pragma unroll
        for (int i = 0; i < 8; i++) av[i] = aptr ? load_act(aptr, k0 + part * 8 + i, p.a_type) : 0.0f;
        if (wrow < p.n) {
            dequant8<FMT>(p, wrow, k0 + part * 8, wv);
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) wv[i] = 0.0f;
        }
        __syncthreads();  // previous step's readers are done
#pragma unroll
        for (int i = 0; i < 8; i++) {
            As[part * 8 + i][lr] = av[i];
            Bs[part * 8 + i][lr] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float4 a4 = *(const float4 *)&As[kk][ty * 4];
            float4 b4 = *(const float4 *)&Bs[kk][tx * 4];
            float a_[4] = {a4.x, a4.y, a4.z, a4.w}, b_[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a_[i], b_[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        uint32_t r = row0 + ty * 4 + i;
        if (r >= p.rows) continue;
        if (p.tile_expert) {
            const int32_t pair = p.row_pair[r];
            if (pair < 0) continue;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t col = col0 + tx * 4 + j;
                if (col < p.n) p.out[p.out_off + (uint64_t)pair * p.n + col] = acc[i][j];
            }
            continue;
        }
        uint32_t bt = r / p.m, ii = r % p.m;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint32_t col = col0 + tx * 4 + j;
            if (col >= p.n) continue;
            float v = acc[i][j];
            if (p.extra) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)ii * p.ex_s1 + (int64_t)col * p.ex_s2];
            p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)ii * p.out_rs + col] = v;
        }
    }
}

cudaError_t launch_qgemm_f32(int fmt, const GemmF32Args &a, cudaStream_t stream) {
    if (a.rows == 0 || a.n == 0) return cudaSuccess;
    dim3 grid((a.n + BN - 1) / BN, (a.rows + BM - 1) / BM);
    if (grid.y > 65535) return cudaErrorInvalidValue;
    switch (fmt) {
        case FMT_Q4K: qgemm_f32_kernel<FMT_Q4K><<<grid, 256, 0, stream>>>(a); break;
        case FMT_Q5K: qgemm_f32_kernel<FMT_Q5K><<<grid, 256, 0, stream>>>(a); break;
        case FMT_Q6K: qgemm_f32_kernel<FMT_Q6K><<<grid, 256, 0, stream>>>(a); break;
        case FMT_INT8: qgemm_f32_kernel<FMT_INT8><<<grid, 256, 0, stream>>>(a); break;
        case FMT_INT4: qgemm_f32_kernel<FMT_INT4><<<grid, 256, 0, stream>>>(a); break;
        case FMT_MXFP4: qgemm_f32_kernel<FMT_MXFP4><<<grid, 256, 0, stream>>>(a); break;
        case FMT_IQ2XXS:
        case FMT_IQ2XS:
        case FMT_IQ2S:
        case FMT_IQ3XXS: {
            const uint8_t *grids = iq_grids();
            if (!grids) return cudaErrorNotReady;
            GemmF32Args b = a;
            b.iq_grid = grids + iq_grid_offset(fmt);
            if (fmt == FMT_IQ2XXS) qgemm_f32_kernel<FMT_IQ2XXS><<<grid, 256, 0, stream>>>(b);
            else if (fmt == FMT_IQ2XS) qgemm_f32_kernel<FMT_IQ2XS><<<grid, 256, 0, stream>>>(b);
            else if (fmt == FMT_IQ2S) qgemm_f32_kernel<FMT_IQ2S><<<grid, 256, 0, stream>>>(b);
            else qgemm_f32_kernel<FMT_IQ3XXS><<<grid, 256, 0, stream>>>(b);
            break;
        }
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

}  // namespace lb

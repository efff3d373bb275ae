// Weight quantizers on the device, byte-identical to lapid-quant's reference quantizers.
//
//   Q4_K  crates/lapid-quant/src/kquant.rs:42-121 (make_qkx2_quants), :188-260
//   Q5_K  the same search with 5-bit levels (nmax 31, rmin -0.5, 15 steps), :263-287
//   Q6_K  crates/lapid-quant/src/kquant.rs:124-174 (make_qx_quants, rmse_type 1), :290-334
//   Int8  crates/lapid-quant/src/imp.rs:24-40, :95-115
//
// The searches are sequential f32 recurrences whose rounding order defines the output bytes, so
// the parallelism is across sub-blocks, never inside one: one thread owns one sub-block (32
// values for Q4_K, 16 for Q6_K) and runs the reference's loops in the reference's order with
// separately rounded operations; the 8 / 16 threads of a super-block then agree on the block
// scale through warp shuffles, and the quants are packed through shared memory so the stores
// are whole bytes. Compile this file with -fmad=false as a second guard against contraction.
#include "common.cuh"
#include "kernels.h"

namespace lb {

__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

// Asymmetric (scale, min) search for one 32-value sub-block; L receives the chosen levels.
template <int FMT> __device__ float make_qkx2_32(const float *x, const float *w, uint8_t *L, uint8_t *Laux, float &the_min) {
    const int n = 32, nmax = FMT == FMT_Q5K ? 31 : 15, nstep = FMT == FMT_Q5K ? 15 : 20;
    const float rmin = FMT == FMT_Q5K ? -0.5f : -1.0f, rdelta = 0.1f;
    float mn = x[0], mx = x[0];
    float sum_w = w[0];
    float sum_x = xmul(sum_w, x[0]);
    for (int i = 1; i < n; i++) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
        sum_w = xadd(sum_w, w[i]);
        sum_x = xadd(sum_x, xmul(w[i], x[i]));
    }
    if (mn > 0.0f) mn = 0.0f;
    if (mx == mn) {
        for (int i = 0; i < n; i++) L[i] = 0;
        the_min = -mn;
        return 0.0f;
    }
    float iscale = xdiv((float)nmax, xsub(mx, mn));
    float scale = xdiv(1.0f, iscale);
    float best = 0.0f;
    for (int i = 0; i < n; i++) {
        int l = clampi(nearest_int(xmul(iscale, xsub(x[i], mn))), 0, nmax);
        L[i] = (uint8_t)l;
        float diff = xsub(xadd(xmul(scale, (float)l), mn), x[i]);
        best = xadd(best, xmul(w[i], xmul(diff, diff)));
    }
    for (int is = 0; is <= nstep; is++) {
        iscale = xdiv(xadd(xadd(rmin, xmul(rdelta, (float)is)), (float)nmax), xsub(mx, mn));
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; i++) {
            int l = clampi(nearest_int(xmul(iscale, xsub(x[i], mn))), 0, nmax);
            Laux[i] = (uint8_t)l;
            float wi = w[i], lf = (float)l;
            sum_l = xadd(sum_l, xmul(wi, lf));
            sum_l2 = xadd(sum_l2, xmul(xmul(wi, lf), lf));
            sum_xl = xadd(sum_xl, xmul(xmul(wi, lf), x[i]));
        }
        float D = xsub(xmul(sum_w, sum_l2), xmul(sum_l, sum_l));
        if (D > 0.0f) {
            float this_scale = xdiv(xsub(xmul(sum_w, sum_xl), xmul(sum_x, sum_l)), D);
            float this_min = xdiv(xsub(xmul(sum_l2, sum_x), xmul(sum_l, sum_xl)), D);
            if (this_min > 0.0f) {
                this_min = 0.0f;
                this_scale = xdiv(sum_xl, sum_l2);
            }
            float cur = 0.0f;
            for (int i = 0; i < n; i++) {
                float diff = xsub(xadd(xmul(this_scale, (float)Laux[i]), this_min), x[i]);
                cur = xadd(cur, xmul(w[i], xmul(diff, diff)));
            }
            if (cur < best) {
                for (int i = 0; i < n; i++) L[i] = Laux[i];
                best = cur;
                scale = this_scale;
                mn = this_min;
            }
        }
    }
    the_min = -mn;
    return scale;
}

constexpr int Q4_BLOCKS_PER_CTA = 32;  // 8 threads per super-block, 256 threads

template <int FMT>
__global__ void __launch_bounds__(256) quantize_q4k_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                           uint64_t n_blocks) {
    constexpr int BB = FMT == FMT_Q5K ? Q5K_BYTES : Q4K_BYTES, NMAX = FMT == FMT_Q5K ? 31 : 15;
    __shared__ uint8_t sL[Q4_BLOCKS_PER_CTA][QK];
    const int tid = threadIdx.x;
    const int lb_ = tid >> 3;  // super-block within the CTA
    const int j = tid & 7;     // sub-block within the super-block
    for (uint64_t base = (uint64_t)blockIdx.x * Q4_BLOCKS_PER_CTA; base < n_blocks;
         base += (uint64_t)gridDim.x * Q4_BLOCKS_PER_CTA) {
        uint64_t blk = base + lb_;
        bool live = blk < n_blocks;
        float x[32], w[32];
        uint8_t L[32], Laux[32];
        float scale = 0.0f, mn = 0.0f;
        if (live) {
            const float4 *xp = (const float4 *)(src + blk * QK + 32 * j);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float4 v = xp[i];
                x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
            }
            float sum_x2 = 0.0f;
            for (int i = 0; i < 32; i++) sum_x2 = xadd(sum_x2, xmul(x[i], x[i]));
            float av_x = __fsqrt_rn(xdiv(sum_x2, 32.0f));
            for (int i = 0; i < 32; i++) w[i] = xadd(av_x, fabsf(x[i]));
            scale = make_qkx2_32<FMT>(x, w, L, Laux, mn);
        }
        // the eight threads of a super-block are eight consecutive lanes: exchange by shuffle
        float scales[8], mins[8];
#pragma unroll
        for (int t = 0; t < 8; t++) {
            scales[t] = __shfl_sync(0xffffffffu, scale, (tid & 24) + t);
            mins[t] = __shfl_sync(0xffffffffu, mn, (tid & 24) + t);
        }
        float max_scale = 0.0f, max_min = 0.0f;
#pragma unroll
        for (int t = 0; t < 8; t++) {
            if (scales[t] > max_scale) max_scale = scales[t];
            if (mins[t] > max_min) max_min = mins[t];
        }
        float inv_scale = max_scale > 0.0f ? xdiv(63.0f, max_scale) : 0.0f;
        float inv_min = max_min > 0.0f ? xdiv(63.0f, max_min) : 0.0f;
        uint8_t ls[8], lm[8];
#pragma unroll
        for (int t = 0; t < 8; t++) {
            // the C original stores nearest_int() in a uint8_t (wraps) before MIN(63, .)
            uint8_t a = (uint8_t)nearest_int(xmul(inv_scale, scales[t]));
            uint8_t b = (uint8_t)nearest_int(xmul(inv_min, mins[t]));
            ls[t] = a > 63 ? 63 : a;
            lm[t] = b > 63 ? 63 : b;
        }
        __half dh = __float2half_rn(xdiv(max_scale, 63.0f));
        __half mh = __float2half_rn(xdiv(max_min, 63.0f));
        if (live) {
            float d = xmul(__half2float(dh), (float)ls[j]);
            if (d != 0.0f) {
                float dm = xmul(__half2float(mh), (float)lm[j]);
                for (int i = 0; i < 32; i++) L[i] = (uint8_t)clampi(nearest_int(xdiv(xadd(x[i], dm), d)), 0, NMAX);
            }
            for (int i = 0; i < 32; i++) sL[lb_][32 * j + i] = L[i];
            if (j == 0) {
                uint8_t *out = dst + blk * BB;
                unsigned short dbits = __half_as_ushort(dh), mbits = __half_as_ushort(mh);
                out[0] = dbits & 0xff; out[1] = dbits >> 8;
                out[2] = mbits & 0xff; out[3] = mbits >> 8;
                uint8_t sc[12];
                for (int t = 0; t < 12; t++) sc[t] = 0;
                for (int t = 0; t < 8; t++) {
                    if (t < 4) {
                        sc[t] = ls[t];
                        sc[t + 4] = lm[t];
                    } else {
                        sc[t + 4] = (ls[t] & 0xF) | ((lm[t] & 0xF) << 4);
                        sc[t - 4] |= (ls[t] >> 4) << 6;
                        sc[t] |= (lm[t] >> 4) << 6;
                    }
                }
                for (int t = 0; t < 12; t++) out[4 + t] = sc[t];
            }
        }
        __syncthreads();
        // pack nibbles: byte i of pair k = L[64k + i] | L[64k + 32 + i] << 4; 128 bytes per block
        for (int o = tid; o < Q4_BLOCKS_PER_CTA * 128; o += 256) {
            int b = o >> 7, t = o & 127;
            uint64_t gb = base + b;
            if (gb < n_blocks) {
                int k = t >> 5, i = t & 31;
                dst[gb * BB + (FMT == FMT_Q5K ? 48 : 16) + t] = (sL[b][64 * k + i] & 15) | ((sL[b][64 * k + 32 + i] & 15) << 4);
            }
        }
        if constexpr (FMT == FMT_Q5K) {  // the fifth bits: bit s of qh[i] belongs to element 32 s + i
            for (int o = tid; o < Q4_BLOCKS_PER_CTA * 32; o += 256) {
                int b = o >> 5, i = o & 31;
                uint64_t gb = base + b;
                if (gb < n_blocks) {
                    uint8_t h = 0;
#pragma unroll
                    for (int sblk = 0; sblk < 8; sblk++) h |= (uint8_t)((sL[b][32 * sblk + i] >> 4) << sblk);
                    dst[gb * BB + 16 + i] = h;
                }
            }
        }
        __syncthreads();
    }
}

// Symmetric search for one 16-value sub-block (nmax 32). L receives l + 32.
__device__ float make_qx_rmse1_16(const float *x, int8_t *L) {
    const int n = 16, nmax = 32;
    float mx = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; i++) {
        float ax = fabsf(x[i]);
        if (ax > amax) {
            amax = ax;
            mx = x[i];
        }
    }
    if (amax < 1e-15f) {
        for (int i = 0; i < n; i++) L[i] = 0;
        return 0.0f;
    }
    float iscale = xdiv(-(float)nmax, mx);
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; i++) {
        int l = clampi(nearest_int(xmul(iscale, x[i])), -nmax, nmax - 1);
        L[i] = (int8_t)(l + nmax);
        float w = xmul(x[i], x[i]);
        float lf = (float)l;
        sumlx = xadd(sumlx, xmul(xmul(w, x[i]), lf));
        suml2 = xadd(suml2, xmul(xmul(w, lf), lf));
    }
    float scale = suml2 != 0.0f ? xdiv(sumlx, suml2) : 0.0f;
    float best = xmul(scale, sumlx);
    for (int is = -9; is <= 9; is++) {
        if (is == 0) continue;
        iscale = xdiv(-xadd((float)nmax, xmul(0.1f, (float)is)), mx);
        sumlx = 0.0f;
        suml2 = 0.0f;
        for (int i = 0; i < n; i++) {
            float lf = (float)clampi(nearest_int(xmul(iscale, x[i])), -nmax, nmax - 1);
            float w = xmul(x[i], x[i]);
            sumlx = xadd(sumlx, xmul(xmul(w, x[i]), lf));
            suml2 = xadd(suml2, xmul(xmul(w, lf), lf));
        }
        if (suml2 > 0.0f && xmul(sumlx, sumlx) > xmul(best, suml2)) {
            for (int i = 0; i < n; i++) L[i] = (int8_t)(nmax + clampi(nearest_int(xmul(iscale, x[i])), -nmax, nmax - 1));
            scale = xdiv(sumlx, suml2);
            best = xmul(scale, sumlx);
        }
    }
    return scale;
}

constexpr int Q6_BLOCKS_PER_CTA = 16;  // 16 threads per super-block

__global__ void __launch_bounds__(256) quantize_q6k_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst,
                                                           uint64_t n_blocks) {
    __shared__ uint8_t sL[Q6_BLOCKS_PER_CTA][QK];
    const int tid = threadIdx.x;
    const int lb_ = tid >> 4;
    const int j = tid & 15;
    for (uint64_t base = (uint64_t)blockIdx.x * Q6_BLOCKS_PER_CTA; base < n_blocks;
         base += (uint64_t)gridDim.x * Q6_BLOCKS_PER_CTA) {
        uint64_t blk = base + lb_;
        bool live = blk < n_blocks;
        float x[16];
        int8_t L[16];
        float scale = 0.0f;
        if (live) {
            const float4 *xp = (const float4 *)(src + blk * QK + 16 * j);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float4 v = xp[i];
                x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
            }
            scale = make_qx_rmse1_16(x, L);
        }
        // first sub-block with the largest |scale| decides the block scale (kquant.rs:296-303)
        float max_scale = 0.0f, max_abs = 0.0f;
#pragma unroll
        for (int t = 0; t < 16; t++) {
            float s = __shfl_sync(0xffffffffu, scale, (tid & 16) + t);
            float as = fabsf(s);
            if (as > max_abs) {
                max_abs = as;
                max_scale = s;
            }
        }
        bool zero_block = max_abs < 1e-15f;
        float iscale = zero_block ? 0.0f : xdiv(-128.0f, max_scale);
        __half dh = zero_block ? __float2half_rn(0.0f) : __float2half_rn(xdiv(1.0f, iscale));
        int sc = nearest_int(xmul(iscale, scale));
        if (sc > 127) sc = 127;
        int8_t sc8 = (int8_t)sc;
        if (live) {
            uint8_t *out = dst + blk * Q6K_BYTES;
            if (zero_block) {
                for (int i = 0; i < 16; i++) sL[lb_][16 * j + i] = 0;
                out[192 + j] = 0;
                if (j == 0) {
                    out[208] = 0;
                    out[209] = 0;
                }
            } else {
                float d = xmul(__half2float(dh), (float)sc8);
                if (d != 0.0f)
                    for (int i = 0; i < 16; i++) L[i] = (int8_t)(clampi(nearest_int(xdiv(x[i], d)), -32, 31) + 32);
                for (int i = 0; i < 16; i++) sL[lb_][16 * j + i] = (uint8_t)L[i];
                out[192 + j] = (uint8_t)sc8;
                if (j == 0) {
                    unsigned short dbits = __half_as_ushort(dh);
                    out[208] = dbits & 0xff;
                    out[209] = dbits >> 8;
                }
            }
        }
        __syncthreads();
        // ql (128 bytes) and qh (64 bytes) per block, interleaved over the two 128-halves
        for (int o = tid; o < Q6_BLOCKS_PER_CTA * 192; o += 256) {
            int b = o / 192, t = o % 192;
            uint64_t gb = base + b;
            if (gb >= n_blocks) continue;
            const uint8_t *l = sL[b];
            uint8_t v;
            if (t < 128) {
                int k = t >> 6, r = t & 63;          // ql[64k + r]
                int i = r & 31, second = r >> 5;     // r < 32: elements i, i+64; else i+32, i+96
                int e0 = 128 * k + i + 32 * second;
                v = (l[e0] & 0xF) | ((l[e0 + 64] & 0xF) << 4);
            } else {
                int t2 = t - 128;
                int k = t2 >> 5, i = t2 & 31;
                int e0 = 128 * k + i;
                v = (l[e0] >> 4) | ((l[e0 + 32] >> 4) << 2) | ((l[e0 + 64] >> 4) << 4) | ((l[e0 + 96] >> 4) << 6);
            }
            dst[gb * Q6K_BYTES + t] = v;
        }
        __syncthreads();
    }
}

// One thread per 32-value group: d = amax/127, q = clamp(round_half_away(x * (1/d)), +-127).
__global__ void __launch_bounds__(256) quantize_int8_kernel(const float *__restrict__ src, int8_t *__restrict__ qs,
                                                            uint16_t *__restrict__ scales, uint64_t n_groups) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        const float4 *xp = (const float4 *)(src + g * 32);
        float x[32];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float4 v = xp[i];
            x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            float a = fabsf(x[i]);
            if (a > amax) amax = a;
        }
        float d = xdiv(amax, 127.0f);
        float id = d != 0.0f ? xdiv(1.0f, d) : 0.0f;
        uint32_t packed[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            uint32_t wv = 0;
#pragma unroll
            for (int t = 0; t < 4; t++) {
                float pr = xmul(x[4 * i + t], id);
                float r = fminf(fmaxf(roundf(pr), -127.0f), 127.0f);
                int q = (pr != pr) ? 0 : (int)r;  // a NaN product quantizes to 0 (imp.rs:36-37)
                wv |= (uint32_t)(uint8_t)(int8_t)q << (8 * t);
            }
            packed[i] = wv;
        }
        uint4 *qp = (uint4 *)(qs + g * 32);
        qp[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        qp[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        scales[g] = __half_as_ushort(__float2half_rn(d));
    }
}

// Int4 (crates/lapid-quant/src/imp.rs:47-71): d = (the value of largest magnitude) / -8, q = trunc(x / d + 8.5)
// clamped to 0..15, byte j = element j | element j + 16 << 4. One thread per 32-group.
__global__ void __launch_bounds__(256) quantize_int4_kernel(const float *__restrict__ src, uint8_t *__restrict__ qs,
                                                            uint16_t *__restrict__ scales, uint64_t n_groups) {
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t g = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        const float4 *xp = (const float4 *)(src + g * 32);
        float x[32];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            float4 v = xp[i];
            x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
        }
        float amax = 0.0f, mx = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            float a = fabsf(x[i]);
            if (amax < a) {
                amax = a;
                mx = x[i];
            }
        }
        float d = mx == 0.0f ? 0.0f : xdiv(mx, -8.0f);
        float id = d != 0.0f ? xdiv(1.0f, d) : 0.0f;
        auto nib = [&](float v) -> uint32_t {
            float t = xadd(xmul(v, id), 8.5f);
            int q = (t != t) ? 0 : (t >= 2147483648.0f ? 2147483647 : (t <= -2147483648.0f ? (-2147483647 - 1) : (int)t));
            return (uint32_t)clampi(q, 0, 15);
        };
        uint32_t packed[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t wv = 0;
#pragma unroll
            for (int t = 0; t < 4; t++) wv |= (nib(x[4 * i + t]) | (nib(x[4 * i + t + 16]) << 4)) << (8 * t);
            packed[i] = wv;
        }
        *(uint4 *)(qs + g * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        scales[g] = __half_as_ushort(__float2half_rn(d));
    }
}

// MXFP4 (crates/lapid-quant/src/mxfp4.rs:27-49): one warp per 32-element block, lane = element.
//   e = u8(floor(log2(amax)) - 2 + 127) (0 for an all-zero block), d = 2^(e - 128),
//   code = the first of the 16 values KV * d closest to x.
// The reference takes log2 in f32 from its maths library; here it is taken in f64 and rounded to f32, which
// gives the correctly rounded f32 logarithm (the cases where the two could differ need a logarithm within
// 2^-29 of a rounding boundary; inputs just below a power of two, whose logarithm rounds up to the integer,
// come out the same).
__global__ void __launch_bounds__(256) quantize_mxfp4_kernel(const float *__restrict__ src, uint8_t *__restrict__ dst, uint64_t n_blocks) {
    const int lane = threadIdx.x & 31;
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    for (uint64_t blk = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); blk < n_blocks; blk += warps) {
        const float x = src[blk * GROUP + lane];
        float amax = fabsf(x);
        if (!(amax == amax)) amax = 0.0f;  // f32::max ignores a NaN operand
#pragma unroll
        for (int o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        uint32_t e = 0;
        if (amax > 0.0f) {
            const float l = (float)log2((double)amax);
            const float v = xadd(xsub(floorf(l), 2.0f), 127.0f);
            e = v <= 0.0f ? 0u : (v >= 255.0f ? 255u : (uint32_t)v);  // `as u8` saturates
        }
        const float d = e8m0_half(e);
        uint32_t best = 0;
        float best_err = fabsf(xsub(xmul(0.0f, d), x));
#pragma unroll
        for (uint32_t i = 1; i < 16; i++) {
            const float err = fabsf(xsub(xmul((float)mxfp4_kv(i), d), x));
            if (err < best_err) {
                best = i;
                best_err = err;
            }
        }
        const uint32_t hi = __shfl_down_sync(0xffffffffu, best, 16);
        uint8_t *out = dst + blk * MXFP4_BYTES;
        if (lane < 16) out[1 + lane] = (uint8_t)(best | (hi << 4));
        if (lane == 0) out[0] = (uint8_t)e;
    }
}

cudaError_t launch_quantize(int fmt, const float *src, uint64_t rows, uint64_t cols, uint64_t scales_offset,
                            uint64_t total_bytes, void *dst, int sm_count, cudaStream_t stream) {
    cudaError_t e = cudaMemsetAsync(dst, 0, total_bytes, stream);  // padding (and gaps) are zero
    if (e != cudaSuccess) return e;
    uint64_t n = rows * cols;
    if (n == 0) return cudaSuccess;
    uint64_t cap = (uint64_t)sm_count * 8;
    if (fmt == FMT_Q4K) {
        uint64_t nb = n / QK, ctas = (nb + Q4_BLOCKS_PER_CTA - 1) / Q4_BLOCKS_PER_CTA;
        quantize_q4k_kernel<FMT_Q4K><<<(int)(ctas < cap ? ctas : cap), 256, 0, stream>>>(src, (uint8_t *)dst, nb);
    } else if (fmt == FMT_Q5K) {
        uint64_t nb = n / QK, ctas = (nb + Q4_BLOCKS_PER_CTA - 1) / Q4_BLOCKS_PER_CTA;
        quantize_q4k_kernel<FMT_Q5K><<<(int)(ctas < cap ? ctas : cap), 256, 0, stream>>>(src, (uint8_t *)dst, nb);
    } else if (fmt == FMT_Q6K) {
        uint64_t nb = n / QK, ctas = (nb + Q6_BLOCKS_PER_CTA - 1) / Q6_BLOCKS_PER_CTA;
        quantize_q6k_kernel<<<(int)(ctas < cap ? ctas : cap), 256, 0, stream>>>(src, (uint8_t *)dst, nb);
    } else if (fmt == FMT_MXFP4) {
        uint64_t nb = n / GROUP, ctas = (nb + 7) / 8;
        quantize_mxfp4_kernel<<<(int)(ctas < cap ? ctas : cap), 256, 0, stream>>>(src, (uint8_t *)dst, nb);
    } else if (fmt == FMT_INT4) {
        uint64_t ng = n / GROUP, ctas = (ng + 255) / 256;
        uint8_t *d = (uint8_t *)dst;
        quantize_int4_kernel<<<(int)(ctas < cap ? ctas : cap), 256, 0, stream>>>(src, d, (uint16_t *)(d + scales_offset), ng);
    } else {
        uint64_t ng = n / GROUP, ctas = (ng + 255) / 256;
        uint8_t *d = (uint8_t *)dst;
        quantize_int8_kernel<<<(int)(ctas < cap ? ctas : cap), 256, 0, stream>>>(src, (int8_t *)d,
                                                                                (uint16_t *)(d + scales_offset), ng);
    }
    return cudaGetLastError();
}

}  // namespace lb

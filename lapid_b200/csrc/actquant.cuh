// Quantizing activations where they are produced: the kernel that computes an activation row
// (normalisation, SwiGLU product) also writes it as the int8 operand of the decode GEMV that
// follows, so that GEMV needs no pre-pass of its own. Same arithmetic, bit for bit, as the
// pre-pass kernel (actquant.cu; crates/lapid-cpu/src/matmul/quant.rs:68-89), same three layouts
// (ActQuantArgs::records).
//
// A thread holds four consecutive elements of a row; the eight lanes that hold one 32-element
// group must be eight consecutive lanes starting at a multiple of eight, and every lane of the
// warp must make the call (lanes without data pass active = false).
#pragma once
#include "common.cuh"
#include "kernels.h"

namespace lb {

__device__ __forceinline__ void act_quant_quad(const ActOut &o, bool active, uint32_t r, uint32_t col, float4 v) {
    float x[4] = {v.x, v.y, v.z, v.w};
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float a = fabsf(x[i]);
        if (active && a == a) amax = fmaxf(amax, a);  // f32::max ignores a NaN operand
    }
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, s));
    const float d = xdiv(amax, 127.0f);
    const float id = d > 0.0f ? xdiv(1.0f, d) : 0.0f;
    int q[4], sum = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float rr = xsub(xadd(xmul(x[i], id), 12582912.0f), 12582912.0f);
        int t = (rr != rr) ? 0 : (int)rr;
        t = t < -127 ? -127 : (t > 127 ? 127 : t);
        q[i] = t;
        sum += active ? t : 0;
    }
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
    if (!active) return;
    const uint32_t packed = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
    const uint32_t g = col / GROUP, e = col % GROUP;  // group of the row, first element inside it (a multiple of 4)
    const float bsum = xmul(d, (float)sum);
    if (o.records == 2) {
        const uint32_t sb = g & 7;
        uint8_t *blk = (uint8_t *)o.qa + (uint64_t)(g >> 3) * (256 * o.rows + 512);
        *(uint32_t *)(blk + (sb * o.rows + r) * 32 + e) = packed;
        if (e == 0) {
            float *sc = (float *)(blk + 256 * o.rows) + (((sb >> 1) * 4 + (r >> 1)) * 2 + (sb & 1)) * 2 + (r & 1);
            sc[0] = d;
            sc[64] = bsum;
        }
    } else if (o.records == 1) {
        uint8_t *rec = (uint8_t *)o.qa + ((uint64_t)r * (o.k / QK) + (g >> 3)) * REC + 80 * ((g & 7) >> 1);
        *(uint32_t *)(rec + 32 * (g & 1) + e) = packed;
        if (e == 0) {
            *(float *)(rec + 64 + 4 * (g & 1)) = d;
            *(float *)(rec + 72 + 4 * (g & 1)) = bsum;
        }
    } else {
        const uint32_t kg = o.k / GROUP;
        *(uint32_t *)(o.qa + (uint64_t)r * o.k + col) = packed;
        if (e == 0) {
            o.da[(uint64_t)r * kg + g] = d;
            if (o.bs) o.bs[(uint64_t)r * kg + g] = bsum;
        }
    }
}

}  // namespace lb

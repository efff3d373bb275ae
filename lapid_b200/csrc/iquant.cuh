// Device helpers for ggml's grid-based i-quants as lapid keeps them (256-element super-blocks stored exactly as in
// GGUF; crates/lapid-quant/src/iq2.rs:6-15, iq3.rs:5-10):
//
//   IQ2_XXS (66 B): f16 d | 8 x (u32: four grid indices | u32: four 7-bit sign indices + 4-bit scale)
//   IQ2_XS  (74 B): f16 d | u16[32]: 9-bit grid index | 7-bit sign index << 9 | scales[8]: 4 bits per 16 elements
//   IQ2_S   (82 B): f16 d | qs[32] index low bytes | signs[32] | qh[8]: two high index bits per 8-group | scales[8]
//   IQ3_XXS (98 B): f16 d | qs[64]: one grid index per 4 elements | 8 x u32: four 7-bit sign indices + 4-bit scale
//
// Every format is x = db(half) * grid byte * (+1 | -1) with one grid entry per 8 elements (IQ3_XXS: two entries of 4)
// and db = d * (0.5 + scale) * 0.25 (IQ3_XXS: * 0.5) per 16 or 32 elements. The codebooks are data of the formats;
// each device holds one copy of them in global memory (iq_grids()), in the order the reference's grid fixture uses
// (crates/lapid-quant/tests/iquant_golden.rs:53-62). The 128 sign patterns need no table: pattern i is i with an
// eighth bit that makes the number of set bits even (crates/lapid-quant/src/iqgrid.rs:19-30).
// Blocks are only 2-byte aligned: everything wider is assembled from 16-bit loads.
#pragma once
#include "common.cuh"

namespace lb {

constexpr int FMT_IQ2XXS = 10, FMT_IQ2S = 11, FMT_IQ3XXS = 12, FMT_IQ2XS = 13;  // crates/lapid-c/src/lib.rs:53-60
constexpr int IQ2XXS_BYTES = 66, IQ2XS_BYTES = 74, IQ2S_BYTES = 82, IQ3XXS_BYTES = 98;
// byte offsets of the codebooks inside the per-device table
constexpr int IQ_OFF_2XXS = 0, IQ_OFF_2S = 2048, IQ_OFF_3XXS = 10240, IQ_OFF_KSIGNS = 11264, IQ_OFF_2XS = 11392, IQ_GRID_BYTES = 15488;

__host__ __device__ constexpr bool is_iq(int fmt) { return fmt >= FMT_IQ2XXS && fmt <= FMT_IQ2XS; }
__host__ __device__ constexpr int iq_block_bytes(int fmt) {
    return fmt == FMT_IQ2XXS ? IQ2XXS_BYTES : fmt == FMT_IQ2XS ? IQ2XS_BYTES : fmt == FMT_IQ2S ? IQ2S_BYTES : IQ3XXS_BYTES;
}
// where a format's codebook starts in the table, and its length
__host__ __device__ constexpr int iq_grid_offset(int fmt) {
    return fmt == FMT_IQ2XXS ? IQ_OFF_2XXS : fmt == FMT_IQ2XS ? IQ_OFF_2XS : fmt == FMT_IQ2S ? IQ_OFF_2S : IQ_OFF_3XXS;
}
__host__ __device__ constexpr int iq_grid_bytes(int fmt) {
    return fmt == FMT_IQ2XXS ? 2048 : fmt == FMT_IQ2XS ? 4096 : fmt == FMT_IQ2S ? 8192 : 1024;
}

// The table on the current device (nullptr before iq_grids_upload()), and the upload (once per device; not
// during a stream capture).
const uint8_t *iq_grids();
cudaError_t iq_grids_upload();

__device__ __forceinline__ uint32_t ld16(const uint8_t *p) { return *(const uint16_t *)p; }
__device__ __forceinline__ uint32_t ld32_by16(const uint8_t *p) { return ld16(p) | (ld16(p + 2) << 16); }
// ksigns[i] of the reference
__device__ __forceinline__ uint32_t iq_ksign(uint32_t i7) { return i7 | ((__popc(i7) & 1u) << 7); }

// 8-group j (0..32) of the block at b (crates/lapid-cpu/src/iquant.rs:40-64): its grid bytes (lo = elements 0..3,
// hi = 4..7) and its eight sign bits. `grid` is the format's own codebook (global or shared memory).
template <int FMT> __device__ __forceinline__ void iq_group8(const uint8_t *b, int j, const uint8_t *grid, uint32_t &lo, uint32_t &hi, uint32_t &signs) {
    const int ib = j >> 2, l = j & 3;
    if constexpr (FMT == FMT_IQ2XXS) {
        const uint32_t a1 = ld32_by16(b + 6 + 8 * ib);
        const uint2 g = *(const uint2 *)(grid + 8 * (uint32_t)b[2 + 8 * ib + l]);
        lo = g.x, hi = g.y;
        signs = iq_ksign((a1 >> (7 * l)) & 127u);
    } else if constexpr (FMT == FMT_IQ2XS) {
        const uint32_t q = ld16(b + 2 + 2 * j);
        const uint2 g = *(const uint2 *)(grid + 8 * (q & 511u));
        lo = g.x, hi = g.y;
        signs = iq_ksign(q >> 9);
    } else if constexpr (FMT == FMT_IQ2S) {
        const uint32_t idx = (uint32_t)b[2 + j] | (((uint32_t)b[66 + ib] << (8 - 2 * l)) & 0x300u);
        const uint2 g = *(const uint2 *)(grid + 8 * idx);
        lo = g.x, hi = g.y;
        signs = b[34 + j];
    } else {
        const uint32_t aux = ld32_by16(b + 66 + 4 * ib);
        const uint32_t i2 = ld16(b + 2 + 8 * ib + 2 * l);
        lo = *(const uint32_t *)(grid + 4 * (i2 & 255u));
        hi = *(const uint32_t *)(grid + 4 * (i2 >> 8));
        signs = iq_ksign((aux >> (7 * l)) & 127u);
    }
}

// db of the 16-element half h (0..16) of the block at b: the reference's expression, each operation rounded on its
// own (crates/lapid-quant/src/iq2.rs:43, :59, :78; iq3.rs:25; crates/lapid-cpu/src/iquant.rs:66-89).
template <int FMT> __device__ __forceinline__ float iq_half_scale(const uint8_t *b, int h) {
    const float d = half_bits_to_float(ld16(b));
    const int ib = h >> 1;
    uint32_t s;
    if constexpr (FMT == FMT_IQ2XXS) s = ld16(b + 8 + 8 * ib) >> 12;  // top four bits of the second u32
    else if constexpr (FMT == FMT_IQ3XXS) s = ld16(b + 68 + 4 * ib) >> 12;
    else {
        const uint32_t sc = b[(FMT == FMT_IQ2XS ? 66 : 74) + ib];
        s = (h & 1) ? sc >> 4 : sc & 15u;
    }
    return xmul(xmul(d, xadd(0.5f, (float)s)), FMT == FMT_IQ3XXS ? 0.5f : 0.25f);
}

// Element e (0..256) of the block at b, bit for bit as the reference's dequantizers give it.
template <int FMT> __device__ __forceinline__ float iq_element(const uint8_t *b, int e, const uint8_t *grid) {
    uint32_t lo, hi, signs;
    iq_group8<FMT>(b, e >> 3, grid, lo, hi, signs);
    const int i = e & 7;
    const uint32_t g = ((i < 4 ? lo : hi) >> (8 * (i & 3))) & 255u;
    const float v = xmul(iq_half_scale<FMT>(b, e >> 4), (float)g);
    return (signs >> i) & 1u ? -v : v;
}

// Four grid bytes with the signs of bits 0..3 of `s` applied, as four int8 values.
__device__ __forceinline__ uint32_t iq_apply_signs(uint32_t g, uint32_t s) {
    const uint32_t m = (((s & 15u) * 0x00204081u) & 0x01010101u) * 0xFFu;  // 0xFF in the bytes whose sign bit is set
    return __vsub4(g ^ m, m);
}

}  // namespace lb

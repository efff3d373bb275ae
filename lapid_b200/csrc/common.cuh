// Shared device helpers: block geometry of the GGUF formats lapid keeps (Q4_K, Q6_K) and of its
// Int8 plane layout, exact (never contracted) f32 arithmetic for the bit-exact paths, and the
// 6-bit scale/min unpacking of Q4_K headers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kernels.h"

namespace lb {

constexpr int FMT_INT8 = 4;  // lapid dtype codes (crates/lapid-c/src/lib.rs:37-60)
constexpr int FMT_INT4 = 5;  // nibble planes: byte j of a 32-group holds element j (low) and j + 16 (high); x = (q - 8) * d
constexpr int FMT_Q4K = 6;
constexpr int FMT_Q5K = 7;
constexpr int FMT_Q6K = 8;
constexpr int FMT_MXFP4 = 9;  // ggml block_mxfp4: 32 elements in 17 bytes, e8m0 scale + e2m1 nibbles (byte j: element j low, j + 16 high)

constexpr int GROUP = 32;
constexpr int QK = 256;
constexpr int Q4K_BYTES = 144;
constexpr int Q5K_BYTES = 176;  // Q4_K's header, then the fifth bits qh[32], then the nibbles qs[128]
constexpr int Q6K_BYTES = 210;
constexpr int MXFP4_BYTES = 17;

// Separately rounded IEEE operations. nvcc fuses a*b+c into an FMA unless told otherwise; the
// reference never does ("do not simplify the arithmetic", crates/lapid-quant/src/kquant.rs:3-4),
// so every operation that must reproduce its bits goes through these.
__device__ __forceinline__ float xmul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float xadd(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float xsub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float xdiv(float a, float b) { return __fdiv_rn(a, b); }

__device__ __forceinline__ float half_bits_to_float(uint32_t h) {
    return __half2float(__ushort_as_half((unsigned short)h));
}

// Activation element types of a launch (MatMulSpec.a_dtype): lapid-cpu widens f16 / bf16 rows to f32 before anything
// else happens to them (`load_contig`, crates/lapid-cpu/src/matmul/mod.rs:165-286); both widenings are exact.
constexpr int ACT_F32 = 0, ACT_F16 = 1, ACT_BF16 = 2;
__host__ __device__ constexpr uint32_t act_elem_bytes(int a_type) { return a_type == ACT_F32 ? 4u : 2u; }
// Element i of the row that starts at `row`.
__device__ __forceinline__ float load_act(const void *row, uint64_t i, int a_type) {
    if (a_type == ACT_F32) return ((const float *)row)[i];
    const unsigned short h = ((const unsigned short *)row)[i];
    return a_type == ACT_F16 ? __half2float(__ushort_as_half(h)) : __uint_as_float((uint32_t)h << 16);
}
// Start of row r = bt*m + i of an activation operand: base + (off + bt*bs + i*rs) elements.
__device__ __forceinline__ const void *act_row(const void *base, int a_type, uint64_t off, uint64_t bs, uint64_t rs, uint32_t r, uint32_t m) {
    return (const char *)base + (off + (uint64_t)(r / m) * bs + (uint64_t)(r % m) * rs) * act_elem_bytes(a_type);
}

// MXFP4 (crates/lapid-quant/src/mxfp4.rs:14-25): x = KV[nibble] * d, KV = the doubled e2m1 values
// {0,1,2,3,4,6,8,12} and their negatives, d = 2^(e - 128) (a denormal for e < 2).
__device__ __forceinline__ int mxfp4_kv(uint32_t nib) {
    const uint32_t mag = (uint32_t)((0x0C08060403020100ull >> (8 * (nib & 7))) & 0xff);
    return (nib & 8) ? -(int)mag : (int)mag;
}
__device__ __forceinline__ float e8m0_half(uint32_t e) { return __uint_as_float(e < 2 ? 0x00200000u << e : (e - 1) << 23); }
// element `e` (0..31) of the block at `b`
__device__ __forceinline__ float mxfp4_element(const uint8_t *b, uint32_t e) {
    const uint32_t q = b[1 + (e & 15)];
    return xmul((float)mxfp4_kv(e < 16 ? q & 15 : q >> 4), e8m0_half(b[0]));
}

// `prmt.b32` as the instruction defines it (selector nibble: bits 0..2 pick one of the eight source bytes, bit 3 replaces
// the byte by eight copies of its top bit; the __byte_perm intrinsic drops bit 3).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// Four MXFP4 codes in the nibbles of the low 16 bits of `h` -> their KV values (the doubled e2m1 values, mxfp4_kv) as four
// int8, byte i = nibble i. Four nibbles are exactly a `prmt` selector: with the sign bits masked off, one `prmt` over
// the table of magnitudes gives the four |KV|, a second over the negated magnitudes the four -|KV|; `prmt` of 0x80
// bytes with the unmasked half as selector gives 0x80 where a sign bit is clear (byte copied) and 0xFF where it is set
// (top bit replicated), which a shift and one logic operation turn into a byte mask and a last one uses to pick per
// byte. The code 8 ("-0") comes out as 0.
__device__ __forceinline__ uint32_t mxfp4_kv4(uint32_t h) {
    const uint32_t sel = h & 0x7777u;
    const uint32_t pos = prmt(0x03020100u, 0x0C080604u, sel);  // 0, 1, 2, 3 | 4, 6, 8, 12
    const uint32_t neg = prmt(0xFDFEFF00u, 0xF4F8FAFCu, sel);  // 0, -1, -2, -3 | -4, -6, -8, -12
    const uint32_t r = prmt(0x80808080u, 0x80808080u, h);
    const uint32_t m = (r & 0x7F7F7F7Fu) | ((r << 1) & 0x80808080u);  // 0x00 / 0xFF
    return (pos & ~m) | (neg & m);
}

// The epilogue expression of a launch at one output element (postfix program, see EpiProg): a four-deep stack in
// registers, one pass over the program's words. f32 throughout; Exp, Log, Sin, Cos, Tanh, Erf and Pow are CUDA's
// full-precision functions, Recip and Div IEEE divisions (the reference's CPU backend has polynomial versions of its
// own: results agree to a few ulp, not bit for bit).
__device__ __forceinline__ float epi_eval(const EpiProg &e, float acc, float extra) {
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    for (uint32_t i = 0; i < e.n; i++) {
        const uint32_t w = e.code[i], op = w & 0xffu;
        if (op == EPI_LOAD || op == EPI_CONST) {
            const float v = op == EPI_CONST ? __uint_as_float(e.code[++i]) : ((w >> 8) ? extra : acc);
            s3 = s2, s2 = s1, s1 = s0, s0 = v;
        } else if (op < EPI_UNARY_END) {
            const float x = s0;
            s0 = op == EPI_NEG ? -x : op == EPI_EXP ? expf(x) : op == EPI_LOG ? logf(x) : op == EPI_SQRT ? sqrtf(x)
               : op == EPI_RSQRT ? 1.0f / sqrtf(x) : op == EPI_RECIP ? 1.0f / x : op == EPI_SIN ? sinf(x) : op == EPI_COS ? cosf(x)
               : op == EPI_TANH ? tanhf(x) : op == EPI_ERF ? erff(x) : fabsf(x);
        } else if (op < EPI_BINARY_END) {
            const float a = s1, b = s0;
            s0 = op == EPI_ADD ? a + b : op == EPI_SUB ? a - b : op == EPI_MUL ? a * b : op == EPI_DIV ? a / b : op == EPI_MAX ? fmaxf(a, b)
               : op == EPI_MIN ? fminf(a, b) : op == EPI_POW ? powf(a, b) : op == EPI_CMPLT ? (a < b ? 1.0f : 0.0f) : (a == b ? 1.0f : 0.0f);
            s1 = s2, s2 = s3;
        } else {  // EPI_WHERE: cond, a, b -> cond != 0 ? a : b
            s0 = s2 != 0.0f ? s1 : s0;
            s1 = s3;
        }
    }
    return s0;
}
// What a kernel that evaluates expressions itself stores for accumulator `v` of the output element whose extra lies at index `idx`.
template <class P> __device__ __forceinline__ float epilogue(const P &p, float v, int64_t idx) {
    if (p.epi.n == 0) return p.extra ? v + p.extra[idx] : v;
    return epi_eval(p.epi, v, p.extra ? p.extra[idx] : 0.0f);
}

// ggml's nearest_int (crates/lapid-quant/src/kquant.rs:25-28): round half to even through the
// 1.5 * 2^23 offset, valid for |x| <= 4194303.
__device__ __forceinline__ int nearest_int(float f) {
    float v = xadd(f, 12582912.0f);
    return (int)(__float_as_uint(v) & 0x007fffffu) - 0x00400000;
}

// 6-bit scale and min of sub-block j (0..8) from the 12 packed bytes of a Q4_K header
// (crates/lapid-quant/src/kquant.rs:178-184). `s` points at the 12 bytes.
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *s, int &sc, int &mn) {
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

// The same unpacking from the three 32-bit words that hold the 12 bytes (w0 = bytes 0..3,
// w1 = 4..7, w2 = 8..11): scales and mins of sub-blocks 2p and 2p+1 for pair p.
__device__ __forceinline__ void scale_min_pair(int p, uint32_t w0, uint32_t w1, uint32_t w2, int &sc0, int &mn0,
                                               int &sc1, int &mn1) {
    if (p < 2) {
        int sh = 16 * p;  // bytes 2p, 2p+1 of w0 (scales) and w1 (mins)
        sc0 = (w0 >> sh) & 63;
        sc1 = (w0 >> (sh + 8)) & 63;
        mn0 = (w1 >> sh) & 63;
        mn1 = (w1 >> (sh + 8)) & 63;
    } else {
        int sh = 16 * (p - 2);  // j = 2p, 2p+1 -> bytes j+4 = 8+2(p-2).. of the 12, i.e. w2
        uint32_t b0 = (w2 >> sh) & 0xff, b1 = (w2 >> (sh + 8)) & 0xff;
        uint32_t lo0 = (w0 >> sh) & 0xff, lo1 = (w0 >> (sh + 8)) & 0xff;  // s[j-4]
        uint32_t hi0 = (w1 >> sh) & 0xff, hi1 = (w1 >> (sh + 8)) & 0xff;  // s[j]
        sc0 = (b0 & 0xF) | ((lo0 >> 6) << 4);
        mn0 = (b0 >> 4) | ((hi0 >> 6) << 4);
        sc1 = (b1 & 0xF) | ((lo1 >> 6) << 4);
        mn1 = (b1 >> 4) | ((hi1 >> 6) << 4);
    }
}

}  // namespace lb

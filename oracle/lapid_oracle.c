/*
 * lapid_oracle.c -- CPU restatement of lapid's quantized-matmul path. TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA kernels are compared against and the CPU baseline that the
 * benchmark times beside them. Nothing that ships (the package, the C-ABI library) links, loads
 * or calls it; only the tests, the smoke check and the benchmark's cpu-baseline legs do.
 *
 * It restates, function for function, the arithmetic of the Rust reference (which cannot be
 * compiled where this was written: no Rust toolchain). Every f32 operation is a separately
 * rounded IEEE operation in the order the reference writes it: build with -ffp-contract=off.
 *
 *   storage contract ............ crates/lapid-quant/src/lib.rs:27-125
 *   Q4_K / Q5_K / Q6_K quantizers  crates/lapid-quant/src/kquant.rs:25-334
 *   ... and dequantizers ........ crates/lapid-quant/src/kquant.rs:337-396
 *   Int8 (GGUF Q8_0 as planes) .. crates/lapid-quant/src/imp.rs:24-40, :73-116, :143-200
 *   Int4 (nibble planes) ........ crates/lapid-quant/src/imp.rs:47-71, :148-156; crates/lapid-cpu/src/qmat.rs:97-112
 *   i-quants (dequantizers, decode tile) crates/lapid-quant/src/iq2.rs:38-90, iq3.rs:18-39; crates/lapid-cpu/src/iquant.rs:40-128
 *   f32 -> f16 .................. `half` 2.7.1 f16::from_f32 (Cargo.lock:1188), IEEE round to
 *                                 nearest even; not vendored in the reference tree, so restated
 *                                 from the IEEE definition and pinned by the 0x3008 known answer
 *                                 (crates/lapid-quant/src/imp.rs:276) and an exhaustive check
 *                                 against numpy's float16 conversion in the tests
 *   f16 -> f32 .................. crates/lapid-cpu/src/typed.rs:13-21
 *   activation quantizer ........ crates/lapid-cpu/src/matmul/quant.rs:68-89, math.rs:134-136
 *   decode tiles (m <= 8) ....... crates/lapid-cpu/src/kquant.rs:36-91, :202-244 (K formats),
 *                                 crates/lapid-cpu/src/matmul/qkernels.rs:60-84 (Int8)
 *   prefill (m > 8) ............. crates/lapid-cpu/src/matmul/qdeq.rs:26-123,
 *                                 crates/lapid-cpu/src/matmul/kernels.rs:29-46, :95-119
 *   dispatch and validation ..... crates/lapid-cpu/src/matmul/mod.rs:45, :165-262
 *
 * Parity status: Int8 bytes are pinned by the reference's known-answer vector; Q4_K / Q5_K / Q6_K
 * dequantization is pinned bit-for-bit against an independent third-party dequantizer (the
 * `gguf` Python package) in the tests; K-format *quantizer bytes* are pinned only by the
 * reference's property tests (round-trip error bounds, constants, zeros) because the reference
 * checks in no golden bytes for them: quantizer byte parity is "parity unpinned". The i-quant
 * dequantizers are pinned bit for bit by the golden bytes the reference itself holds
 * (crates/lapid-quant/tests/fixtures/iquant/) and by the `gguf` package's dequantizers.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LO_FMT_INT8 4
#define LO_FMT_INT4 5
#define LO_FMT_Q4K 6
#define LO_FMT_Q5K 7
#define LO_FMT_Q6K 8
#define LO_FMT_MXFP4 9
#define MXFP4_BYTES 17
/* the grid-based i-quants (crates/lapid-c/src/lib.rs:53-60; block sizes crates/lapid-quant/src/iq2.rs:24-26, iq3.rs:16) */
#define LO_FMT_IQ2XXS 10
#define LO_FMT_IQ2S 11
#define LO_FMT_IQ3XXS 12
#define LO_FMT_IQ2XS 13
#define IQ2XXS_BYTES 66
#define IQ2XS_BYTES 74
#define IQ2S_BYTES 82
#define IQ3XXS_BYTES 98

#define GROUP 32
#define ALIGN 256
#define QK 256
#define Q4K_BYTES 144
#define Q5K_BYTES 176
#define Q6K_BYTES 210

/* ------------------------------------------------------------------ bit helpers */
static inline uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float bits_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* IEEE binary32 -> binary16, round to nearest even (half::f16::from_f32 semantics). */
uint16_t lo_f32_to_f16(float f) {
    uint32_t x = f32_bits(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t man = x & 0x007fffffu;
    int exp = (int)((x >> 23) & 0xff);
    if (exp == 0xff) {
        if (man == 0) return (uint16_t)(sign | 0x7c00u);
        return (uint16_t)(sign | 0x7c00u | 0x0200u | (man >> 13));
    }
    int e = exp - 127 + 15;
    if (e >= 31) return (uint16_t)(sign | 0x7c00u);
    if (e <= 0) {
        if (e < -10) return (uint16_t)sign;
        man |= 0x00800000u;
        int shift = 14 - e;
        uint32_t hm = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (hm & 1u))) hm++;
        return (uint16_t)(sign | hm);
    }
    uint32_t h = sign | ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) h++;
    return (uint16_t)h;
}

/* crates/lapid-cpu/src/typed.rs:13-21 -- exact for every finite half, subnormals included. */
float lo_f16_to_f32(uint16_t h16) {
    uint32_t h = h16;
    uint32_t sign = (h & 0x8000u) << 16;
    uint32_t em = (h & 0x7fffu) << 13;
    uint32_t normal = f32_bits(bits_f32(em) * bits_f32(0x77800000u));
    uint32_t bits = ((h & 0x7c00u) == 0x7c00u) ? (em | 0x7f800000u) : normal;
    return bits_f32(bits | sign);
}

static inline float rd_h(const uint8_t *b, size_t o) { return lo_f16_to_f32((uint16_t)(b[o] | (b[o + 1] << 8))); }
static inline void wr_h(uint8_t *b, size_t o, float v) {
    uint16_t h = lo_f32_to_f16(v);
    b[o] = (uint8_t)(h & 0xff);
    b[o + 1] = (uint8_t)(h >> 8);
}

/* crates/lapid-quant/src/kquant.rs:25-28 */
static inline int nearest_int(float fval) {
    float val = fval + 12582912.0f;
    return (int)(f32_bits(val) & 0x007fffffu) - 0x00400000;
}
int lo_nearest_int(float f) { return nearest_int(f); }

static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* ------------------------------------------------------------------ layout (lib.rs:27-125) */
static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

static int block_elems(int fmt) { return (fmt == LO_FMT_INT8 || fmt == LO_FMT_INT4 || fmt == LO_FMT_MXFP4) ? GROUP : QK; }
static int is_iqfmt(int fmt) { return fmt == LO_FMT_IQ2XXS || fmt == LO_FMT_IQ2S || fmt == LO_FMT_IQ3XXS || fmt == LO_FMT_IQ2XS; }
static int block_bytes(int fmt) {
    switch (fmt) {
        case LO_FMT_Q4K: return Q4K_BYTES;
        case LO_FMT_Q5K: return Q5K_BYTES;
        case LO_FMT_Q6K: return Q6K_BYTES;
        case LO_FMT_MXFP4: return MXFP4_BYTES;
        case LO_FMT_IQ2XXS: return IQ2XXS_BYTES;
        case LO_FMT_IQ2XS: return IQ2XS_BYTES;
        case LO_FMT_IQ2S: return IQ2S_BYTES;
        case LO_FMT_IQ3XXS: return IQ3XXS_BYTES;
        default: return 0;
    }
}
static int is_kfmt(int fmt) { return fmt == LO_FMT_Q4K || fmt == LO_FMT_Q5K || fmt == LO_FMT_Q6K; }

/* out = {qs_offset, qs_bytes, scales_offset, scales_bytes, total}; returns 0, or -1 on a bad
 * format / cols not a multiple of the block. */
int lo_layout(int fmt, size_t rows, size_t cols, size_t out[5]) {
    if (fmt != LO_FMT_INT8 && fmt != LO_FMT_INT4 && fmt != LO_FMT_MXFP4 && !is_kfmt(fmt) && !is_iqfmt(fmt)) return -1;
    size_t be = (size_t)block_elems(fmt);
    if (cols % be != 0) return -1;
    if (block_bytes(fmt) != 0) {
        size_t n = rows * (cols / be) * (size_t)block_bytes(fmt);
        out[0] = 0; out[1] = n; out[2] = n; out[3] = 0; out[4] = align_up(n, ALIGN);
        return 0;
    }
    size_t qs = fmt == LO_FMT_INT8 ? rows * cols : rows * cols / 2; /* Int4: two elements of one group per byte */
    size_t so = align_up(qs, ALIGN);
    size_t sb = rows * (cols / GROUP) * 2;
    out[0] = 0; out[1] = qs; out[2] = so; out[3] = sb; out[4] = align_up(so + sb, ALIGN);
    return 0;
}

/* ------------------------------------------------------------------ Q4_K quantizer */
/* kquant.rs:42-121: asymmetric scale + min search over one sub-block. Returns scale, *the_min. */
static float make_qkx2(int n, const float *x, const float *w, int nmax, uint8_t *L, uint8_t *Laux,
                       float rmin, float rdelta, int nstep, float *the_min) {
    float mn = x[0], mx = x[0];
    float sum_w = w[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; i++) {
        if (x[i] < mn) mn = x[i];
        if (x[i] > mx) mx = x[i];
        float wi = w[i];
        sum_w += wi;
        sum_x += wi * x[i];
    }
    if (mn > 0.0f) mn = 0.0f;
    if (mx == mn) {
        for (int i = 0; i < n; i++) L[i] = 0;
        *the_min = -mn;
        return 0.0f;
    }
    float iscale = (float)nmax / (mx - mn);
    float scale = 1.0f / iscale;
    float best = 0.0f;
    for (int i = 0; i < n; i++) {
        int l = nearest_int(iscale * (x[i] - mn));
        L[i] = (uint8_t)clampi(l, 0, nmax);
        float diff = scale * (float)L[i] + mn - x[i];
        best += w[i] * (diff * diff);
    }
    if (nstep < 1) {
        *the_min = -mn;
        return scale;
    }
    for (int is = 0; is <= nstep; is++) {
        iscale = (rmin + rdelta * (float)is + (float)nmax) / (mx - mn);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; i++) {
            int l = clampi(nearest_int(iscale * (x[i] - mn)), 0, nmax);
            Laux[i] = (uint8_t)l;
            float wi = w[i];
            float lf = (float)l;
            sum_l += wi * lf;
            sum_l2 += wi * lf * lf;
            sum_xl += wi * lf * x[i];
        }
        float D = sum_w * sum_l2 - sum_l * sum_l;
        if (D > 0.0f) {
            float this_scale = (sum_w * sum_xl - sum_x * sum_l) / D;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / D;
            if (this_min > 0.0f) {
                this_min = 0.0f;
                this_scale = sum_xl / sum_l2;
            }
            float cur = 0.0f;
            for (int i = 0; i < n; i++) {
                float diff = this_scale * (float)Laux[i] + this_min - x[i];
                cur += w[i] * (diff * diff);
            }
            if (cur < best) {
                memcpy(L, Laux, (size_t)n);
                best = cur;
                scale = this_scale;
                mn = this_min;
            }
        }
    }
    *the_min = -mn;
    return scale;
}

/* kquant.rs:178-184 */
static inline void scale_min_k4(int j, const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* kquant.rs:186-247: the shared first half of the Q4_K / Q5_K quantizers: per-32 scales and mins,
 * the packed 6-bit scales, d / dmin in head[0..4], and the final quants L (0..nmax) per element. */
static void quantize_k45(const float *x, int nmax, float rmin, int nstep, uint8_t *head, uint8_t *L) {
    uint8_t Laux[32];
    float weights[32], scales[8], mins[8];
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
        const float *xs = x + 32 * j;
        float sum_x2 = 0.0f;
        for (int l = 0; l < 32; l++) sum_x2 += xs[l] * xs[l];
        float av_x = sqrtf(sum_x2 / 32.0f);
        for (int l = 0; l < 32; l++) weights[l] = av_x + fabsf(xs[l]);
        float m;
        float s = make_qkx2(32, xs, weights, nmax, L + 32 * j, Laux, rmin, 0.1f, nstep, &m);
        scales[j] = s;
        mins[j] = m;
        if (s > max_scale) max_scale = s;
        if (m > max_min) max_min = m;
    }
    float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
    float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
    uint8_t *sc = head + 4;
    memset(sc, 0, 12);
    for (int j = 0; j < 8; j++) {
        /* the C original stores nearest_int() in a uint8_t before MIN(63, .) */
        uint8_t ls = (uint8_t)nearest_int(inv_scale * scales[j]);
        uint8_t lm = (uint8_t)nearest_int(inv_min * mins[j]);
        if (ls > 63) ls = 63;
        if (lm > 63) lm = 63;
        if (j < 4) {
            sc[j] = ls;
            sc[j + 4] = lm;
        } else {
            sc[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
            sc[j - 4] |= (uint8_t)((ls >> 4) << 6);
            sc[j] |= (uint8_t)((lm >> 4) << 6);
        }
    }
    wr_h(head, 0, max_scale / 63.0f);
    wr_h(head, 2, max_min / 63.0f);
    float d_all = rd_h(head, 0), dmin_all = rd_h(head, 2);
    for (int j = 0; j < 8; j++) {
        uint8_t s, m;
        scale_min_k4(j, sc, &s, &m);
        float d = d_all * (float)s;
        if (d == 0.0f) continue;
        float dm = dmin_all * (float)m;
        for (int ii = 0; ii < 32; ii++) {
            int q = nearest_int((x[32 * j + ii] + dm) / d);
            L[32 * j + ii] = (uint8_t)clampi(q, 0, nmax);
        }
    }
}

/* kquant.rs:250-260 */
void lo_quantize_q4k_block(const float *x, uint8_t *out) {
    uint8_t L[QK];
    quantize_k45(x, 15, -1.0f, 20, out, L);
    uint8_t *qs = out + 16;
    for (int k = 0; k < 4; k++)
        for (int i = 0; i < 32; i++) qs[32 * k + i] = (uint8_t)(L[64 * k + i] | (L[64 * k + i + 32] << 4));
}

/* kquant.rs:263-287: as Q4_K with 5-bit quants; the fifth bits of the 8 sub-blocks share qh[32] */
void lo_quantize_q5k_block(const float *x, uint8_t *out) {
    uint8_t L[QK];
    quantize_k45(x, 31, -0.5f, 15, out, L);
    uint8_t *qh = out + 16, *ql = out + 48;
    memset(qh, 0, 32);
    uint8_t m1 = 1, m2 = 2;
    for (int k = 0; k < 4; k++) {
        for (int j = 0; j < 32; j++) {
            uint8_t l1 = L[64 * k + j], l2 = L[64 * k + j + 32];
            if (l1 > 15) {
                l1 -= 16;
                qh[j] |= m1;
            }
            if (l2 > 15) {
                l2 -= 16;
                qh[j] |= m2;
            }
            ql[32 * k + j] = (uint8_t)(l1 | (l2 << 4));
        }
        m1 <<= 2;
        m2 <<= 2;
    }
}

/* ------------------------------------------------------------------ Q6_K quantizer */
/* kquant.rs:124-174: symmetric rmse search (rmse_type 1, weights x^2). L receives l + nmax. */
static float make_qx_rmse1(int n, const float *x, int nmax, int8_t *L) {
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
    float iscale = -(float)nmax / mx;
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; i++) {
        int l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
        L[i] = (int8_t)(l + nmax);
        float w = x[i] * x[i];
        float lf = (float)l;
        sumlx += w * x[i] * lf;
        suml2 += w * lf * lf;
    }
    float scale = suml2 != 0.0f ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; is++) {
        if (is == 0) continue;
        iscale = -((float)nmax + 0.1f * (float)is) / mx;
        sumlx = 0.0f;
        suml2 = 0.0f;
        for (int i = 0; i < n; i++) {
            float lf = (float)clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
            float w = x[i] * x[i];
            sumlx += w * x[i] * lf;
            suml2 += w * lf * lf;
        }
        if (suml2 > 0.0f && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; i++) {
                int l = clampi(nearest_int(iscale * x[i]), -nmax, nmax - 1);
                L[i] = (int8_t)(nmax + l);
            }
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

/* kquant.rs:290-334 */
void lo_quantize_q6k_block(const float *x, uint8_t *out) {
    int8_t L[QK];
    float scales[16];
    float max_scale = 0.0f, max_abs = 0.0f;
    for (int ib = 0; ib < 16; ib++) {
        float s = make_qx_rmse1(16, x + 16 * ib, 32, L + 16 * ib);
        scales[ib] = s;
        float as = fabsf(s);
        if (as > max_abs) {
            max_abs = as;
            max_scale = s;
        }
    }
    memset(out, 0, Q6K_BYTES);
    if (max_abs < 1e-15f) return;
    float iscale = -128.0f / max_scale;
    wr_h(out, 208, 1.0f / iscale);
    for (int ib = 0; ib < 16; ib++) {
        int v = nearest_int(iscale * scales[ib]);
        if (v > 127) v = 127;
        out[192 + ib] = (uint8_t)(int8_t)v;
    }
    float d_all = rd_h(out, 208);
    for (int j = 0; j < 16; j++) {
        float d = d_all * (float)(int8_t)out[192 + j];
        if (d == 0.0f) continue;
        for (int ii = 0; ii < 16; ii++) {
            int q = clampi(nearest_int(x[16 * j + ii] / d), -32, 31);
            L[16 * j + ii] = (int8_t)(q + 32);
        }
    }
    uint8_t *ql = out, *qh = out + 128;
    for (int k = 0; k < 2; k++) {
        for (int i = 0; i < 32; i++) {
            uint8_t a = (uint8_t)L[128 * k + i], b = (uint8_t)L[128 * k + i + 32];
            uint8_t c = (uint8_t)L[128 * k + i + 64], d = (uint8_t)L[128 * k + i + 96];
            ql[64 * k + i] = (uint8_t)((a & 0xF) | ((c & 0xF) << 4));
            ql[64 * k + i + 32] = (uint8_t)((b & 0xF) | ((d & 0xF) << 4));
            qh[32 * k + i] = (uint8_t)((a >> 4) | ((b >> 4) << 2) | ((c >> 4) << 4) | ((d >> 4) << 6));
        }
    }
}

/* ------------------------------------------------------------------ dequantizers */
/* kquant.rs:337-352 */
void lo_dequantize_q4k_block(const uint8_t *b, float *y) {
    float d = rd_h(b, 0), mn = rd_h(b, 2);
    const uint8_t *scales = b + 4, *qs = b + 16;
    for (int j = 0; j < 4; j++) {
        const uint8_t *q = qs + 32 * j;
        uint8_t s1, m1, s2, m2;
        scale_min_k4(2 * j, scales, &s1, &m1);
        scale_min_k4(2 * j + 1, scales, &s2, &m2);
        float d1 = d * (float)s1, mm1 = mn * (float)m1;
        float d2 = d * (float)s2, mm2 = mn * (float)m2;
        float *o = y + 64 * j;
        for (int l = 0; l < 32; l++) {
            o[l] = d1 * (float)(q[l] & 0xF) - mm1;
            o[l + 32] = d2 * (float)(q[l] >> 4) - mm2;
        }
    }
}

/* kquant.rs:355-373 */
void lo_dequantize_q5k_block(const uint8_t *b, float *y) {
    float d = rd_h(b, 0), mn = rd_h(b, 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *qs = b + 48;
    for (int j = 0; j < 4; j++) {
        const uint8_t *q = qs + 32 * j;
        uint8_t u1 = (uint8_t)(1u << (2 * j)), u2 = (uint8_t)(2u << (2 * j));
        uint8_t s1, m1, s2, m2;
        scale_min_k4(2 * j, scales, &s1, &m1);
        scale_min_k4(2 * j + 1, scales, &s2, &m2);
        float d1 = d * (float)s1, mm1 = mn * (float)m1;
        float d2 = d * (float)s2, mm2 = mn * (float)m2;
        float *o = y + 64 * j;
        for (int l = 0; l < 32; l++) {
            int h1 = (qh[l] & u1) ? 16 : 0, h2 = (qh[l] & u2) ? 16 : 0;
            o[l] = d1 * (float)((q[l] & 0xF) + h1) - mm1;
            o[l + 32] = d2 * (float)((q[l] >> 4) + h2) - mm2;
        }
    }
}

/* kquant.rs:376-396 */
void lo_dequantize_q6k_block(const uint8_t *b, float *y) {
    float d = rd_h(b, 208);
    for (int n = 0; n < 2; n++) {
        const uint8_t *ql = b + 64 * n, *qh = b + 128 + 32 * n;
        const int8_t *sc = (const int8_t *)(b + 192 + 8 * n);
        float *o = y + 128 * n;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int q1 = (int)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
            int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            o[l] = (d * (float)sc[is]) * (float)q1;
            o[l + 32] = (d * (float)sc[is + 2]) * (float)q2;
            o[l + 64] = (d * (float)sc[is + 4]) * (float)q3;
            o[l + 96] = (d * (float)sc[is + 6]) * (float)q4;
        }
    }
}

/* ------------------------------------------------------------------ Int8 planes (imp.rs) */
/* imp.rs:24-40. Rust's f32::round rounds half away from zero; `as i32` maps NaN to 0. */
static float quant_group_i8(const float *x, uint8_t *q) {
    float amax = 0.0f;
    for (int i = 0; i < GROUP; i++) {
        float a = fabsf(x[i]);
        if (a > amax) amax = a;
    }
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < GROUP; i++) {
        float r = roundf(x[i] * id);
        if (r != r) {
            q[i] = 0;
            continue;
        }
        if (r < -127.0f) r = -127.0f;
        if (r > 127.0f) r = 127.0f;
        q[i] = (uint8_t)(int8_t)(int)r;
    }
    return d;
}

/* imp.rs:47-71: Int4 group. d = (the value of largest magnitude) / -8, so that value maps to quant 0;
 * byte j holds element j (low nibble) and element j + 16 (high nibble) as q = trunc(x/d + 8.5) in 0..15. */
static inline uint8_t nibble_i4(float v) {
    float t = v + 8.5f;
    int i;
    if (t != t) i = 0;                       /* `as i32`: NaN -> 0, saturating */
    else if (t >= 2147483648.0f) i = 2147483647;
    else if (t <= -2147483648.0f) i = -2147483647 - 1;
    else i = (int)t;                          /* truncates toward zero */
    return (uint8_t)clampi(i, 0, 15);
}
static float quant_group_i4(const float *x, uint8_t *q) {
    float amax = 0.0f, mx = 0.0f;
    for (int i = 0; i < GROUP; i++) {
        float a = fabsf(x[i]);
        if (amax < a) {
            amax = a;
            mx = x[i];
        }
    }
    float d = mx == 0.0f ? 0.0f : mx / -8.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int j = 0; j < GROUP / 2; j++) q[j] = (uint8_t)(nibble_i4(x[j] * id) | (nibble_i4(x[j + GROUP / 2] * id) << 4));
    return d;
}

/* ------------------------------------------------------------------ MXFP4 (crates/lapid-quant/src/mxfp4.rs) */
/* 32 elements in 17 bytes: e (e8m0) | qs[16], byte j = element j (low nibble) | element j + 16 (high nibble);
 * x = KV[nibble] * d with the doubled e2m1 values KV and d = 2^(e - 128). */
static const int8_t MXFP4_KV[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12}; /* mxfp4.rs:19 */

/* mxfp4.rs:22-25: d as f32 bits (a denormal for e < 2) */
static inline float e8m0_half(uint8_t e) { return bits_f32(e < 2 ? (uint32_t)0x00200000u << e : (uint32_t)(e - 1) << 23); }

/* mxfp4.rs:27-38: the first code with the smallest |KV * d - x| */
static uint8_t mxfp4_best_index(float x, float d) {
    uint8_t best = 0;
    float best_err = fabsf((float)MXFP4_KV[0] * d - x);
    for (int i = 1; i < 16; i++) {
        float err = fabsf((float)MXFP4_KV[i] * d - x);
        if (err < best_err) {
            best = (uint8_t)i;
            best_err = err;
        }
    }
    return best;
}

/* mxfp4.rs:41-49. `as u8` saturates: values below 0 give 0, above 255 give 255 (NaN gives 0). */
void lo_quantize_mxfp4_block(const float *x, uint8_t *out) {
    float amax = 0.0f;
    for (int i = 0; i < GROUP; i++) {
        float a = fabsf(x[i]);
        if (a > amax) amax = a; /* f32::max ignores a NaN operand */
    }
    uint8_t e = 0;
    if (amax > 0.0f) {
        float v = floorf(log2f(amax)) - 2.0f + 127.0f;
        e = (v != v) ? 0 : (v <= 0.0f ? 0 : (v >= 255.0f ? 255 : (uint8_t)v));
    }
    float d = e8m0_half(e);
    out[0] = e;
    for (int j = 0; j < GROUP / 2; j++)
        out[1 + j] = (uint8_t)(mxfp4_best_index(x[j], d) | (mxfp4_best_index(x[j + GROUP / 2], d) << 4));
}

/* mxfp4.rs:52-59 */
void lo_dequantize_mxfp4_block(const uint8_t *b, float *y) {
    float d = e8m0_half(b[0]);
    for (int j = 0; j < GROUP / 2; j++) {
        uint8_t q = b[1 + j];
        y[j] = (float)MXFP4_KV[q & 15] * d;
        y[j + GROUP / 2] = (float)MXFP4_KV[q >> 4] * d;
    }
}

/* mxfp4.rs:66-84: packed e2m1 pairs (byte i = element 2i low, 2i + 1 high) + one e8m0 scale per 32 elements
 * -> MXFP4 blocks. `out` holds rows * cols / 32 * 17 bytes. */
void lo_mxfp4_from_e2m1_pairs(const uint8_t *packed, const uint8_t *scales, size_t rows, size_t cols, uint8_t *out) {
    size_t nb = rows * cols / GROUP;
    for (size_t bi = 0; bi < nb; bi++) {
        const uint8_t *src = packed + bi * (GROUP / 2);
        uint8_t *dst = out + bi * MXFP4_BYTES;
        uint8_t codes[GROUP];
        dst[0] = scales[bi];
        for (int i = 0; i < GROUP / 2; i++) {
            codes[2 * i] = src[i] & 15;
            codes[2 * i + 1] = src[i] >> 4;
        }
        for (int j = 0; j < GROUP / 2; j++) dst[1 + j] = (uint8_t)(codes[j] | (codes[j + GROUP / 2] << 4));
    }
}

/* lib.rs:131 / imp.rs:73-116. `out` holds layout.total bytes; padding is zeroed. Returns 0, or
 * -1 when the format is unknown or cols is not a positive multiple of the block length. */
int lo_quantize(int fmt, const float *data, size_t rows, size_t cols, uint8_t *out) {
    size_t L[5];
    if (cols == 0 || lo_layout(fmt, rows, cols, L) != 0) return -1;
    if (is_iqfmt(fmt)) return -1; /* the lattice-search quantizers (iq2.rs:99-452, iq3.rs:47-220) are not restated */
    memset(out, 0, L[4]);
    if (fmt == LO_FMT_MXFP4) {
        size_t nb = rows * cols / GROUP;
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < (long long)nb; i++) lo_quantize_mxfp4_block(data + (size_t)i * GROUP, out + (size_t)i * MXFP4_BYTES);
        return 0;
    }
    if (is_kfmt(fmt)) {
        size_t nb = rows * cols / QK;
        size_t bb = (size_t)block_bytes(fmt);
#pragma omp parallel for schedule(static)
        for (long long i = 0; i < (long long)nb; i++) {
            if (fmt == LO_FMT_Q4K) lo_quantize_q4k_block(data + (size_t)i * QK, out + (size_t)i * bb);
            else if (fmt == LO_FMT_Q5K) lo_quantize_q5k_block(data + (size_t)i * QK, out + (size_t)i * bb);
            else lo_quantize_q6k_block(data + (size_t)i * QK, out + (size_t)i * bb);
        }
        return 0;
    }
    size_t ng = rows * (cols / GROUP);
#pragma omp parallel for schedule(static)
    for (long long gi = 0; gi < (long long)ng; gi++) {
        float d = fmt == LO_FMT_INT8 ? quant_group_i8(data + (size_t)gi * GROUP, out + (size_t)gi * GROUP)
                                     : quant_group_i4(data + (size_t)gi * GROUP, out + (size_t)gi * (GROUP / 2));
        wr_h(out, L[2] + (size_t)gi * 2, d);
    }
    return 0;
}

/* imp.rs:124-160 */
int lo_dequantize_iq_block(int fmt, const uint8_t *b, float *y);
int lo_dequantize_row(int fmt, const uint8_t *bytes, size_t rows, size_t cols, size_t row, float *out) {
    size_t L[5];
    if (cols == 0 || lo_layout(fmt, rows, cols, L) != 0 || row >= rows) return -1;
    if (is_iqfmt(fmt)) {
        size_t nb = cols / QK, bb = (size_t)block_bytes(fmt);
        for (size_t b = 0; b < nb; b++)
            if (lo_dequantize_iq_block(fmt, bytes + (row * nb + b) * bb, out + b * QK) != 0) return -1;
        return 0;
    }
    if (fmt == LO_FMT_MXFP4) {
        size_t nb = cols / GROUP;
        for (size_t b = 0; b < nb; b++) lo_dequantize_mxfp4_block(bytes + (row * nb + b) * MXFP4_BYTES, out + b * GROUP);
        return 0;
    }
    if (is_kfmt(fmt)) {
        size_t nb = cols / QK, bb = (size_t)block_bytes(fmt);
        const uint8_t *rb = bytes + row * nb * bb;
        for (size_t b = 0; b < nb; b++) {
            if (fmt == LO_FMT_Q4K) lo_dequantize_q4k_block(rb + b * bb, out + b * QK);
            else if (fmt == LO_FMT_Q5K) lo_dequantize_q5k_block(rb + b * bb, out + b * QK);
            else lo_dequantize_q6k_block(rb + b * bb, out + b * QK);
        }
        return 0;
    }
    size_t gpr = cols / GROUP;
    for (size_t g = 0; g < gpr; g++) {
        float d = rd_h(bytes, L[2] + (row * gpr + g) * 2);
        if (fmt == LO_FMT_INT4) { /* imp.rs:148-156 */
            const uint8_t *b = bytes + (row * cols + g * GROUP) / 2;
            for (int j = 0; j < GROUP / 2; j++) {
                out[g * GROUP + j] = (float)((int)(b[j] & 0x0F) - 8) * d;
                out[g * GROUP + j + GROUP / 2] = (float)((int)(b[j] >> 4) - 8) * d;
            }
            continue;
        }
        const int8_t *q = (const int8_t *)(bytes + row * cols + g * GROUP);
        for (int t = 0; t < GROUP; t++) out[g * GROUP + t] = (float)q[t] * d;
    }
    return 0;
}

/* imp.rs:162-169 */
int lo_dequantize(int fmt, const uint8_t *bytes, size_t rows, size_t cols, float *out) {
    size_t L[5];
    if (cols == 0 || lo_layout(fmt, rows, cols, L) != 0) return -1;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)rows; r++) lo_dequantize_row(fmt, bytes, rows, cols, (size_t)r, out + (size_t)r * cols);
    return 0;
}

/* imp.rs:171-200. K formats: copy + zero pad. Int8: GGUF block_q8_0 (f16 d, 32 x i8) -> planes.
 * Returns 0, -1 bad format/shape, -2 when n_bytes is not what the shape needs. */
int lo_from_ggml_blocks(int fmt, const uint8_t *blocks, size_t n_bytes, size_t rows, size_t cols, uint8_t *out) {
    size_t L[5];
    if (cols == 0 || lo_layout(fmt, rows, cols, L) != 0) return -1;
    if (fmt != LO_FMT_INT8 && fmt != LO_FMT_INT4) {
        if (n_bytes != L[1]) return -2;
        memset(out, 0, L[4]);
        memcpy(out, blocks, L[1]);
        return 0;
    }
    size_t ng = rows * (cols / GROUP);
    size_t blk = fmt == LO_FMT_INT8 ? 34 : 18, payload = fmt == LO_FMT_INT8 ? GROUP : GROUP / 2; /* block_q8_0 / block_q4_0 */
    if (n_bytes != ng * blk) return -2;
    memset(out, 0, L[4]);
    for (size_t gi = 0; gi < ng; gi++) {
        const uint8_t *b = blocks + gi * blk;
        out[L[2] + gi * 2] = b[0];
        out[L[2] + gi * 2 + 1] = b[1];
        memcpy(out + gi * payload, b + 2, payload);
    }
    return 0;
}

/* ------------------------------------------------------------------ activation quantizer */
/* crates/lapid-cpu/src/matmul/quant.rs:68-89. x, q: k values; s (and bs when not NULL): k/32. */
void lo_quantize_row_sums(const float *x, size_t k, int8_t *q, float *s, float *bs) {
    size_t ng = k / GROUP;
    for (size_t g = 0; g < ng; g++) {
        const float *xg = x + g * GROUP;
        float mx[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int c = 0; c < 4; c++)
            for (int l = 0; l < 8; l++) {
                float a = fabsf(xg[c * 8 + l]);
                if (a > mx[l]) mx[l] = a; /* f32::max ignores a NaN operand */
            }
        float amax = 0.0f;
        for (int l = 0; l < 8; l++)
            if (mx[l] > amax) amax = mx[l];
        float d = amax / 127.0f;
        float id = d > 0.0f ? 1.0f / d : 0.0f;
        s[g] = d;
        int sum = 0;
        for (int t = 0; t < GROUP; t++) {
            float r = (xg[t] * id + 12582912.0f) - 12582912.0f; /* math.rs:134-136 */
            /* Rust's `as i32` saturates and maps NaN to 0 (a C cast of an out-of-range float is undefined): a
             * group of denormals has d > 0 but 1/d = inf, so r can be +-inf here */
            int v = (r != r) ? 0 : r >= 2147483648.0f ? 2147483647 : r <= -2147483648.0f ? (-2147483647 - 1) : (int)r;
            v = clampi(v, -127, 127);
            q[g * GROUP + t] = (int8_t)v;
            sum += v;
        }
        if (bs) bs[g] = d * (float)sum;
    }
}

/* ------------------------------------------------------------------ decode tiles */
/* crates/lapid-cpu/src/kquant.rs:51-91 */
static void unpack_block(int fmt, const uint8_t *b, int8_t *out) {
    if (fmt == LO_FMT_Q4K) {
        const uint8_t *qs = b + 16;
        for (int j = 0; j < 4; j++)
            for (int l = 0; l < 32; l++) {
                uint8_t x = qs[j * 32 + l];
                out[j * 64 + l] = (int8_t)(x & 0xF);
                out[j * 64 + 32 + l] = (int8_t)(x >> 4);
            }
        return;
    }
    if (fmt == LO_FMT_Q5K) {
        const uint8_t *qh = b + 16, *qs = b + 48;
        for (int j = 0; j < 4; j++) {
            uint8_t u1 = (uint8_t)(1u << (2 * j)), u2 = (uint8_t)(2u << (2 * j));
            for (int l = 0; l < 32; l++) {
                uint8_t x = qs[j * 32 + l];
                out[j * 64 + l] = (int8_t)((x & 0xF) + ((qh[l] & u1) ? 16 : 0));
                out[j * 64 + 32 + l] = (int8_t)((x >> 4) + ((qh[l] & u2) ? 16 : 0));
            }
        }
        return;
    }
    for (int n = 0; n < 2; n++) {
        const uint8_t *ql = b + n * 64, *qh = b + 128 + n * 32;
        int8_t *o = out + n * 128;
        for (int l = 0; l < 32; l++) {
            o[l] = (int8_t)(((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
            o[l + 32] = (int8_t)(((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
            o[l + 64] = (int8_t)(((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
            o[l + 96] = (int8_t)(((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
        }
    }
}

static inline float idot(const int8_t *a, const int8_t *w, int n) {
    int s = 0;
    for (int t = 0; t < n; t++) s += (int)a[t] * (int)w[t];
    return (float)s;
}

/* One output column of the K-format decode path for `rows` activation rows:
 * crates/lapid-cpu/src/kquant.rs:202-244 (the tile computes 4 columns x R rows; each (row, column)
 * accumulator is independent, so one column at a time gives the same values). */
static void kcol(int fmt, const uint8_t *wrow, size_t k, size_t rows, const int8_t *qa, const float *sa,
                 const float *bsa, float *acc /* [rows] */) {
    size_t kg = k / GROUP;
    int8_t q[QK];
    size_t bb = (size_t)block_bytes(fmt);
    for (size_t r = 0; r < rows; r++) acc[r] = 0.0f;
    for (size_t blk = 0; blk < k / QK; blk++) {
        const uint8_t *b = wrow + blk * bb;
        unpack_block(fmt, b, q);
        float s[8], m[8];
        float d6 = 0.0f;
        if (fmt == LO_FMT_Q4K || fmt == LO_FMT_Q5K) { /* kquant.rs:36-46 */
            float d = rd_h(b, 0), dmin = rd_h(b, 2);
            for (int j = 0; j < 8; j++) {
                uint8_t sc, mn;
                scale_min_k4(j, b + 4, &sc, &mn);
                s[j] = d * (float)sc;
                m[j] = dmin * (float)mn;
            }
        } else {
            d6 = rd_h(b, 208);
        }
        for (size_t r = 0; r < rows; r++) {
            const int8_t *a = qa + r * k + blk * QK;
            const float *as = sa + r * kg + blk * 8;
            if (fmt == LO_FMT_Q6K) {
                for (int g = 0; g < 8; g++) {
                    int n = g / 4, w = g % 4;
                    float s0 = (float)(int8_t)b[192 + n * 8 + 2 * w];
                    float s1 = (float)(int8_t)b[192 + n * 8 + 2 * w + 1];
                    float v = s0 * idot(a + g * 32, q + g * 32, 16) + s1 * idot(a + g * 32 + 16, q + g * 32 + 16, 16);
                    acc[r] += d6 * as[g] * v;
                }
            } else {
                const float *abs_ = bsa + r * kg + blk * 8;
                for (int g = 0; g < 8; g++) acc[r] += s[g] * as[g] * idot(a + g * 32, q + g * 32, 32) - m[g] * abs_[g];
            }
        }
    }
}

/* ------------------------------------------------------------------ i-quants (crates/lapid-quant/src/iq2.rs, iq3.rs; crates/lapid-cpu/src/iquant.rs)
 * The codebooks are data of the formats, not arithmetic: the caller hands in the 15488 bytes the reference keeps
 * as its own test fixture (crates/lapid-quant/tests/fixtures/iquant/grids.bin, read by iquant_golden.rs:53-62 as
 * iq2xxs_grid u64[256] | iq2s_grid u64[1024] | iq3xxs_grid u32[256] | ksigns u8[128] | iq2xs_grid u64[512]). */
#define IQ_GRID_BYTES 15488
static uint8_t IQ_GRIDS[IQ_GRID_BYTES];
static int iq_grids_set = 0;
void lo_set_iq_grids(const uint8_t *bytes) {
    memcpy(IQ_GRIDS, bytes, IQ_GRID_BYTES);
    iq_grids_set = 1;
}
static inline uint32_t rd_u32(const uint8_t *b, size_t o) { return (uint32_t)b[o] | ((uint32_t)b[o + 1] << 8) | ((uint32_t)b[o + 2] << 16) | ((uint32_t)b[o + 3] << 24); }

/* iquant.rs:40-64 (`group8`): the 8 grid bytes of 8-group j (0..32) and its sign bits */
static uint8_t iq_group8(int fmt, const uint8_t *b, int j, uint8_t g[8]) {
    const uint8_t *ksigns = IQ_GRIDS + 11264;
    int ib = j / 4, l = j % 4;
    if (fmt == LO_FMT_IQ2XXS) {
        uint32_t a1 = rd_u32(b, 6 + 8 * (size_t)ib);
        memcpy(g, IQ_GRIDS + 8 * (size_t)b[2 + 8 * ib + l], 8);
        return ksigns[(a1 >> (7 * l)) & 127];
    }
    if (fmt == LO_FMT_IQ2XS) {
        uint32_t q = (uint32_t)b[2 + 2 * j] | ((uint32_t)b[3 + 2 * j] << 8);
        memcpy(g, IQ_GRIDS + 11392 + 8 * (size_t)(q & 511), 8);
        return ksigns[q >> 9];
    }
    if (fmt == LO_FMT_IQ2S) {
        size_t idx = (size_t)b[2 + j] | (((size_t)b[66 + ib] << (8 - 2 * l)) & 0x300);
        memcpy(g, IQ_GRIDS + 2048 + 8 * idx, 8);
        return b[34 + j];
    }
    uint32_t aux = rd_u32(b, 66 + 4 * (size_t)ib);
    memcpy(g, IQ_GRIDS + 10240 + 4 * (size_t)b[2 + 8 * ib + 2 * l], 4);
    memcpy(g + 4, IQ_GRIDS + 10240 + 4 * (size_t)b[2 + 8 * ib + 2 * l + 1], 4);
    return ksigns[(aux >> (7 * l)) & 127];
}

/* iquant.rs:66-89 (`half_scales`), the same expressions as the dequantizers (iq2.rs:41-44, :59-60, :78; iq3.rs:24-25) */
static void iq_half_scales(int fmt, const uint8_t *b, float s[16]) {
    float d = rd_h(b, 0);
    for (int ib = 0; ib < 8; ib++) {
        float v0, v1;
        if (fmt == LO_FMT_IQ2XXS) {
            v0 = v1 = d * (0.5f + (float)(rd_u32(b, 6 + 8 * (size_t)ib) >> 28)) * 0.25f;
        } else if (fmt == LO_FMT_IQ2XS || fmt == LO_FMT_IQ2S) {
            uint8_t sc = b[(fmt == LO_FMT_IQ2XS ? 66 : 74) + ib];
            v0 = d * (0.5f + (float)(sc & 15)) * 0.25f;
            v1 = d * (0.5f + (float)(sc >> 4)) * 0.25f;
        } else {
            v0 = v1 = d * (0.5f + (float)(rd_u32(b, 66 + 4 * (size_t)ib) >> 28)) * 0.5f;
        }
        s[2 * ib] = v0;
        s[2 * ib + 1] = v1;
    }
}

/* iq2.rs:38-90, iq3.rs:18-39: y = db * f32(grid byte) * (+1 | -1) */
int lo_dequantize_iq_block(int fmt, const uint8_t *b, float *y) {
    if (!is_iqfmt(fmt) || !iq_grids_set) return -1;
    float s[16];
    iq_half_scales(fmt, b, s);
    for (int j = 0; j < 32; j++) {
        uint8_t g[8];
        uint8_t signs = iq_group8(fmt, b, j, g);
        for (int i = 0; i < 8; i++) y[8 * j + i] = s[j / 2] * (float)g[i] * ((signs >> i) & 1 ? -1.0f : 1.0f);
    }
    return 0;
}

/* iquant.rs:92-103 (`unpack_block`) and :108-128 (`tile_scalar`): one output column,
 * acc += sc[h] * da[h / 2] * f32(dot of 16 elements), halves in order */
static void iqcol(int fmt, const uint8_t *wrow, size_t k, size_t rows, const int8_t *qa, const float *sa, float *acc) {
    size_t kg = k / GROUP, bb = (size_t)block_bytes(fmt);
    int8_t q[QK];
    float sc[16];
    for (size_t r = 0; r < rows; r++) acc[r] = 0.0f;
    for (size_t blk = 0; blk < k / QK; blk++) {
        const uint8_t *b = wrow + blk * bb;
        for (int j = 0; j < 32; j++) {
            uint8_t g[8];
            uint8_t signs = iq_group8(fmt, b, j, g);
            for (int i = 0; i < 8; i++) q[8 * j + i] = (signs >> i) & 1 ? (int8_t)-(int)g[i] : (int8_t)g[i];
        }
        iq_half_scales(fmt, b, sc);
        for (size_t r = 0; r < rows; r++) {
            const int8_t *a = qa + r * k + blk * QK;
            for (int h = 0; h < 16; h++) acc[r] += sc[h] * sa[r * kg + blk * 8 + (size_t)h / 2] * idot(a + 16 * h, q + 16 * h, 16);
        }
    }
}

/* crates/lapid-cpu/src/mxfp4.rs:27-58: one output column of the MXFP4 decode tile, acc += d * da * f32(dot) */
static void mxcol(const uint8_t *wrow, size_t k, size_t rows, const int8_t *qa, const float *sa, float *acc) {
    size_t kg = k / GROUP;
    int8_t q[GROUP];
    for (size_t r = 0; r < rows; r++) acc[r] = 0.0f;
    for (size_t blk = 0; blk < kg; blk++) {
        const uint8_t *b = wrow + blk * MXFP4_BYTES;
        for (int j = 0; j < GROUP / 2; j++) {
            q[j] = MXFP4_KV[b[1 + j] & 15];
            q[j + GROUP / 2] = MXFP4_KV[b[1 + j] >> 4];
        }
        float d = e8m0_half(b[0]);
        for (size_t r = 0; r < rows; r++) acc[r] += d * sa[r * kg + blk] * idot(qa + r * k + blk * GROUP, q, GROUP);
    }
}

/* crates/lapid-cpu/src/matmul/qkernels.rs:60-84 */
static void i8col(int fmt, const uint8_t *bytes, size_t scales_off, size_t col, size_t k, size_t rows, const int8_t *qa,
                  const float *sa, float *acc) {
    size_t kg = k / GROUP;
    int8_t unpacked[GROUP];
    for (size_t r = 0; r < rows; r++) acc[r] = 0.0f;
    for (size_t g = 0; g < kg; g++) {
        const int8_t *bq = (const int8_t *)(bytes + col * k + g * GROUP);
        if (fmt == LO_FMT_INT4) { /* QMat::group_i8, qmat.rs:97-112: nibbles re-centred to -8..7 */
            const uint8_t *b = bytes + (col * k + g * GROUP) / 2;
            for (int j = 0; j < GROUP / 2; j++) {
                unpacked[j] = (int8_t)((int)(b[j] & 0x0F) - 8);
                unpacked[j + GROUP / 2] = (int8_t)((int)(b[j] >> 4) - 8);
            }
            bq = unpacked;
        }
        float db = rd_h(bytes, scales_off + (col * kg + g) * 2);
        for (size_t r = 0; r < rows; r++) {
            float da = sa[r * kg + g];
            acc[r] += idot(qa + r * k + g * GROUP, bq, GROUP) * (da * db);
        }
    }
}

/* ------------------------------------------------------------------ the launch */
typedef struct {
    size_t offset, batch_stride, row_stride;
} lo_view;

/* Error codes mirror the reference's `Error::code` strings (crates/lapid-cpu/src/matmul/mod.rs). */
#define LO_OK 0
#define LO_INVALID_LAUNCH 1
#define LO_SHAPE_MISMATCH 2
#define LO_OUT_OF_BOUNDS 3
#define LO_UNSUPPORTED 4

/*
 * out[bt, i, j] = sum_p A[bt, i, p] * dequant(W)[j, p] (+ bias[j] when bias != NULL), as
 * `matmul::run` computes it for a quantized, transposed B (mod.rs:165-262):
 *   batch*m <= 8 (and !force_f32_act): int8 activations x integer weights (quant.rs:91-185);
 *   otherwise: f32 activations x dequantized f32 weights, accumulated in k order (qdeq.rs);
 *     fma != 0 accumulates with a fused multiply-add like the x86 AVX2 micro-kernel
 *     (kernels.rs:95-119), fma == 0 with a separate multiply and add like `micro_scalar` on x86.
 * a_len / out_len / w_len are the element / byte counts of the buffers, for validation.
 * `path` (when not NULL) receives 0 for the int8-activation path, 1 for the f32 path.
 */
int lo_matmul(int fmt, const float *a, size_t a_len, lo_view av, const uint8_t *w, size_t w_len, size_t w_rows,
              size_t w_cols, const float *bias, float *out, size_t out_len, lo_view ov, size_t batch, size_t m,
              size_t n, size_t k, int force_f32_act, int fma, int *path) {
    size_t rows = batch * m;
    if (rows * n == 0) return LO_OK;
    size_t last = ov.offset + (batch - 1) * ov.batch_stride + (m - 1) * ov.row_stride + n;
    if (out_len < last) return LO_OUT_OF_BOUNDS;
    if (k > 0) {
        size_t alast = av.offset + (batch - 1) * av.batch_stride + (m - 1) * av.row_stride + k;
        if (a_len < alast) return LO_OUT_OF_BOUNDS;
    }
    if (k == 0) {
        for (size_t r = 0; r < rows; r++) {
            float *o = out + ov.offset + (r / m) * ov.batch_stride + (r % m) * ov.row_stride;
            for (size_t j = 0; j < n; j++) o[j] = bias ? 0.0f + bias[j] : 0.0f;
        }
        return LO_OK;
    }
    size_t L[5];
    if (lo_layout(fmt, w_rows, w_cols, L) != 0) return LO_INVALID_LAUNCH; /* QMat::new, qmat.rs:38-60 */
    if (w_len < L[2] + L[3]) return LO_OUT_OF_BOUNDS;
    if (w_rows != n || w_cols != k) return LO_SHAPE_MISMATCH;
    if (is_iqfmt(fmt) && !iq_grids_set) return LO_UNSUPPORTED;

    if (rows <= 8 && !force_f32_act) {
        if (path) *path = 0;
        size_t kg = k / GROUP;
        int8_t *qa = (int8_t *)malloc(rows * k);
        float *sa = (float *)malloc(rows * kg * sizeof(float));
        float *bs = (float *)malloc(rows * kg * sizeof(float));
        for (size_t r = 0; r < rows; r++) {
            const float *x = a + av.offset + (r / m) * av.batch_stride + (r % m) * av.row_stride;
            lo_quantize_row_sums(x, k, qa + r * k, sa + r * kg, (fmt == LO_FMT_Q4K || fmt == LO_FMT_Q5K) ? bs + r * kg : NULL);  /* quant.rs:101 */
        }
        size_t bb = (size_t)block_bytes(fmt);
#pragma omp parallel for schedule(static)
        for (long long j = 0; j < (long long)n; j++) {
            float acc[8];
            if (fmt == LO_FMT_MXFP4) mxcol(w + (size_t)j * kg * MXFP4_BYTES, k, rows, qa, sa, acc);
            else if (is_iqfmt(fmt)) iqcol(fmt, w + (size_t)j * (k / QK) * bb, k, rows, qa, sa, acc);
            else if (fmt == LO_FMT_INT8 || fmt == LO_FMT_INT4) i8col(fmt, w, L[2], (size_t)j, k, rows, qa, sa, acc);
            else kcol(fmt, w + (size_t)j * (k / QK) * bb, k, rows, qa, sa, bs, acc);
            for (size_t r = 0; r < rows; r++) {
                float v = bias ? acc[r] + bias[j] : acc[r];
                out[ov.offset + (r / m) * ov.batch_stride + (r % m) * ov.row_stride + (size_t)j] = v;
            }
        }
        free(qa);
        free(sa);
        free(bs);
        return LO_OK;
    }

    if (path) *path = 1;
    /* qdeq: every output is the sum over p = 0..k, in order, of a[p] * w[p] from a zero
     * accumulator. As in the reference, A is packed once into k-major panels of MR = 6 rows and
     * the weights are expanded into k-major panels of NR = 16 columns (pack_panel,
     * qdeq.rs:26-55); a 6 x 16 register tile walks k (kernels.rs:29-46, :95-119). */
    enum { MRP = 6, NRP = 16 };
    size_t mpan = (rows + MRP - 1) / MRP;
    size_t npan = (n + NRP - 1) / NRP;
    float *ap = (float *)malloc(mpan * k * MRP * sizeof(float));
#pragma omp parallel for schedule(static)
    for (long long ip = 0; ip < (long long)mpan; ip++) {
        for (int r = 0; r < MRP; r++) {
            size_t rr = (size_t)ip * MRP + (size_t)r;
            float *dst = ap + (size_t)ip * k * MRP + (size_t)r;
            if (rr < rows) {
                const float *x = a + av.offset + (rr / m) * av.batch_stride + (rr % m) * av.row_stride;
                for (size_t p = 0; p < k; p++) dst[p * MRP] = x[p];
            } else {
                for (size_t p = 0; p < k; p++) dst[p * MRP] = 0.0f;
            }
        }
    }
#pragma omp parallel
    {
        float *wp = (float *)malloc((size_t)NRP * k * sizeof(float));
        float *rowbuf = (float *)malloc(k * sizeof(float));
#pragma omp for schedule(dynamic, 1)
        for (long long pj = 0; pj < (long long)npan; pj++) {
            size_t j0 = (size_t)pj * NRP;
            size_t jn = n - j0 < NRP ? n - j0 : NRP;
            for (size_t c = 0; c < NRP; c++) {
                if (c < jn) {
                    lo_dequantize_row(fmt, w, w_rows, w_cols, j0 + c, rowbuf);
                    for (size_t p = 0; p < k; p++) wp[p * NRP + c] = rowbuf[p];
                } else {
                    for (size_t p = 0; p < k; p++) wp[p * NRP + c] = 0.0f;
                }
            }
            for (size_t ip = 0; ip < mpan; ip++) {
                const float *apn = ap + ip * k * MRP;
                float acc[MRP][NRP];
                for (int r = 0; r < MRP; r++)
                    for (int c = 0; c < NRP; c++) acc[r][c] = 0.0f;
                if (fma) {
                    for (size_t p = 0; p < k; p++) {
                        const float *wr = wp + p * NRP;
                        const float *ar = apn + p * MRP;
                        for (int r = 0; r < MRP; r++)
                            for (int c = 0; c < NRP; c++) acc[r][c] = fmaf(ar[r], wr[c], acc[r][c]);
                    }
                } else {
                    for (size_t p = 0; p < k; p++) {
                        const float *wr = wp + p * NRP;
                        const float *ar = apn + p * MRP;
                        for (int r = 0; r < MRP; r++)
                            for (int c = 0; c < NRP; c++) acc[r][c] = ar[r] * wr[c] + acc[r][c];
                    }
                }
                for (int r = 0; r < MRP; r++) {
                    size_t rr = ip * MRP + (size_t)r;
                    if (rr >= rows) break;
                    float *o = out + ov.offset + (rr / m) * ov.batch_stride + (rr % m) * ov.row_stride + j0;
                    for (size_t c = 0; c < jn; c++) o[c] = bias ? acc[r][c] + bias[j0 + c] : acc[r][c];
                }
            }
        }
        free(wp);
        free(rowbuf);
    }
    free(ap);
    return LO_OK;
}

int lo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void lo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

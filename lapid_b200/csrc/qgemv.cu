// Decode GEMV over quantized weights: out[r, j] = sum_k A[r, k] * dequant(W)[j, k] for 1..8
// activation rows, computed with lapid-cpu's int8-activation arithmetic
// (crates/lapid-cpu/src/matmul/quant.rs:91-185):
//
//   Q4_K  acc += (d*sc_g)*da_g*f32(sum_32 qa*qw) - (dmin*m_g)*bs_g      crates/lapid-cpu/src/kquant.rs:236-239
//   Q6_K  acc += (d*da_g)*(sc_2g*f32(sum_16) + sc_2g+1*f32(sum_16))      crates/lapid-cpu/src/kquant.rs:224-233
//   Int8  acc += f32(sum_32 qa*qb)*(da_g*db_g)                           crates/lapid-cpu/src/matmul/qkernels.rs:60-84
//
// The integer dot products are exact, so only the order of the f32 group sums differs from the
// CPU path (which itself differs between its scalar, AVX2 and NEON tiles).
//
// Shape of the kernel. The op is a pure stream over the weight bytes (0.5625 / 0.8203 / 1.0625
// bytes per element), so it is built around keeping HBM requests in flight:
//  * every warp owns a private ring of shared-memory stages and fills it with 128-bit
//    `cp.async` copies (coalesced, L1-bypassing, no registers held while in flight). A stage is
//    eight 256-element super-blocks of each of C weight rows; rows are byte streams, so the
//    2-byte-aligned 210-byte Q6_K blocks cost nothing extra: the copy moves the 16-byte aligned
//    superset of the span and the consumer indexes from the remainder;
//  * warps never synchronise with each other: a warp waits on its own copy groups only;
//  * a lane owns 64 weights of one super-block per stage and keeps them unpacked in registers
//    while it walks the activation rows (`dp4a` against int8 activations served by L1);
//  * per task (C output columns) one warp-shuffle reduction, then lane 0 applies the epilogue;
//  * weights do not depend on the producer of the activations, so staging starts before the
//    programmatic-dependent-launch wait: the ring is already full when the activations arrive.
#include "common.cuh"
#include "kernels.h"

namespace lb {

constexpr int WARPS = 8;          // warps per CTA
constexpr int STAGE_BLOCKS = 8;   // super-blocks (256 elements) per stage and weight row

template <int FMT> struct Geo;
template <> struct Geo<FMT_Q4K> { static constexpr int SPAN = STAGE_BLOCKS * Q4K_BYTES + 16; };
template <> struct Geo<FMT_Q5K> { static constexpr int SPAN = STAGE_BLOCKS * Q5K_BYTES + 16; };
template <> struct Geo<FMT_Q6K> { static constexpr int SPAN = STAGE_BLOCKS * Q6K_BYTES + 16; };
// Int8: 2048 quant bytes (+16) then 64 f16 scales (+16)
template <> struct Geo<FMT_INT8> {
    static constexpr int QSPAN = STAGE_BLOCKS * 256 + 16;
    static constexpr int SPAN = QSPAN + STAGE_BLOCKS * 16 + 16;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void *sdst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(sdst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Warp-collective copy of global bytes [gbeg, gbeg+len) so that byte gbeg lands at
// sdst + (gbeg & 15). `base` and `sdst` are 16-byte aligned. Chunks that would read past the end
// of the buffer are moved byte by byte instead.
__device__ __forceinline__ void warp_copy_span(uint8_t *sdst, const uint8_t *base, uint64_t gbeg, uint32_t len,
                                               uint64_t buf_bytes, int lane) {
    uint64_t a0 = gbeg & ~15ull;
    uint32_t nchunks = (uint32_t)((gbeg - a0) + len + 15) >> 4;
    for (uint32_t ch = lane; ch < nchunks; ch += 32) {
        uint64_t ga = a0 + 16ull * ch;
        if (ga + 16 <= buf_bytes) {
            cp_async16(sdst + 16 * ch, base + ga);
        } else {
            for (int b = 0; b < 16; b++) sdst[16 * ch + b] = (ga + b < buf_bytes) ? base[ga + b] : (uint8_t)0;
        }
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// 32 bytes at a 2-byte aligned shared address as eight words
__device__ __forceinline__ void lds_32B_align2(const uint8_t *p, uint32_t (&w)[8]) {
    const uint32_t *q = (const uint32_t *)((uintptr_t)p & ~(uintptr_t)3);
    uint32_t sh = ((uint32_t)(uintptr_t)p & 3u) * 8u;
    uint32_t prev = q[0];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        uint32_t nxt = q[i + 1];
        w[i] = __funnelshift_r(prev, nxt, sh);
        prev = nxt;
    }
}

template <int FMT, int M, int C, int STAGES>
__global__ void __launch_bounds__(WARPS * 32) qgemv_kernel(GemvArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    constexpr int SPAN = Geo<FMT>::SPAN;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t *ring = smem + (size_t)warp * (STAGES * C * SPAN);
    if (p.ids) {
        // Expert-indexed launch (Kernel::MatMulId at decode sizes): grid row y is one (token, slot)
        // pair, a one-row GEMV of the token's activations against the matrix its id selects. The
        // ids come from the kernel before this one, so nothing is staged ahead of it.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        const uint32_t pair = blockIdx.y, token = pair / p.id_r;
        const int32_t id = p.ids[pair];
        const bool bad = id < 0 || (uint32_t)id >= p.id_e;
        if (bad && p.status && threadIdx.x == 0) atomicOr(p.status, 128);
        p.w += bad ? 0 : (uint64_t)id * p.id_stride;
        p.w_bytes = p.id_stride;
        p.qa += (uint64_t)token * p.k;
        p.da += (uint64_t)token * (p.k / GROUP);
        if (p.bs) p.bs += (uint64_t)token * (p.k / GROUP);
        p.out_off += (uint64_t)pair * p.n;
    }

    const uint32_t k = p.k, n = p.n;
    const uint32_t kg = k / GROUP;
    const uint32_t nblk = (k + QK - 1) / QK;
    const uint32_t nst = (nblk + STAGE_BLOCKS - 1) / STAGE_BLOCKS;
    const uint32_t tasks = (n + C - 1) / C;
    const uint32_t total_warps = gridDim.x * WARPS;
    const uint32_t gw = blockIdx.x * WARPS + warp;
    const uint32_t my_tasks = gw < tasks ? (tasks - gw + total_warps - 1) / total_warps : 0;
    const uint32_t items = my_tasks * nst;

    auto issue = [&](uint32_t item) {
        uint32_t j = item / nst, st = item - j * nst;
        uint32_t t = gw + j * total_warps;
        uint8_t *slot = ring + (size_t)(item % STAGES) * (C * SPAN);
#pragma unroll
        for (int c = 0; c < C; c++) {
            uint32_t row = min(t * C + c, n - 1);  // tail columns repeat the last one; results discarded
            if constexpr (FMT == FMT_INT8) {
                uint32_t e0 = st * STAGE_BLOCKS * QK;
                uint32_t len = min((uint32_t)(STAGE_BLOCKS * QK), k - e0);
                warp_copy_span(slot + c * SPAN, p.w, (uint64_t)row * k + e0, len, p.w_bytes, lane);
                uint32_t g0 = st * STAGE_BLOCKS * 8;
                uint32_t ng = min((uint32_t)(STAGE_BLOCKS * 8), kg - g0);
                warp_copy_span(slot + c * SPAN + Geo<FMT_INT8>::QSPAN, p.w,
                               p.scales_offset + ((uint64_t)row * kg + g0) * 2, ng * 2, p.w_bytes, lane);
            } else {
                constexpr int BB = FMT == FMT_Q4K ? Q4K_BYTES : FMT == FMT_Q5K ? Q5K_BYTES : Q6K_BYTES;
                uint32_t b0 = st * STAGE_BLOCKS;
                uint32_t nb = min((uint32_t)STAGE_BLOCKS, nblk - b0);
                warp_copy_span(slot + c * SPAN, p.w, ((uint64_t)row * nblk + b0) * BB, nb * BB, p.w_bytes, lane);
            }
        }
    };

    // The weights are constants of the model: stage them before waiting for the kernel that
    // produces the activations.
#pragma unroll
    for (int i = 0; i < STAGES - 1; i++) {
        if ((uint32_t)i < items) issue(i);
        cp_async_commit();
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");

    float acc[M][C];
    const int blk_l = lane >> 2, pr = lane & 3;  // lane -> (super-block of the stage, 64-element part)

    for (uint32_t it = 0; it < items; it++) {
        if (it + STAGES - 1 < items) issue(it + STAGES - 1);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncwarp();

        const uint32_t j = it / nst, st = it - j * nst;
        const uint32_t t = gw + j * total_warps;
        if (st == 0) {
#pragma unroll
            for (int r = 0; r < M; r++)
#pragma unroll
                for (int c = 0; c < C; c++) acc[r][c] = 0.0f;
        }
        const uint8_t *slot = ring + (size_t)(it % STAGES) * (C * SPAN);
        const uint32_t blk = st * STAGE_BLOCKS + blk_l;  // super-block along k

        if constexpr (FMT == FMT_Q4K || FMT == FMT_Q5K) {
            // Q5_K is Q4_K with a fifth bit per weight: bit s of qh[l] (32 bytes behind the header) belongs to
            // element 32 s + l, and the nibbles follow at byte 48 (crates/lapid-quant/src/kquant.rs:355-373)
            constexpr int BB = FMT == FMT_Q5K ? Q5K_BYTES : Q4K_BYTES, QS = FMT == FMT_Q5K ? 48 : 16;
            if (blk < nblk) {
                uint32_t wlo[C][8], whi[C][8];
                float s0[C], m0[C], s1[C], m1[C];
#pragma unroll
                for (int c = 0; c < C; c++) {
                    const uint8_t *b = slot + c * SPAN + blk_l * BB;  // 16-byte aligned: 144 = 9*16, 176 = 11*16
                    uint4 h = *(const uint4 *)b;
                    uint4 q0 = *(const uint4 *)(b + QS + 32 * pr);
                    uint4 q1 = *(const uint4 *)(b + QS + 16 + 32 * pr);
                    float d = half_bits_to_float(h.x & 0xffff), dmin = half_bits_to_float(h.x >> 16);
                    int sc0, mn0, sc1, mn1;
                    scale_min_pair(pr, h.y, h.z, h.w, sc0, mn0, sc1, mn1);
                    s0[c] = xmul(d, (float)sc0);
                    m0[c] = xmul(dmin, (float)mn0);
                    s1[c] = xmul(d, (float)sc1);
                    m1[c] = xmul(dmin, (float)mn1);
                    uint32_t v[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        wlo[c][i] = v[i] & 0x0F0F0F0Fu;
                        whi[c][i] = (v[i] >> 4) & 0x0F0F0F0Fu;
                    }
                    if constexpr (FMT == FMT_Q5K) {
                        uint4 h0 = *(const uint4 *)(b + 16), h1 = *(const uint4 *)(b + 32);
                        uint32_t hq[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            wlo[c][i] |= ((hq[i] >> (2 * pr)) & 0x01010101u) << 4;
                            whi[c][i] |= ((hq[i] >> (2 * pr + 1)) & 0x01010101u) << 4;
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < M; r++) {
                    const uint4 *ap = (const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)blk * QK + 64 * pr);
                    uint4 a0 = __ldg(ap), a1 = __ldg(ap + 1), a2 = __ldg(ap + 2), a3 = __ldg(ap + 3);
                    float2 das = __ldg((const float2 *)(p.da + (uint64_t)r * kg + blk * 8 + 2 * pr));
                    float2 bss = __ldg((const float2 *)(p.bs + (uint64_t)r * kg + blk * 8 + 2 * pr));
                    int al[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
                    int ah[8] = {(int)a2.x, (int)a2.y, (int)a2.z, (int)a2.w, (int)a3.x, (int)a3.y, (int)a3.z, (int)a3.w};
#pragma unroll
                    for (int c = 0; c < C; c++) {
                        int dl = 0, dh = 0;
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            dl = __dp4a((int)wlo[c][i], al[i], dl);
                            dh = __dp4a((int)whi[c][i], ah[i], dh);
                        }
                        float a_ = acc[r][c];
                        a_ = fmaf(s0[c] * das.x, (float)dl, a_);
                        a_ = fmaf(-m0[c], bss.x, a_);
                        a_ = fmaf(s1[c] * das.y, (float)dh, a_);
                        a_ = fmaf(-m1[c], bss.y, a_);
                        acc[r][c] = a_;
                    }
                }
            }
        } else if constexpr (FMT == FMT_Q6K) {
            // lane part pr = (half n, wlo): groups g = 4n+wlo (low nibbles of ql) and g+2 (high nibbles)
            if (blk < nblk) {
                const int nh = pr >> 1, wlo_ = pr & 1;
                uint32_t wa[C][8], wb[C][8];
                float sa0[C], sa1[C], sb0[C], sb1[C], dd[C];
#pragma unroll
                for (int c = 0; c < C; c++) {
                    uint32_t row = min(t * C + c, n - 1);
                    uint32_t off = (uint32_t)((((uint64_t)row * nblk + st * STAGE_BLOCKS) * Q6K_BYTES) & 15);
                    const uint8_t *b = slot + c * SPAN + off + blk_l * Q6K_BYTES;  // 2-byte aligned
                    uint32_t ql[8], qh[8];
                    lds_32B_align2(b + 64 * nh + 32 * wlo_, ql);
                    lds_32B_align2(b + 128 + 32 * nh, qh);
                    const int shA = 2 * wlo_, shB = 2 * (wlo_ + 2);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        uint32_t lo = ql[i] & 0x0F0F0F0Fu, hi = (ql[i] >> 4) & 0x0F0F0F0Fu;
                        uint32_t ha = ((qh[i] >> shA) & 0x03030303u) << 4, hb = ((qh[i] >> shB) & 0x03030303u) << 4;
                        wa[c][i] = __vsub4(lo | ha, 0x20202020u);
                        wb[c][i] = __vsub4(hi | hb, 0x20202020u);
                    }
                    const int8_t *sc = (const int8_t *)(b + 192 + 8 * nh);
                    sa0[c] = (float)sc[2 * wlo_];
                    sa1[c] = (float)sc[2 * wlo_ + 1];
                    sb0[c] = (float)sc[2 * (wlo_ + 2)];
                    sb1[c] = (float)sc[2 * (wlo_ + 2) + 1];
                    dd[c] = half_bits_to_float((uint32_t)b[208] | ((uint32_t)b[209] << 8));
                }
                const uint32_t ga = blk * 8 + 4 * nh + wlo_;  // group index along k; gb = ga + 2
#pragma unroll
                for (int r = 0; r < M; r++) {
                    const uint4 *apA = (const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)ga * GROUP);
                    uint4 a0 = __ldg(apA), a1 = __ldg(apA + 1), a2 = __ldg(apA + 4), a3 = __ldg(apA + 5);
                    float daA = __ldg(p.da + (uint64_t)r * kg + ga), daB = __ldg(p.da + (uint64_t)r * kg + ga + 2);
                    int xa[8] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w};
                    int xb[8] = {(int)a2.x, (int)a2.y, (int)a2.z, (int)a2.w, (int)a3.x, (int)a3.y, (int)a3.z, (int)a3.w};
#pragma unroll
                    for (int c = 0; c < C; c++) {
                        int dA0 = 0, dA1 = 0, dB0 = 0, dB1 = 0;
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            dA0 = __dp4a((int)wa[c][i], xa[i], dA0);
                            dA1 = __dp4a((int)wa[c][4 + i], xa[4 + i], dA1);
                            dB0 = __dp4a((int)wb[c][i], xb[i], dB0);
                            dB1 = __dp4a((int)wb[c][4 + i], xb[4 + i], dB1);
                        }
                        float vA = fmaf(sa1[c], (float)dA1, sa0[c] * (float)dA0);
                        float vB = fmaf(sb1[c], (float)dB1, sb0[c] * (float)dB0);
                        float a_ = acc[r][c];
                        a_ = fmaf(dd[c] * daA, vA, a_);
                        a_ = fmaf(dd[c] * daB, vB, a_);
                        acc[r][c] = a_;
                    }
                }
            }
        } else {  // Int8 planes: lane part = groups g0, g0+1 of its 256-element block
            const uint32_t g0 = blk * 8 + 2 * pr;
            if (g0 < kg) {
                const bool two = g0 + 1 < kg;
                uint32_t wv[C][16];
                float db0[C], db1[C];
#pragma unroll
                for (int c = 0; c < C; c++) {
                    uint32_t row = min(t * C + c, n - 1);
                    const uint8_t *qb = slot + c * SPAN + blk_l * QK + 64 * pr;  // 16-byte aligned (k % 32 == 0)
                    uint4 q0 = *(const uint4 *)qb, q1 = *(const uint4 *)(qb + 16);
                    uint4 q2 = make_uint4(0, 0, 0, 0), q3 = q2;
                    if (two) {
                        q2 = *(const uint4 *)(qb + 32);
                        q3 = *(const uint4 *)(qb + 48);
                    }
                    uint32_t v[16] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w,
                                      q2.x, q2.y, q2.z, q2.w, q3.x, q3.y, q3.z, q3.w};
#pragma unroll
                    for (int i = 0; i < 16; i++) wv[c][i] = v[i];
                    uint32_t soff = (uint32_t)((p.scales_offset + ((uint64_t)row * kg + st * STAGE_BLOCKS * 8) * 2) & 15);
                    const uint16_t *sp = (const uint16_t *)(slot + c * SPAN + Geo<FMT_INT8>::QSPAN + soff) + blk_l * 8 + 2 * pr;
                    db0[c] = half_bits_to_float(sp[0]);
                    db1[c] = two ? half_bits_to_float(sp[1]) : 0.0f;
                }
#pragma unroll
                for (int r = 0; r < M; r++) {
                    const uint4 *ap = (const uint4 *)(p.qa + (uint64_t)r * k + (uint64_t)g0 * GROUP);
                    uint4 a0 = __ldg(ap), a1 = __ldg(ap + 1);
                    uint4 a2 = make_uint4(0, 0, 0, 0), a3 = a2;
                    float da0 = __ldg(p.da + (uint64_t)r * kg + g0), da1 = 0.0f;
                    if (two) {
                        a2 = __ldg(ap + 2);
                        a3 = __ldg(ap + 3);
                        da1 = __ldg(p.da + (uint64_t)r * kg + g0 + 1);
                    }
                    int x[16] = {(int)a0.x, (int)a0.y, (int)a0.z, (int)a0.w, (int)a1.x, (int)a1.y, (int)a1.z, (int)a1.w,
                                 (int)a2.x, (int)a2.y, (int)a2.z, (int)a2.w, (int)a3.x, (int)a3.y, (int)a3.z, (int)a3.w};
#pragma unroll
                    for (int c = 0; c < C; c++) {
                        int d0 = 0, d1 = 0;
#pragma unroll
                        for (int i = 0; i < 8; i++) {
                            d0 = __dp4a((int)wv[c][i], x[i], d0);
                            d1 = __dp4a((int)wv[c][8 + i], x[8 + i], d1);
                        }
                        float a_ = acc[r][c];
                        a_ = fmaf((float)d0, da0 * db0[c], a_);
                        a_ = fmaf((float)d1, da1 * db1[c], a_);
                        acc[r][c] = a_;
                    }
                }
            }
        }
        __syncwarp();  // every lane is done with this slot before the next copy may overwrite it

        if (st == nst - 1) {
#pragma unroll
            for (int r = 0; r < M; r++) {
#pragma unroll
                for (int c = 0; c < C; c++) {
                    float v = warp_sum(acc[r][c]);
                    uint32_t col = t * C + c;
                    if (lane == 0 && col < n) {
                        uint32_t bt = r / p.m, i = r % p.m;
                        if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)col * p.ex_s2];
                        p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + col] = v;
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
}

__global__ void fill_zero_k_kernel(GemvArgs p) {
    uint64_t total = (uint64_t)p.rows * p.n;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        uint32_t r = (uint32_t)(idx / p.n), col = (uint32_t)(idx % p.n);
        uint32_t bt = r / p.m, i = r % p.m;
        float v = 0.0f;
        if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)i * p.ex_s1 + (int64_t)col * p.ex_s2];
        p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)i * p.out_rs + col] = v;
    }
}

cudaError_t launch_fill_zero_k(const GemvArgs &args, cudaStream_t stream) {
    uint64_t total = (uint64_t)args.rows * args.n;
    if (total == 0) return cudaSuccess;
    fill_zero_k_kernel<<<(unsigned)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256), 256, 0, stream>>>(args);
    return cudaGetLastError();
}

// ---- dispatch -------------------------------------------------------------------------------
// Ring depth per columns-per-task: the bytes a warp keeps in flight are (STAGES-1) * C stages,
// about 3.5-4.6 KB for Q4_K in every configuration, i.e. 55-75 KB per SM at 16 resident warps --
// above the ~45 KB per SM that HBM latency x bandwidth asks for.
template <int C> struct Depth { static constexpr int STAGES = C == 1 ? 4 : (C == 2 ? 3 : 2); };

template <int FMT, int M, int C>
static cudaError_t launch_one(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t stream) {
    constexpr int STAGES = Depth<C>::STAGES;
    auto kern = qgemv_kernel<FMT, M, C, STAGES>;
    constexpr size_t smem = (size_t)WARPS * STAGES * C * Geo<FMT>::SPAN;
    static_assert(smem <= 227 * 1024, "ring does not fit in shared memory");
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    static OccupancyCache occupancy;
    int ctas_per_sm = 1;
    if (cudaError_t e = occupancy.get(kern, WARPS * 32, smem, &ctas_per_sm); e != cudaSuccess) return e;
    uint32_t tasks = (a.n + C - 1) / C;
    uint32_t want = (tasks + WARPS - 1) / WARPS;
    uint32_t cap = (uint32_t)sm_count * (uint32_t)ctas_per_sm;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(want < cap ? want : cap);
    if (a.ids) {  // one grid row per (token, slot) pair; the rows share the resident slots
        const uint32_t share = cap / a.id_pairs > 0 ? cap / a.id_pairs : 1;
        cfg.gridDim = dim3(want < share ? want : share, a.id_pairs);
    }
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, a);
}

template <int FMT, int M> static cudaError_t launch_m(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    // Columns per warp task: more columns amortise the activation reads over more weights, fewer
    // give more tasks. Keep at least ~2 tasks per resident warp where the matrix allows it.
    uint32_t resident_warps = (uint32_t)sm_count * WARPS * 2;
    if (M >= 3 && a.n / 4 >= resident_warps) return launch_one<FMT, M, 4>(a, sm_count, pdl, s);
    if (a.n / 2 >= resident_warps) return launch_one<FMT, M, 2>(a, sm_count, pdl, s);
    return launch_one<FMT, M, 1>(a, sm_count, pdl, s);
}

template <int FMT> static cudaError_t launch_fmt(const GemvArgs &a, int sm_count, bool pdl, cudaStream_t s) {
    switch (a.rows) {
        case 1: return launch_m<FMT, 1>(a, sm_count, pdl, s);
        case 2: return launch_m<FMT, 2>(a, sm_count, pdl, s);
        case 3: return launch_m<FMT, 3>(a, sm_count, pdl, s);
        case 4: return launch_m<FMT, 4>(a, sm_count, pdl, s);
        case 5: return launch_m<FMT, 5>(a, sm_count, pdl, s);
        case 6: return launch_m<FMT, 6>(a, sm_count, pdl, s);
        case 7: return launch_m<FMT, 7>(a, sm_count, pdl, s);
        case 8: return launch_m<FMT, 8>(a, sm_count, pdl, s);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_qgemv(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream) {
    if (args.n == 0 || args.rows == 0) return cudaSuccess;
    switch (fmt) {
        case FMT_Q4K: return launch_fmt<FMT_Q4K>(args, sm_count, pdl, stream);
        case FMT_Q5K: return launch_fmt<FMT_Q5K>(args, sm_count, pdl, stream);
        case FMT_Q6K: return launch_fmt<FMT_Q6K>(args, sm_count, pdl, stream);
        case FMT_INT8: return launch_fmt<FMT_INT8>(args, sm_count, pdl, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_qgemv_moe(int fmt, const GemvArgs &args, int sm_count, bool pdl, cudaStream_t stream) {
    if (!args.ids || args.id_r == 0 || args.id_e == 0 || args.rows < 1 || args.rows > 8 || ((uintptr_t)args.w & 15) || (args.id_stride & 15))
        return cudaErrorInvalidValue;
    if ((uint64_t)args.rows * args.id_r > 65535) return cudaErrorInvalidValue;  // grid rows
    GemvArgs one = args;
    one.id_pairs = args.rows * args.id_r;
    one.rows = 1;
    one.m = 1;
    return launch_qgemv(fmt, one, sm_count, pdl, stream);
}

cudaError_t qgemv_init() { return cudaSuccess; }

}  // namespace lb

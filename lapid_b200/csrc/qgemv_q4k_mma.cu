// Q4_K decode GEMV for 2..8 activation rows on the warp-level int8 tensor-core instruction
// (arithmetic: see qgemv.cu; the integer dot products are the same, only the order of the f32
// sums over sub-blocks and k-chunks differs).
//
// With several activation rows the dp4a kernel is bound by instruction issue, not by
// memory: every weight byte is multiplied M times by scalar-per-lane instructions. Here one
// `mma.sync.m16n8k32.u8.s8` covers 16 weight rows x 32 k x 8 activation rows, so the integer
// work per weight byte no longer grows with M; what is left is the f32 scaling of each
// 32-element sub-block, which the format forces (every sub-block has its own weight scale and
// every activation group its own scale).
//
//  * A CTA works on tiles of 16*TILES weight rows. Its warps split K: warp w takes the k-chunks
//    (two super-blocks, 512 weights per row) w, w+WARPS, ... of every tile, so a matrix with few
//    rows still gives every SM work. Partial 16x8 tiles are summed in shared memory in warp
//    order (deterministic), one element per thread, and written with the epilogue.
//  * Weights reach the SM through per-warp rings of stages, each filled by ONE tensor-map copy
//    (TMA, `cp.async.bulk.tensor.2d`: a box of 16*TILES rows x 288 bytes of the packed matrix,
//    completion on an mbarrier); rows past the end of the matrix and the missing half of an
//    odd last k-chunk arrive as zeros. The row stride of 288 bytes makes the fragment loads
//    (64 bits per lane: words 2t and 2t+1 of a 32-byte half-pair, rows t/4) bank-conflict free.
//  * Within a sub-block the k order of an integer dot product is free as long as both operands
//    use the same one, so lane t of a row group takes weights 8t..8t+7 (one 64-bit load gives
//    the low nibbles of sub-block 2j and the high nibbles of 2j+1) and activations 8t..8t+7.
//    High nibbles are used in place (16*q, exact factor 1/16 folded into the scale).
//  * The pre-pass writes the int8 activations as tiles: per super-block, [sub-block][row][32]
//    quants, then the group scales as [sub-block pair][row pair][sub-block & 1][row & 1] (da) and the same
//    for d*sum(q) (bs), so a lane's B fragment is one 64-bit load and its scales are conflict-free 128-bit loads.
//  * The 6-bit scales and mins of a stage are decoded once per (row, super-block) by one lane and
//    passed through shared memory; a thread needs them for four rows.
//  * Every mbarrier wait is bounded; a wait that gives up sets the host-visible status word.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "kernels.h"
#include "tp_ll.cuh"

namespace lb {
namespace mm {

constexpr int STAGES = 2;
constexpr int ROWB = 2 * Q4K_BYTES;  // 288: two super-blocks of one weight row
constexpr int BAR_BYTES = 256;
constexpr int SC_STRIDE = 80;  // decoded scales of one (row, super-block): 16 floats, padded against bank conflicts

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
// x counts 32-bit elements of a row of the packed matrix (a multiple of 72, so 16-byte aligned), y rows
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     s32(dst)),
                 "l"((uint64_t)map), "r"(x), "r"(y), "r"(s32(bar))
                 : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < (1u << 22); spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(s32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// 16 weight rows (unsigned bytes) x 32 k x 8 activation rows (signed bytes). The accumulators
// start at the bit pattern of 1.5 * 2^23: the integer dot product (|dot| < 2^22) lands in the
// mantissa, so the result reinterpreted as f32 is 12582912 + dot and one exact addition
// replaces the int -> float conversion.
constexpr float MAGIC = 12582912.0f;
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0x4B400000));
}

// Two f32 lanes in one 64-bit register pair (Blackwell's packed f32 instructions).
__device__ __forceinline__ uint64_t pack2i(int lo, int hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}

__device__ __forceinline__ float scale_byte(uint32_t w, uint32_t sel, float d, float neg_d23) {
    return fmaf(d, __uint_as_float(__byte_perm(w, 0x4B000000u, sel)), neg_d23);
}

__host__ __device__ constexpr uint32_t act_block_bytes(uint32_t rows) { return 256 * rows + 512; }

template <int NG> struct WeightMapsT {
    CUtensorMap m[NG];  // packed weights of each member: [n rows][k/256 * 36 words], box 72 words x 16*TILES rows
};

// EARLY (GemvArgs::early of every member): the activations are older than the kernel in front of this one, so
// the kernel reads and computes without waiting for it, parks the tiles' results in shared memory and
// stores them after the dependency wait. Launched as ONE small CTA per SM, so that the kernels of
// consecutive launches share the SMs and the ramp-up of one hides behind the tail of the other.
constexpr int PEND_TILES = 8;
template <int WARPS, int TILES, int NG, bool EARLY = false>
__global__ void __launch_bounds__(WARPS * 32, 1)
qgemv_q4k_mma_kernel(const __grid_constant__ WeightMapsT<NG> maps, GemvGroupT<NG> grp) {
    constexpr int THREADS = WARPS * 32;
    constexpr int RPT = 16 * TILES;           // weight rows per tile
    constexpr int STAGE = RPT * ROWB;         // bytes per ring stage
    constexpr int ELEMS = RPT * 8;            // outputs per tile
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int gq = lane >> 2, t4 = lane & 3;
    const uint32_t M = grp.item[0].rows;
    const uint32_t nblk = grp.item[0].k / QK;
    const uint32_t iters = (nblk + 1) / 2;  // k-chunks per tile; warp w takes w, w + WARPS, ...
    const uint32_t ABLK = act_block_bytes(M);
    const uint32_t tasks = grp.task_end[grp.count - 1];
    auto locate = [&](uint32_t t, uint32_t &local) -> int {
        if constexpr (NG == 1) {
            local = t;
            return 0;
        }
        int i = 0;
        while (t >= grp.task_end[i]) i++;
        local = t - (i ? grp.task_end[i - 1] : 0);
        return i;
    };
    const uint32_t t_lo = (uint32_t)(((uint64_t)tasks * blockIdx.x) / gridDim.x);
    const uint32_t t_hi = (uint32_t)(((uint64_t)tasks * (blockIdx.x + 1)) / gridDim.x);

    uint64_t *bars = (uint64_t *)smem + warp * STAGES;
    uint8_t *ring = smem + BAR_BYTES + (size_t)warp * (STAGES * STAGE);
    uint8_t *scs = smem + BAR_BYTES + (size_t)WARPS * STAGES * STAGE + (size_t)warp * (32 * SC_STRIDE);
    float *red = (float *)(smem + BAR_BYTES + (size_t)WARPS * (STAGES * STAGE + 32 * SC_STRIDE));  // [2][WARPS][ELEMS]
    uint8_t *acts = (uint8_t *)(red + 2 * WARPS * ELEMS);

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < STAGES; s++) mbar_init(bars + s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();

    // producer cursor: (tile, k-chunk, ring slot); a warp without a k-chunk (iters < WARPS) never issues
    uint32_t pt = t_lo, pit = warp, pslot = 0;
    auto issue = [&]() {
        if (pt >= t_hi || (uint32_t)warp >= iters) return;
        if (lane == 0) {
            uint32_t local;
            const int item = locate(pt, local);
            mbar_expect_tx(bars + pslot, STAGE);  // the whole box counts, zero fill included
            tma_load_2d(ring + (size_t)pslot * STAGE, &maps.m[item], (int)(pit * (ROWB / 4)), (int)(local * RPT), bars + pslot);
        }
        pslot ^= 1;
        pit += WARPS;
        if (pit >= iters) {
            pit = warp;
            pt++;
        }
    };
    issue();
    issue();

    // early (GemvArgs::early): the activations are older than the kernel in front of this one, so they are
    // fetched, and the first tile computed, while that kernel still runs; only the stores wait for it
    constexpr bool early = EARLY;
    auto copy_acts = [&]() {
        const uint32_t chunks = nblk * ABLK / 16;
        for (int i = 0; i < grp.count; i++) {
            if (!grp.act_copy[i]) continue;
            const uint8_t *src = (const uint8_t *)grp.item[i].qa;
            uint8_t *dst = acts + grp.act_off[i];
            for (uint32_t c = threadIdx.x; c < chunks; c += THREADS)
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s32(dst + 16 * c)), "l"(src + 16 * (size_t)c) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (early) copy_acts();
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (!early) asm volatile("griddepcontrol.wait;" ::: "memory");
    bool waited = !early;

    __shared__ TpPushCtx tp_ctx;  // only the first member of a launch may push (tensor-parallel launches are never grouped)
    if (grp.item[0].tp && threadIdx.x == 0) tp_push_ctx_load(&tp_ctx, grp.item[0].tp);
    if (!early) copy_acts();
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // parked tiles (EARLY): [tile][ELEMS], each element written and later stored by the same thread
    float *pend = (float *)(acts + grp.act_bytes);
    uint32_t npend = 0;
    const uint32_t pend_first = t_lo;  // the CTA's tiles are consecutive; they are parked from its first one on
    auto flush_pending = [&]() {
        for (uint32_t q = 0; q < npend; q++) {
            uint32_t local;
            const int item = locate(pend_first + q, local);
            const GemvArgs &p = grp.item[item];
            for (uint32_t e = threadIdx.x; e < (uint32_t)ELEMS; e += THREADS) {
                float v = pend[q * ELEMS + e];
                const uint32_t el = e & 31, i = (e >> 5) & 3, tl = e >> 7;
                const uint32_t row = local * RPT + tl * 16 + (el >> 2) + ((i & 2) ? 8 : 0);
                const uint32_t r = 2 * (el & 3) + (i & 1);
                if (row < p.n && r < grp.item[0].rows) {
                    const uint32_t bt = r / p.m, ri = r % p.m;
                    if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)ri * p.ex_s1 + (int64_t)row * p.ex_s2];
                    p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)ri * p.out_rs + row] = v;
                }
            }
        }
        npend = 0;
    };

    const uint32_t colq = (uint32_t)gq < M ? gq : 0;        // activation row of this lane's B fragment
    const uint32_t cp = (uint32_t)(2 * t4) < M ? t4 : 0;    // activation row pair of this lane's C fragment
    const uint64_t neg_magic = pack2(-MAGIC, -MAGIC);
    bool healthy = true;
    uint32_t cslot = 0, cpar = 0, par = 0;
    for (uint32_t t = t_lo; t < t_hi; t++, par ^= 1) {
        uint32_t local;
        const int item = locate(t, local);
        const GemvArgs &p = grp.item[item];
        const uint8_t *iacts = acts + grp.act_off[item];
        float acc[TILES][4];
#pragma unroll
        for (int tl = 0; tl < TILES; tl++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[tl][i] = 0.0f;

        for (uint32_t it = warp; it < iters; it += WARPS) {
            if (healthy && !mbar_wait(bars + cslot, cpar)) {
                healthy = false;
                if (lane == 0 && grp.item[0].status) atomicOr(grp.item[0].status, 1);
            }
            const uint8_t *stage = ring + (size_t)cslot * STAGE;
            const uint32_t nb = min(2u, nblk - 2 * it);
            // ---- decode the 6-bit scales and mins: one lane per (row, super-block)
            auto decode = [&](uint32_t rr, uint32_t b, uint32_t slot) {
                const uint4 h = *(const uint4 *)(stage + rr * ROWB + b * Q4K_BYTES);
                const float d = half_bits_to_float(h.x & 0xffff), dmin = -half_bits_to_float(h.x >> 16);
                const float nd = d * -8388608.0f, ndmin = dmin * -8388608.0f;
                const uint32_t w0 = h.y, w1 = h.z, w2 = h.w;
                const uint32_t sc_lo = w0 & 0x3F3F3F3Fu, mn_lo = w1 & 0x3F3F3F3Fu;
                const uint32_t sc_hi = (w2 & 0x0F0F0F0Fu) | (((w0 >> 6) & 0x03030303u) << 4);
                const uint32_t mn_hi = ((w2 >> 4) & 0x0F0F0F0Fu) | (((w1 >> 6) & 0x03030303u) << 4);
                float w[16];
#pragma unroll
                for (int s = 0; s < 8; s++) {
                    const uint32_t sel = 0x7440u + (s & 3);
                    const float sc = scale_byte(s < 4 ? sc_lo : sc_hi, sel, d, nd);
                    w[s] = (s & 1) ? sc * 0.0625f : sc;                             // d * sc (high nibbles: / 16)
                    w[8 + s] = scale_byte(s < 4 ? mn_lo : mn_hi, sel, dmin, ndmin);  // -dmin * m
                }
                float4 *dst = (float4 *)(scs + slot * SC_STRIDE);
                dst[0] = make_float4(w[0], w[1], w[2], w[3]);
                dst[1] = make_float4(w[4], w[5], w[6], w[7]);
                dst[2] = make_float4(w[8], w[9], w[10], w[11]);
                dst[3] = make_float4(w[12], w[13], w[14], w[15]);
            };
            if (healthy) {
#pragma unroll
                for (int ph = 0; ph < (TILES == 2 ? 2 : 1); ph++) {
                    if constexpr (TILES == 2) {
                        if ((uint32_t)ph < nb) decode(lane, ph, lane);
                    } else {
                        if ((uint32_t)(lane >> 4) < nb) decode(lane & 15, lane >> 4, lane);
                    }
                    __syncwarp();
#pragma unroll
                    for (int bb = 0; bb < (TILES == 2 ? 1 : 2); bb++) {
                        const uint32_t b = TILES == 2 ? ph : bb;
                        if (b >= nb) break;
                        const uint8_t *ab = iacts + (size_t)(2 * it + b) * ABLK;
                        const float4 *dsp = (const float4 *)(ab + 256 * M) + cp;  // scales: [sub-block pair][row pair][sub-block & 1][row & 1]
                        ulonglong2 dav[4];  // {da[c0], da[c1]} of sub-blocks 2i, 2i + 1
                        float4 bsv[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            dav[i] = ((const ulonglong2 *)dsp)[4 * i];
                            bsv[i] = dsp[16 + 4 * i];
                        }
                        const float *bs = (const float *)bsv;  // [sub-block][2]
                        float4 wv[TILES][2][4];  // [tile][row half][W1 0..3, W1 4..7, W2 0..3, W2 4..7]
#pragma unroll
                        for (int tl = 0; tl < TILES; tl++)
#pragma unroll
                            for (int hf = 0; hf < 2; hf++) {
                                const uint32_t rr = tl * 16 + hf * 8 + gq;
                                const uint32_t slot = TILES == 2 ? rr : b * 16 + rr;
                                const float4 *src = (const float4 *)(scs + slot * SC_STRIDE);
#pragma unroll
                                for (int i = 0; i < 4; i++) wv[tl][hf][i] = src[i];
                            }
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const uint2 blo = *(const uint2 *)(ab + (2 * j) * (M * 32) + colq * 32 + 8 * t4);
                            const uint2 bhi = *(const uint2 *)(ab + (2 * j + 1) * (M * 32) + colq * 32 + 8 * t4);
#pragma unroll
                            for (int tl = 0; tl < TILES; tl++) {
                                const uint8_t *wrow = stage + (tl * 16 + gq) * ROWB + b * Q4K_BYTES + 16 + j * 32 + 8 * t4;
                                const uint2 wa = *(const uint2 *)wrow, wb = *(const uint2 *)(wrow + 8 * ROWB);
                                int cl[4], ch[4];
                                mma_u8s8(cl, wa.x & 0x0F0F0F0Fu, wb.x & 0x0F0F0F0Fu, wa.y & 0x0F0F0F0Fu, wb.y & 0x0F0F0F0Fu, blo.x, blo.y);
                                mma_u8s8(ch, wa.x & 0xF0F0F0F0u, wb.x & 0xF0F0F0F0u, wa.y & 0xF0F0F0F0u, wb.y & 0xF0F0F0F0u, bhi.x, bhi.y);
                                // int -> f32 and the activation scale on packed f32x2: the two outputs
                                // of a row are one register pair, and so are their activation scales
                                float gl[4], gh[4];
                                unpack2(mul2(add2(pack2i(cl[0], cl[1]), neg_magic), dav[j].x), gl[0], gl[1]);
                                unpack2(mul2(add2(pack2i(cl[2], cl[3]), neg_magic), dav[j].x), gl[2], gl[3]);
                                unpack2(mul2(add2(pack2i(ch[0], ch[1]), neg_magic), dav[j].y), gh[0], gh[1]);
                                unpack2(mul2(add2(pack2i(ch[2], ch[3]), neg_magic), dav[j].y), gh[2], gh[3]);
#pragma unroll
                                for (int i = 0; i < 4; i++) {
                                    const float *w = (const float *)wv[tl][i >> 1];
                                    const int c = i & 1;
                                    float a = acc[tl][i];
                                    a = fmaf(gl[i], w[2 * j], a);
                                    a = fmaf(w[8 + 2 * j], bs[(2 * j) * 2 + c], a);
                                    a = fmaf(gh[i], w[2 * j + 1], a);
                                    a = fmaf(w[8 + 2 * j + 1], bs[(2 * j + 1) * 2 + c], a);
                                    acc[tl][i] = a;
                                }
                            }
                        }
                    }
                    __syncwarp();  // the scale scratch is rewritten by the next phase
                }
            }
            __syncwarp();  // every lane is done reading the slot before it is refilled
            issue();
            cslot ^= 1;
            if (cslot == 0) cpar ^= 1;
        }

        // ---- sum the warps' partial tiles (warp order) and store: one output per thread
        float *mine = red + ((size_t)par * WARPS + warp) * ELEMS;
#pragma unroll
        for (int tl = 0; tl < TILES; tl++)
#pragma unroll
            for (int i = 0; i < 4; i++) mine[(tl * 4 + i) * 32 + lane] = acc[tl][i];
        __syncthreads();  // the buffer of the other parity is free again once every warp got here
        if (EARLY && !waited) {  // park the tile: nothing is written before the kernel in front has completed
            for (uint32_t e = threadIdx.x; e < (uint32_t)ELEMS; e += THREADS) {
                const float *src = red + (size_t)par * WARPS * ELEMS + e;
                float v = src[0];
#pragma unroll
                for (int w = 1; w < WARPS; w++) v += src[(size_t)w * ELEMS];
                pend[npend * ELEMS + e] = v;
            }
            if (++npend == PEND_TILES) {
                asm volatile("griddepcontrol.wait;" ::: "memory");
                waited = true;
                flush_pending();
            }
            continue;
        }
        for (uint32_t e = threadIdx.x; e < (uint32_t)ELEMS; e += THREADS) {
            const float *src = red + (size_t)par * WARPS * ELEMS + e;
            float v = src[0];
#pragma unroll
            for (int w = 1; w < WARPS; w++) v += src[(size_t)w * ELEMS];
            const uint32_t el = e & 31, i = (e >> 5) & 3, tl = e >> 7;
            const uint32_t row = local * RPT + tl * 16 + (el >> 2) + ((i & 2) ? 8 : 0);
            const uint32_t r = 2 * (el & 3) + (i & 1);
            if (row < p.n && r < M) {
                const uint32_t bt = r / p.m, ri = r % p.m;
                if (p.extra && !p.epi.n) v += p.extra[p.ex_off + (int64_t)bt * p.ex_s0 + (int64_t)ri * p.ex_s1 + (int64_t)row * p.ex_s2];
                if (p.tp) tp_push_value(&tp_ctx, (uint64_t)r * p.n + row, v);  // row-parallel partial: to every rank
                else p.out[p.out_off + (uint64_t)bt * p.out_bs + (uint64_t)ri * p.out_rs + row] = v;
            }
        }
    }
    if (!waited) {  // (a CTA without a tile must not let the grid end early either)
        asm volatile("griddepcontrol.wait;" ::: "memory");
        if constexpr (EARLY) flush_pending();
    }
}

struct Config {
    int warps, tiles;
};
static const Config CONFIGS[] = {{8, 2}, {8, 1}, {4, 1}};
static int g_force_config = -1;

static size_t early_pend_bytes(int tiles) { return (size_t)PEND_TILES * 16 * tiles * 8 * 4; }
static size_t fixed_smem(const Config &c) {
    const size_t stage = (size_t)16 * c.tiles * ROWB;
    return BAR_BYTES + (size_t)c.warps * (STAGES * stage + 32 * SC_STRIDE) + (size_t)2 * c.warps * 16 * c.tiles * 8 * 4;
}

// distinct activation operands of the group -> offsets into the shared-memory copy
static void plan_acts(GemvGroup &g) {
    const uint32_t bytes = (g.item[0].k / QK) * act_block_bytes(g.item[0].rows);
    g.act_bytes = 0;
    for (int i = 0; i < g.count; i++) {
        g.act_copy[i] = 1;
        for (int j = 0; j < i; j++)
            if (g.item[j].qa == g.item[i].qa) {
                g.act_off[i] = g.act_off[j];
                g.act_copy[i] = 0;
                break;
            }
        if (g.act_copy[i]) {
            g.act_off[i] = g.act_bytes;
            g.act_bytes += bytes;
        }
    }
}

static int pick_config(size_t act_bytes) {
    if (g_force_config >= 0) return fixed_smem(CONFIGS[g_force_config]) + act_bytes <= 227 * 1024 - 256 ? g_force_config : -1;
    // small activation tiles: three of the small CTAs per SM beat one large one (more tiles in
    // flight, shorter barriers); otherwise the largest layout that fits
    if (3 * (fixed_smem(CONFIGS[2]) + act_bytes + 1024) <= 227 * 1024) return 2;
    for (int i = 0; i < (int)(sizeof(CONFIGS) / sizeof(CONFIGS[0])); i++)
        if (fixed_smem(CONFIGS[i]) + act_bytes <= 227 * 1024 - 256) return i;
    return -1;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
    }
    return fn;
}

// A tensor map depends only on (address, n, k, box rows): the last few are remembered, a decode
// loop asks for the same handful every token.
static bool weight_map(const GemvArgs &a, uint32_t box_rows, CUtensorMap &out) {
    struct Entry {
        const void *w;
        uint32_t n, k, rows;
        CUtensorMap map;
    };
    static Entry cache[64];
    static int used = 0, next = 0;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    for (int i = 0; i < used; i++)
        if (cache[i].w == a.w && cache[i].n == a.n && cache[i].k == a.k && cache[i].rows == box_rows) {
            out = cache[i].map;
            return true;
        }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    const uint32_t nblk = a.k / QK;
    cuuint64_t dims[2] = {(cuuint64_t)nblk * (Q4K_BYTES / 4), a.n};
    cuuint64_t strides[1] = {(cuuint64_t)nblk * Q4K_BYTES};
    cuuint32_t box[2] = {ROWB / 4, box_rows};
    cuuint32_t es[2] = {1, 1};
    if (enc(&out, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void *)a.w, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    Entry &e = cache[used < 64 ? used++ : (next = (next + 1) % 64)];
    e.w = a.w;
    e.n = a.n;
    e.k = a.k;
    e.rows = box_rows;
    e.map = out;
    return true;
}

template <int WARPS, int TILES, int NG, bool EARLY = false>
static cudaError_t launch_n(GemvGroupT<NG> &g, int sm_count, bool pdl, cudaStream_t stream) {
    auto kern = qgemv_q4k_mma_kernel<WARPS, TILES, NG, EARLY>;
    uint32_t tasks = 0;
    WeightMapsT<NG> maps;
    for (int i = 0; i < g.count; i++) {
        tasks += (g.item[i].n + 16 * TILES - 1) / (16 * TILES);
        g.task_end[i] = tasks;
        if (!weight_map(g.item[i], 16 * TILES, maps.m[i])) return cudaErrorNotSupported;
    }
    for (int i = g.count; i < NG; i++) maps.m[i] = maps.m[0];
    const size_t smem = fixed_smem(Config{WARPS, TILES}) + g.act_bytes + (EARLY ? early_pend_bytes(TILES) : 0);
    static DynamicSmemOptIn opted;
    if (cudaError_t e = opted.raise((const void *)kern, smem); e != cudaSuccess) return e;
    uint32_t per_sm = (uint32_t)((227 * 1024) / (smem + 1024));  // shared memory is what limits residency
    if (EARLY) per_sm = 1;  // the other slots belong to the launches around this one
    uint32_t grid = (uint32_t)sm_count * (per_sm ? per_sm : 1);
    if (grid > tasks) grid = tasks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, maps, g);
}

template <int WARPS, int TILES, bool EARLY = false>
static cudaError_t launch_cfg(GemvGroup &g, int sm_count, bool pdl, cudaStream_t stream) {
    if (g.count > 1) return launch_n<WARPS, TILES, GEMV_GROUP_MAX, EARLY>(g, sm_count, pdl, stream);
    GemvSingle one;  // a lone launch passes a sixth of the parameter bytes
    one.item[0] = g.item[0];
    one.act_off[0] = g.act_off[0];
    one.act_copy[0] = g.act_copy[0];
    one.count = 1;
    one.act_bytes = g.act_bytes;
    return launch_n<WARPS, TILES, 1, EARLY>(one, sm_count, pdl, stream);
}

}  // namespace mm

void qgemv_q4k_mma_set_config(int index) { mm::g_force_config = index < 0 || index > 2 ? -1 : index; }

size_t qgemv_q4k_mma_act_bytes(uint32_t rows, uint32_t k) { return (size_t)(k / QK) * mm::act_block_bytes(rows); }

bool qgemv_q4k_mma_shape_ok(uint32_t rows, uint32_t k) {
    if (rows < 1 || rows > 8 || k % QK != 0 || k < QK || !mm::encode_fn()) return false;
    return mm::pick_config(qgemv_q4k_mma_act_bytes(rows, k)) >= 0;
}

// Whether the group (items [0, count)) can run as one launch.
bool qgemv_q4k_mma_group_fits(GemvGroup &g) {
    mm::plan_acts(g);
    return mm::pick_config(g.act_bytes) >= 0;
}

// `ws` set: launches that the balanced-stream kernel (qgemv_kq_stream.cu) runs faster go there. Measured on B200
// (M = 4 and 8, cold HBM): it wins on matrices with at least two of its 128-row units per SM when the launch may
// run ahead of its predecessor (every member early: 8.5 / 8.2 us against 10.0 / 13.2 on 14336 x 4096 and
// 4096 x 14336 at M = 8), and, for dependent launches, from seven rows on (M = 8: 10.2 / 11.6 against 11.3 / 13.2 us;
// at K = 14336 this kernel's activation copy then leaves room for only four warps per SM) and from eight units
// per SM on. Smaller matrices and the other dependent launches stay here: the stream kernel's hand-over of
// partial tiles between CTAs costs about a microsecond at its end.
cudaError_t launch_qgemv_q4k_mma(GemvGroup &g, int sm_count, bool pdl, cudaStream_t stream, StreamWs *ws) {
    if (g.count < 1 || g.count > GEMV_GROUP_MAX) return cudaErrorInvalidValue;
    mm::plan_acts(g);
    if (ws && mm::g_force_config < 0) {
        bool early = pdl;
        uint64_t units = 0;
        for (int i = 0; i < g.count; i++) {
            early = early && g.item[i].early != 0 && g.item[i].tp == nullptr;
            units += (uint64_t)((g.item[i].n + 127) / 128) * ((g.item[i].k / QK + 1) / 2);
        }
        const bool cramped = mm::fixed_smem(mm::CONFIGS[1]) + g.act_bytes > 227 * 1024 - 256;
        if ((units >= 2 * (uint64_t)sm_count && (early || cramped || g.item[0].rows >= 7)) || units >= 8 * (uint64_t)sm_count)
            return launch_qgemv_kq_stream(FMT_Q4K, g, *ws, sm_count, pdl, stream);
    }
    {   // every member early, no tensor-parallel push, and two of the small CTAs fit on an SM: the early instantiation
        bool early = pdl && mm::g_force_config < 0;
        for (int i = 0; i < g.count; i++) early = early && g.item[i].early != 0 && g.item[i].tp == nullptr;
        const size_t smem = mm::fixed_smem(mm::CONFIGS[2]) + g.act_bytes + mm::early_pend_bytes(1);
        if (early && 2 * (smem + 1024) <= 227 * 1024) return mm::launch_cfg<4, 1, true>(g, sm_count, pdl, stream);
    }
    switch (mm::pick_config(g.act_bytes)) {
        case 0: return mm::launch_cfg<8, 2>(g, sm_count, pdl, stream);
        case 1: return mm::launch_cfg<8, 1>(g, sm_count, pdl, stream);
        case 2: return mm::launch_cfg<4, 1>(g, sm_count, pdl, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace lb
